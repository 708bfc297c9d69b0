"""Byte-level tokenizer with the chat specials the agent loop needs.

The framework ships no vocabulary files; a checkpoint directory that carries a ``tokenizer.json`` is read by the model
io layer, everything else (tests, the synthetic recipe, the benchmark) uses this one: ids 0..255 are bytes, the
specials follow. A vocabulary larger than the tokenizer's is fine (the tail ids are never produced by ``encode``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

SPECIALS = ["<|pad|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<|vision_start|>", "<|vision_end|>",
            "<|image_pad|>", "<|mask|>", "<|eos|>"]


@dataclass
class ByteTokenizer:
    vocab_size: int = 256 + len(SPECIALS)

    def __post_init__(self) -> None:
        self.special_ids = {s: 256 + i for i, s in enumerate(SPECIALS)}
        self.id_to_special = {v: k for k, v in self.special_ids.items()}
        self.pad_id, self.eos_id = self.special_ids["<|pad|>"], self.special_ids["<|im_end|>"]
        self.image_pad_id, self.mask_id = self.special_ids["<|image_pad|>"], self.special_ids["<|mask|>"]

    def encode(self, text: str) -> list[int]:
        out: list[int] = []
        i = 0
        while i < len(text):
            if text[i] == "<":
                for s, sid in self.special_ids.items():
                    if text.startswith(s, i):
                        out.append(sid)
                        i += len(s)
                        break
                else:
                    out.extend(text[i].encode("utf-8"))
                    i += 1
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def decode(self, ids: list[int], skip_special: bool = False) -> str:
        parts: list[str] = []
        buf = bytearray()
        for t in ids:
            if t < 256:
                buf.append(t)
                continue
            if buf:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if t in self.id_to_special and not skip_special:
                parts.append(self.id_to_special[t])
        if buf:
            parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    # -- chat template (the one the agent loop renders turn by turn) --------------------------------------------------
    def render_turn(self, role: str, text: str, images: int = 0, image_tokens: int = 0, labels: Optional[list[str]] = None) -> list[int]:
        """``<|im_start|>role\\n`` text [vision blocks] ``<|im_end|>\\n``; an image is a run of pad ids between markers. With
        ``labels`` (one per image) every image follows a line ``[label]`` of its own, so the model reads which camera a picture
        is from right before it (upstream: pear/envs/tool.py:114-127)."""
        ids = [self.special_ids["<|im_start|>"]] + self.encode(role + "\n") + self.encode(text)
        for i in range(images):
            if labels is not None:
                ids += self.encode(f"\n[{labels[i]}]\n")
            ids += [self.special_ids["<|vision_start|>"]] + [self.image_pad_id] * image_tokens + [self.special_ids["<|vision_end|>"]]
        return ids + [self.special_ids["<|im_end|>"]] + self.encode("\n")

    def generation_prompt(self) -> list[int]:
        return [self.special_ids["<|im_start|>"]] + self.encode("assistant\n")

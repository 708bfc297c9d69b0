"""Byte-level tokenizer with the chat specials the agent loop needs.

The framework ships no vocabulary files; a checkpoint directory that carries a ``tokenizer.json`` is read by
``HFTokenizer`` (``load_tokenizer`` picks), everything else (presets, tests, the synthetic recipe, the benchmark) uses the byte
tokenizer: ids 0..255 are bytes, the specials follow. A vocabulary larger than the tokenizer's is fine (the tail ids are never produced by ``encode``).
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
            n = image_tokens[i] if isinstance(image_tokens, (list, tuple)) else image_tokens  # (pictures of different sizes: one count each)
            ids += [self.special_ids["<|vision_start|>"]] + [self.image_pad_id] * n + [self.special_ids["<|vision_end|>"]]
        return ids + [self.special_ids["<|im_end|>"]] + self.encode("\n")

    def generation_prompt(self) -> list[int]:
        return [self.special_ids["<|im_start|>"]] + self.encode("assistant\n")


class HFTokenizer:
    """A checkpoint directory's ``tokenizer.json`` (read with the ``tokenizers`` package) behind the interface of
    :class:`ByteTokenizer`: ``encode`` / ``decode`` / ``render_turn`` / ``generation_prompt`` and the ids of the chat and vision
    specials, which must exist in the vocabulary under the family's names (``<|im_start|>``, ``<|im_end|>``,
    ``<|vision_start|>``, ``<|vision_end|>``, ``<|image_pad|>``). Upstream takes the tokenizer from the model directory through
    its serving stack; the template is the family's ChatML form."""

    REQUIRED = ("<|im_start|>", "<|im_end|>")
    OPTIONAL = ("<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<think>", "</think>", "<|endoftext|>")

    def __init__(self, directory: str):
        import json
        import os

        from tokenizers import Tokenizer

        path = os.path.join(directory, "tokenizer.json")
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        self.special_ids: dict[str, int] = {}
        for name in self.REQUIRED + self.OPTIONAL:
            i = self.tk.token_to_id(name)
            if i is None and name in self.REQUIRED:
                raise KeyError(f"{path}: the vocabulary has no {name} token (the chat template needs it)")
            if i is not None:
                self.special_ids[name] = i
        self.id_to_special = {v: k for k, v in self.special_ids.items()}
        self.eos_id = self.special_ids["<|im_end|>"]
        self.pad_id = self.special_ids.get("<|endoftext|>", self.eos_id)
        self.image_pad_id = self.special_ids.get("<|image_pad|>", -1)
        cfg = os.path.join(directory, "generation_config.json")
        self.extra_stop_ids: tuple[int, ...] = ()
        if os.path.exists(cfg):
            with open(cfg) as f:
                eos = json.load(f).get("eos_token_id", [])
            self.extra_stop_ids = tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]) if int(e) != self.eos_id)

    def encode(self, text: str) -> list[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def decode(self, ids: list[int], skip_special: bool = False) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special)

    def render_turn(self, role: str, text: str, images: int = 0, image_tokens: int = 0, labels: Optional[list[str]] = None) -> list[int]:
        ids = [self.special_ids["<|im_start|>"]] + self.encode(role + "\n") + self.encode(text)
        if images and self.image_pad_id < 0:
            raise KeyError("the vocabulary has no <|image_pad|> token: this tokenizer cannot render pictures")
        for i in range(images):
            if labels is not None:
                ids += self.encode(f"\n[{labels[i]}]\n")
            n = image_tokens[i] if isinstance(image_tokens, (list, tuple)) else image_tokens
            ids += [self.special_ids["<|vision_start|>"]] + [self.image_pad_id] * n + [self.special_ids["<|vision_end|>"]]
        return ids + [self.special_ids["<|im_end|>"]] + self.encode("\n")

    def generation_prompt(self) -> list[int]:
        return [self.special_ids["<|im_start|>"]] + self.encode("assistant\n")


def load_tokenizer(model_path: Optional[str] = None):
    """The tokenizer of a model: the directory's ``tokenizer.json`` when it has one, else the byte tokenizer (presets, tests)."""
    import os

    if model_path and not str(model_path).startswith("preset:") and os.path.exists(os.path.join(str(model_path), "tokenizer.json")):
        return HFTokenizer(str(model_path))
    return ByteTokenizer()

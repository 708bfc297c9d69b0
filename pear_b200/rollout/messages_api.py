"""The Messages form of the model server: ``GET /v1/models``, ``POST /v1/messages`` (whole answers, and event streams whose text deltas go out as the engine produces tokens) and
``POST /v1/messages/count_tokens``, for agent CLIs that speak it.

Upstream's agent harness sits between such a CLI and a serving stack that offers these three routes (the harness reads the
served model's context from ``/v1/models``, sizes every request with ``count_tokens`` and relays ``/v1/messages``:
pear/deploy/harness/claude_code/main.py:60-77, proxy.py:173-230, 285-316). Here the rollout replica's own HTTP application
offers them, over the same engine, prefix cache and tokenizer as its other routes, so ``deploy/harness`` can front a replica
directly.

A message's content is a string or a list of blocks. ``text`` blocks are concatenated; ``image`` blocks (base64 sources) become
runs of picture placeholders whose rows a vision encoder computes, when the server was given one (``vision=``); without an
encoder a request with pictures is refused rather than answered without seeing them.
"""

from __future__ import annotations

import base64
import io
import json
import uuid
from typing import Any, Iterator, Optional

import numpy as np
import torch

from .engine import FinishReason, SamplingParams

END_TURN, MAX_TOKENS = "end_turn", "max_tokens"


def blocks_of(content: Any) -> list[dict]:
    """A message's content as a list of blocks (a string is one text block)."""
    if isinstance(content, str):
        return [{"type": "text", "text": content}]
    return [b if isinstance(b, dict) else {"type": "text", "text": str(b)} for b in (content or [])]


def system_text(system: Any) -> str:
    return "".join(b.get("text", "") for b in blocks_of(system) if b.get("type", "text") == "text") if system else ""


def picture_of(block: dict) -> np.ndarray:
    """uint8 [H, W, 3] of an image block with a base64 source."""
    from PIL import Image

    src = block.get("source") or {}
    if src.get("type") != "base64":
        raise ValueError("image blocks need a base64 source")
    return np.array(Image.open(io.BytesIO(base64.b64decode(src["data"]))).convert("RGB"), dtype=np.uint8)  # (a writable copy)


class MessagesFrontend:
    """Renders Messages requests for one server and shapes its answers."""

    def __init__(self, server, tokenizer, vision=None, max_model_len: Optional[int] = None):
        self.server, self.tokenizer, self.vision = server, tokenizer, vision
        if max_model_len is None:  # what the paged cache holds of one sequence at most
            cfg = server.engine.cfg
            max_model_len = cfg.num_blocks * cfg.block_size
        self.max_model_len = int(max_model_len)

    # -- prompt -----------------------------------------------------------------------------------------------------------
    def render(self, body: dict, with_rows: bool = True):
        """(token ids, embeds or None, mask or None) of a request: the system prompt, every message as one turn of the chat
        template with its pictures' placeholders after its text, and the opened assistant header."""
        tok = self.tokenizer
        ids: list[int] = []
        pictures: list[np.ndarray] = []
        sys_text = system_text(body.get("system"))
        if sys_text:
            ids += tok.render_turn("system", sys_text)
        for m in body.get("messages", []):
            text, frames = "", []
            for b in blocks_of(m.get("content")):
                kind = b.get("type", "text")
                if kind == "text":
                    text += b.get("text", "")
                elif kind == "image":
                    if self.vision is None:
                        raise ValueError("this server has no vision encoder: it cannot read image blocks")
                    frames.append(picture_of(b))
                elif kind == "tool_result":  # what a tool answered, as text of the user's turn
                    text += system_text(b.get("content")) if not isinstance(b.get("content"), str) else b["content"]
                elif kind == "tool_use":  # the assistant's own earlier call, as it wrote it
                    text += json.dumps({"name": b.get("name"), "arguments": b.get("input", {})})
            counts = [self.vision.grid(f)[0] * self.vision.grid(f)[1] for f in frames]
            ids += tok.render_turn(str(m.get("role", "user")), text, images=len(frames), image_tokens=counts) if frames else tok.render_turn(str(m.get("role", "user")), text)
            pictures += frames
        ids += tok.generation_prompt()
        if not pictures or not with_rows:
            return ids, None, None
        rows = np.concatenate([np.asarray(r, dtype=np.float32).reshape(-1, np.asarray(r).shape[-1]) for r in self.vision.encode(pictures)], 0)
        mask = torch.tensor([t == tok.image_pad_id for t in ids])
        if int(mask.sum()) != rows.shape[0]:
            raise ValueError(f"{int(mask.sum())} picture placeholders for {rows.shape[0]} encoded rows")
        emb = torch.zeros(len(ids), rows.shape[1])
        emb[mask] = torch.from_numpy(rows)
        return ids, emb, mask

    # -- answers ----------------------------------------------------------------------------------------------------------
    def count(self, body: dict) -> dict:
        return {"input_tokens": len(self.render(body, with_rows=False)[0])}

    def prepare(self, body: dict):
        """(ids, embeds, mask, sampling parameters, stop ids, session) of a request; refuses a prompt that leaves no room."""
        tok = self.tokenizer
        ids, emb, mask = self.render(body)
        room = self.max_model_len - len(ids)
        if room <= 0:
            raise OverflowError(f"prompt is too long: {len(ids)} tokens > {self.max_model_len} maximum")
        stops = (tok.eos_id,) + tuple(getattr(tok, "extra_stop_ids", ()))
        params = SamplingParams(max_tokens=min(int(body.get("max_tokens") or 256), room), temperature=float(body.get("temperature", 1.0)),
                                top_p=float(body.get("top_p", 1.0)), top_k=int(body.get("top_k", -1) or -1), stop_token_ids=stops)
        return ids, emb, mask, params, stops, (body.get("metadata") or {}).get("user_id")

    def message(self, body: dict, n_prompt: int, output: list, finish, cached: int, stops) -> dict:
        text = self.tokenizer.decode([t for t in output if t not in stops], skip_special=True)
        usage = {"input_tokens": n_prompt - cached, "cache_read_input_tokens": cached, "cache_creation_input_tokens": 0, "output_tokens": len(output)}
        return {"id": f"msg_{uuid.uuid4().hex[:24]}", "type": "message", "role": "assistant", "model": body.get("model", self.server.name),
                "content": [{"type": "text", "text": text}], "stop_reason": END_TURN if finish == FinishReason.STOP else MAX_TOKENS,
                "stop_sequence": None, "usage": usage}

    def run(self, body: dict):
        ids, emb, mask, params, stops, session = self.prepare(body)
        req = self.server.generate(ids, params, session=session, embeds=emb, embeds_mask=mask)
        return self.message(body, len(ids), req.output, req.finish, int(getattr(req, "cached_prefix", 0)), stops)

    def can_stream(self) -> bool:
        """Whether the server hands out the live request with its future (an in-process replica does; a lock-step leader
        creates the request later, on every rank, and the deploy engine decodes a request whole)."""
        return hasattr(self.server, "submit") and not hasattr(self.server, "channel") and hasattr(self.server, "futures")

    def stream(self, prepared, body: dict, poll_s: float = 0.005) -> Iterator[bytes]:
        """The answer as events while it is produced: the text decoded so far, minus what was sent, after every engine step
        that added tokens (text that ends inside a multi-byte character waits for the rest). A request the engine aborts for a
        weight sync goes on as a new request over the prompt plus what was produced."""
        import time as _time

        ids, emb, mask, params, stops, session = prepared
        tok = self.tokenizer
        produced: list[int] = []
        sent, cached, finish, started = "", 0, None, False
        head = self.message(body, len(ids), [], None, 0, stops)
        while True:
            left = params.max_tokens - len(produced)
            prompt = ids + produced
            e, m = emb, mask
            if emb is not None and produced:  # the rows of the tokens produced so far are ordinary embeddings
                e = torch.cat([emb, torch.zeros(len(produced), emb.shape[1])])
                m = torch.cat([mask, torch.zeros(len(produced), dtype=torch.bool)])
            import dataclasses

            fut = self.server.submit(prompt, dataclasses.replace(params, max_tokens=left), session, e, m)
            req = fut.request
            while True:
                done = fut.done()
                out = produced + list(req.output)
                if not started and (out or done):
                    cached = int(getattr(req, "cached_prefix", 0))
                    head["usage"].update(input_tokens=len(ids) - cached, cache_read_input_tokens=cached)
                    yield self.frame("message_start", {"message": {**head, "content": [], "stop_reason": None}})
                    yield self.frame("content_block_start", {"index": 0, "content_block": {"type": "text", "text": ""}})
                    started = True
                text = tok.decode([t for t in out if t not in stops], skip_special=True)
                if not done and text.endswith("\ufffd"):
                    text = text.rstrip("\ufffd")  # an unfinished character: wait for its remaining bytes
                if len(text) > len(sent) and text.startswith(sent):
                    yield self.frame("content_block_delta", {"index": 0, "delta": {"type": "text_delta", "text": text[len(sent):]}})
                    sent = text
                if done:
                    break
                _time.sleep(poll_s)
            req = fut.result()
            produced += list(req.output)
            finish = req.finish
            if finish != FinishReason.ABORTED or len(produced) >= params.max_tokens:
                break
            while self.server.engine.paused and not self.server.stop_flag:
                _time.sleep(poll_s)
        yield self.frame("content_block_stop", {"index": 0})
        yield self.frame("message_delta", {"delta": {"stop_reason": END_TURN if finish == FinishReason.STOP else MAX_TOKENS, "stop_sequence": None},
                                           "usage": {"output_tokens": len(produced)}})
        yield self.frame("message_stop", {})

    @staticmethod
    def frame(kind: str, data: dict) -> bytes:
        return f"event: {kind}\ndata: {json.dumps({'type': kind, **data})}\n\n".encode()

    @staticmethod
    def events(message: dict) -> Iterator[bytes]:
        """A whole answer as the event stream of the Messages form (servers that cannot hand out a live request: the text
        arrives as one delta between the opening and closing events a client's parser expects)."""
        frame = MessagesFrontend.frame

        text = message["content"][0]["text"]
        head = {**message, "content": [], "stop_reason": None, "usage": {**message["usage"], "output_tokens": 0}}
        yield frame("message_start", {"message": head})
        yield frame("content_block_start", {"index": 0, "content_block": {"type": "text", "text": ""}})
        if text:
            yield frame("content_block_delta", {"index": 0, "delta": {"type": "text_delta", "text": text}})
        yield frame("content_block_stop", {"index": 0})
        yield frame("message_delta", {"delta": {"stop_reason": message["stop_reason"], "stop_sequence": None},
                                      "usage": {"output_tokens": message["usage"]["output_tokens"]}})
        yield frame("message_stop", {})


def error_body(kind: str, message: str) -> dict:
    return {"type": "error", "error": {"type": kind, "message": message}}


def register(app, server, tokenizer, vision=None, max_model_len: Optional[int] = None) -> Optional[MessagesFrontend]:
    """Add the three routes to a replica's FastAPI application (nothing without a tokenizer: the form is text in, text out)."""
    if tokenizer is None:
        return None
    from fastapi.responses import JSONResponse, StreamingResponse

    front = MessagesFrontend(server, tokenizer, vision, max_model_len)

    @app.get("/v1/models")
    def models() -> dict:
        return {"object": "list", "data": [{"id": server.name, "object": "model", "max_model_len": front.max_model_len}]}

    @app.post("/v1/messages/count_tokens")
    def count_tokens(body: dict):
        try:
            return front.count(body)
        except ValueError as e:
            return JSONResponse(error_body("invalid_request_error", str(e)), status_code=400)

    @app.post("/v1/messages")
    def messages(body: dict):
        try:
            if body.get("stream") and front.can_stream():
                return StreamingResponse(front.stream(front.prepare(body), body), media_type="text/event-stream")
            message = front.run(body)
        except (ValueError, OverflowError) as e:
            return JSONResponse(error_body("invalid_request_error", str(e)), status_code=400)
        except Exception as e:  # noqa: BLE001 - the engine's failure, as an error the client may retry
            return JSONResponse(error_body("api_error", str(e)), status_code=500)
        if body.get("stream"):
            return StreamingResponse(front.events(message), media_type="text/event-stream")
        return message

    return front

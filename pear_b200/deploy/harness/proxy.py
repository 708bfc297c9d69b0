"""The model server as a session's agent reaches it: a loopback HTTP service that rewrites, sizes, relays and records every
Messages request of every session.

What it does to a request (the behaviour of upstream's proxy, pear/deploy/harness/claude_code/proxy.py:74-543):

* refuses it (409, not to be retried) unless the session runs a turn that still accepts requests;
* tells a compaction's request (the agent asks for a summary of the conversation so far: its instruction opens with a fixed
  marker) from a request of the conversation;
* rewrites it: the service's system prompt instead of the agent's, every picture back in place of its placeholder, the task's
  reference pictures at the head of the first user message, and for a compaction this deployment's own summary instruction in
  place of the agent's, without the last turn's pictures (they would draw the model to act instead of summarising);
* asks the model server for the prompt's token count; a prompt that leaves no room is answered with the "prompt is too long"
  error agents answer with a compaction; a conversation request gets all the output its context leaves, a compaction keeps the
  agent's own budget;
* relays the answer (whole or as an event stream) and reads usage and the stop reason out of it on the way: an answer cut at
  the token limit ends the turn without an action; a compaction's answer without the summary's closing tag is a failure the
  agent retries;
* writes one line per request to the session's audit file, pictures as digests.
"""

from __future__ import annotations

import asyncio
import hashlib
import json
import os
import time
import uuid
from typing import Any, Optional

import aiohttp
from aiohttp import web

from .session import AgentSession, Turn


class RequestAudit:
    """One JSON line per model request of a session; base64 payloads are replaced by their size and digest."""

    def __init__(self, directory: str, session_id: str):
        os.makedirs(directory, exist_ok=True)
        self.path = os.path.join(directory, f"{session_id}.jsonl")

    def write(self, kind: str, turn_id: Optional[str], agent_request: Any, upstream_request: Any, outcome: dict) -> None:
        rec = {"time": time.time(), "kind": kind, "turn_id": turn_id, "agent_request": self.digested(agent_request),
               "upstream_request": self.digested(upstream_request), "outcome": outcome}
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")

    @classmethod
    def digested(cls, value: Any) -> Any:
        if isinstance(value, dict):
            if value.get("type") == "base64" and isinstance(value.get("data"), str):
                raw = value["data"].encode()
                return {**{k: v for k, v in value.items() if k != "data"}, "data_bytes": len(raw), "data_sha256": hashlib.sha256(raw).hexdigest()}
            return {k: cls.digested(v) for k, v in value.items()}
        if isinstance(value, list):
            return [cls.digested(v) for v in value]
        return value


class EngineMetrics:
    """The model server's Prometheus text, read at most once an interval: what usage reports carry of the engine's state."""

    # (the names of rollout/server.py's gauges and counters, without the ``pear_`` prefix)
    KEPT = ("num_running", "num_waiting", "free_blocks", "cached_blocks", "generation_tokens_total", "prompt_tokens_total", "prefix_cache_queries_total",
            "prefix_cache_hits_total", "spec_drafted_total", "spec_accepted_total", "deploy_generation_tokens_total", "deploy_busy_seconds_total")

    def __init__(self, http: aiohttp.ClientSession, url: str, interval_s: float):
        self.http, self.url, self.interval_s = http, url, interval_s
        self.latest: dict[str, float] = {}
        self.read_at = 0.0

    @staticmethod
    def parse(text: str) -> dict[str, float]:
        out = {}
        for line in text.splitlines():
            if not line or line.startswith("#"):
                continue
            name, _, value = line.rpartition(" ")
            name = name.partition("{")[0]
            try:
                out[name.removeprefix("pear_")] = float(value)
            except ValueError:
                pass
        return out

    async def refresh(self) -> dict[str, float]:
        if time.time() - self.read_at >= self.interval_s:
            self.read_at = time.time()
            try:
                async with self.http.get(self.url, timeout=aiohttp.ClientTimeout(total=2.0)) as r:
                    got = self.parse(await r.text())
                self.latest = {k: v for k, v in got.items() if k in self.KEPT}
            except (aiohttp.ClientError, asyncio.TimeoutError):
                pass
        return self.latest


class UpstreamProxy:
    HOST = "127.0.0.1"  # only the sessions' own processes reach it
    MAIN, SUMMARY, REFUSED = "main", "summary", "refused"
    SUMMARY_MARKER = "CRITICAL: Respond with TEXT ONLY."  # how agents of this protocol open a compaction's instruction
    SUMMARY_END = "</summary>"
    FORWARDED_FIELDS = ("model", "messages", "max_tokens", "stream")  # sampling is the server's and the config's
    COUNTED_FIELDS = ("model", "messages", "system")
    REFUSAL_STATUS, RETRY_STATUS, TOO_LONG_STATUS = 409, 500, 400
    SHOULD_RETRY_HEADER = "x-should-retry"
    TOO_LONG_MESSAGE = "prompt is too long: {tokens} tokens > {limit} maximum"
    CUT_MESSAGE = "The answer reached the model's token limit and was cut; no action executes"
    PICTURES_MESSAGE = "The camera images did not reach the model unchanged; no action executes"
    NO_OUTPUT_MESSAGE = "The model server sent no output"
    NO_SUMMARY_MESSAGE = "The model wrote no summary within its output limit"
    PROMPT_KEYS = ("input_tokens", "cache_read_input_tokens", "cache_creation_input_tokens")

    def __init__(self, upstream: str, http: aiohttp.ClientSession, context_limit: int, summary_instruction: str, audit_dir: Optional[str] = None,
                 chat_template_kwargs: Optional[dict] = None, metrics_interval_s: float = 1.0, require_summary_end: bool = True):
        self.upstream, self.http, self.context_limit = upstream.rstrip("/"), http, int(context_limit)
        self.summary_instruction, self.audit_dir = summary_instruction, audit_dir
        self.chat_template_kwargs = dict(chat_template_kwargs or {})
        self.require_summary_end = require_summary_end
        self.metrics = EngineMetrics(http, self.upstream + "/metrics", metrics_interval_s)
        self.sessions: dict[str, AgentSession] = {}
        self.running: dict[str, set] = {}  # session id -> the handler tasks in flight
        self.audits: dict[str, RequestAudit] = {}
        self.url = ""

    async def __aenter__(self) -> "UpstreamProxy":
        app = web.Application(client_max_size=256 * 1024 * 1024)
        app.router.add_post("/{session_id}/v1/messages", self.messages)
        app.router.add_post("/{session_id}/v1/messages/count_tokens", self.count_tokens)
        self._runner = web.AppRunner(app, access_log=None, handler_cancellation=True)
        await self._runner.setup()
        site = web.TCPSite(self._runner, self.HOST, 0)
        await site.start()
        self.url = f"http://{self.HOST}:{self._runner.addresses[0][1]}"
        return self

    async def __aexit__(self, *exc: object) -> None:
        for sid in list(self.sessions):
            await self.cancel(sid)
        await self._runner.cleanup()

    # -- sessions ---------------------------------------------------------------------------------------------------------
    def open(self, session: AgentSession) -> str:
        self.sessions[session.id] = session
        self.running[session.id] = set()
        if self.audit_dir:
            self.audits[session.id] = RequestAudit(self.audit_dir, session.id)
        return f"{self.url}/{session.id}"

    async def close(self, session_id: str) -> None:
        await self.cancel(session_id)
        self.sessions.pop(session_id, None)
        self.running.pop(session_id, None)
        self.audits.pop(session_id, None)

    async def cancel(self, session_id: str) -> None:
        """End the session's requests in flight (an interrupt, a close): the model server sees its client leave."""
        tasks = [t for t in self.running.get(session_id, ()) if not t.done()]
        for t in tasks:
            t.cancel()
        if tasks:
            await asyncio.gather(*tasks, return_exceptions=True)

    def engine_metrics(self) -> dict:
        return dict(self.metrics.latest)

    # -- the two routes ---------------------------------------------------------------------------------------------------
    async def messages(self, request: web.Request) -> web.StreamResponse:
        sid = request.match_info["session_id"]
        session, audit = self.sessions.get(sid), self.audits.get(sid)
        agent_request = await request.json()
        turn = session.turn if session else None
        if turn is None or turn.done.is_set() or turn.refusal or turn.cancellation.is_set():
            if audit:
                audit.write(self.REFUSED, turn.id if turn else None, agent_request, None, {"status": self.REFUSAL_STATUS})
            return self.refusal("The session takes no model request now")
        kind = self.kind_of(agent_request)
        upstream_request = self.rewrite(agent_request, session, kind)
        if kind == self.MAIN:
            # an agent's history only ever loses messages: a picture its request no longer holds is not asked for again
            held = {self.placeholder_of(b) for m in agent_request["messages"] for b in self.blocks(m.get("content"))} | turn.images.keys()
            session.images = {p: img for p, img in session.images.items() if p in held}
        outcome: dict[str, Any] = {}
        task = asyncio.current_task()
        self.running[sid].add(task)
        try:
            return await self.answer(request, session, turn, kind, upstream_request, outcome)
        finally:
            self.running.get(sid, set()).discard(task)
            if audit:
                audit.write(kind, turn.id, agent_request, upstream_request, outcome)

    async def count_tokens(self, request: web.Request) -> web.Response:
        """The agent's own count of a prompt, answered with the model server's count of what the prompt stands for."""
        body = await request.json()
        counted = {k: body[k] for k in self.COUNTED_FIELDS if k in body}
        session = self.sessions.get(request.match_info["session_id"])
        if session is not None:
            counted["messages"] = [self.drawn(m, session.images) for m in counted.get("messages", [])]
            counted["system"] = session.system
        async with self.http.post(self.upstream + "/v1/messages/count_tokens", json=counted) as r:
            return web.Response(status=r.status, body=await r.read(), content_type="application/json")

    # -- rewriting --------------------------------------------------------------------------------------------------------
    def kind_of(self, agent_request: dict) -> str:
        return self.SUMMARY if any(self.instructs_summary(m) for m in agent_request.get("messages", [])) else self.MAIN

    def rewrite(self, agent_request: dict, session: AgentSession, kind: str) -> dict:
        messages = list(agent_request.get("messages", []))
        if kind == self.SUMMARY:
            messages = [self.instructed(m) if self.instructs_summary(m) else m for m in messages]
        messages = [self.drawn(m, session.images) for m in messages]
        if messages and session.references:
            messages[0] = {**messages[0], "content": [*session.references, *self.blocks(messages[0].get("content"))]}
        out = {k: agent_request[k] for k in self.FORWARDED_FIELDS if k in agent_request}
        out.update(messages=messages, system=session.system, metadata={"user_id": session.id})  # (the session names the server's prefix-cache entry)
        if self.chat_template_kwargs:
            out["chat_template_kwargs"] = self.chat_template_kwargs
        return out

    def instructed(self, message: dict) -> dict:
        """A compaction's message with this deployment's instruction in place of the agent's, without the pictures (and their
        labels) of the turn the agent appended it to."""
        content: list[dict] = []
        for b in self.blocks(message.get("content")):
            if self.is_placeholder(b):
                if content and content[-1].get("type") == "text" and not self.is_instruction(content[-1]):
                    content.pop()  # the picture's label, right before it
            else:
                content.append({"type": "text", "text": self.summary_instruction} if self.is_instruction(b) else b)
        return {**message, "content": content}

    @classmethod
    def drawn(cls, message: dict, images: dict) -> dict:
        """``message`` with every known placeholder replaced by its picture."""
        if isinstance(message.get("content"), str) and not any(p in message["content"] for p in images):
            return message
        return {**message, "content": [images.get(cls.placeholder_of(b), b) if cls.is_placeholder(b) else b for b in cls.blocks(message.get("content"))]}

    # -- sizing, checking, relaying ---------------------------------------------------------------------------------------
    async def answer(self, request: web.Request, session: AgentSession, turn: Turn, kind: str, upstream_request: dict, outcome: dict) -> web.StreamResponse:
        counted = {k: upstream_request[k] for k in self.COUNTED_FIELDS if k in upstream_request}
        async with self.http.post(self.upstream + "/v1/messages/count_tokens", json=counted) as r:
            if r.status != 200:  # the model server refuses the prompt itself (pictures without a vision encoder, a malformed block)
                outcome.update(status=r.status, error="count_tokens refused")
                return web.Response(status=r.status, body=await r.read(), content_type="application/json")
            prompt_tokens = int((await r.json())["input_tokens"])
        room = self.context_limit - prompt_tokens
        outcome.update(prompt_tokens=prompt_tokens)
        if room <= 0:
            outcome.update(status=self.TOO_LONG_STATUS)
            msg = self.TOO_LONG_MESSAGE.format(tokens=prompt_tokens, limit=self.context_limit)
            return web.json_response({"type": "error", "error": {"type": "invalid_request_error", "message": msg}}, status=self.TOO_LONG_STATUS)
        asked = int(upstream_request.get("max_tokens") or room)
        upstream_request["max_tokens"] = room if kind == self.MAIN else min(asked, room)
        messages = upstream_request["messages"]
        if self.holds_placeholder(messages) or (kind == self.MAIN and not self.pictures_arrived(turn, messages)):
            turn.refusal = self.PICTURES_MESSAGE
            outcome.update(status=self.REFUSAL_STATUS)
            return self.refusal(turn.refusal)
        if kind == self.MAIN:
            turn.usage.measure_context(prompt_tokens)
        return await self.forward(request, session, turn, kind, upstream_request, outcome)

    async def forward(self, request: web.Request, session: AgentSession, turn: Turn, kind: str, upstream_request: dict, outcome: dict) -> web.StreamResponse:
        rid = uuid.uuid4().hex
        turn.usage.open_request(rid, kind)
        await self.metrics.refresh()
        try:
            async with self.http.post(self.upstream + "/v1/messages", json=upstream_request) as r:
                outcome.update(status=r.status)
                if r.status != 200:
                    return web.Response(status=r.status, body=await r.read(), content_type="application/json")
                if not upstream_request.get("stream"):
                    body = await r.json()
                    text = "".join(b.get("text", "") for b in body.get("content", []) if b.get("type") == "text")
                    bad = self.observe(turn, rid, kind, body.get("usage") or {}, body.get("stop_reason"), text, outcome)
                    return bad or web.json_response(body)
                return await self.relay(request, r, turn, rid, kind, outcome)
        except aiohttp.ClientError as e:
            outcome.update(status=self.RETRY_STATUS, error=str(e))
            return self.failure(f"The model server did not answer: {e}")
        finally:
            session.report_usage(turn)

    async def relay(self, request: web.Request, upstream: aiohttp.ClientResponse, turn: Turn, rid: str, kind: str, outcome: dict) -> web.StreamResponse:
        """Pass an event stream through frame by frame. A compaction's stream is held back until it is whole, so that an answer
        without a summary can still be turned into a failure the agent retries; a conversation's goes out as it arrives."""
        usage: dict = {}
        stop, text, frames, buf = None, [], [], b""
        hold = kind == self.SUMMARY
        response: Optional[web.StreamResponse] = None
        async for chunk in upstream.content.iter_any():
            buf += chunk
            while b"\n\n" in buf:
                frame, buf = buf.split(b"\n\n", 1)
                ev = self.event_of(frame)
                kind_ev = ev.get("type")
                if kind_ev == "message_start":
                    usage.update((ev.get("message") or {}).get("usage") or {})
                elif kind_ev == "content_block_delta":
                    text.append((ev.get("delta") or {}).get("text", ""))
                elif kind_ev == "message_delta":
                    usage.update(ev.get("usage") or {})
                    stop = (ev.get("delta") or {}).get("stop_reason")
                if hold:
                    frames.append(frame + b"\n\n")
                    continue
                if response is None:
                    response = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
                    await response.prepare(request)
                await response.write(frame + b"\n\n")
        whole = "".join(text)
        if not whole and stop is None:
            outcome.update(status=self.RETRY_STATUS, error=self.NO_OUTPUT_MESSAGE)
            if response is None:
                return self.failure(self.NO_OUTPUT_MESSAGE)
        bad = self.observe(turn, rid, kind, usage, stop, whole, outcome)
        if hold:
            if bad is not None:
                return bad
            response = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
            await response.prepare(request)
            for f in frames:
                await response.write(f)
        await response.write_eof()
        return response

    def observe(self, turn: Turn, rid: str, kind: str, usage: dict, stop: Optional[str], text: str, outcome: dict) -> Optional[web.Response]:
        """Record an answer's counts; returns a failure in place of the answer when a compaction produced no summary."""
        prompt = sum(int(usage.get(k) or 0) for k in self.PROMPT_KEYS)
        turn.usage.update(rid, prompt_tokens=prompt, cached_tokens=int(usage.get("cache_read_input_tokens") or 0), output_tokens=int(usage.get("output_tokens") or 0))
        outcome.update(stop_reason=stop, output_tokens=int(usage.get("output_tokens") or 0))
        if kind == self.MAIN and stop == "max_tokens":
            turn.refusal = self.CUT_MESSAGE  # the agent still gets the answer; the turn's result says that nothing executes
        if kind == self.SUMMARY and self.require_summary_end and self.SUMMARY_END not in text:
            outcome.update(status=self.RETRY_STATUS, error=self.NO_SUMMARY_MESSAGE)
            return self.failure(self.NO_SUMMARY_MESSAGE)
        return None

    # -- small things -----------------------------------------------------------------------------------------------------
    @classmethod
    def refusal(cls, message: str) -> web.Response:
        body = {"type": "error", "error": {"type": "invalid_request_error", "message": message}}
        return web.json_response(body, status=cls.REFUSAL_STATUS, headers={cls.SHOULD_RETRY_HEADER: "false"})

    @classmethod
    def failure(cls, message: str) -> web.Response:
        body = {"type": "error", "error": {"type": "api_error", "message": message}}
        return web.json_response(body, status=cls.RETRY_STATUS, headers={cls.SHOULD_RETRY_HEADER: "true"})

    @staticmethod
    def blocks(content: Any) -> list[dict]:
        if isinstance(content, str):
            return [{"type": "text", "text": content}]
        return list(content or [])

    @classmethod
    def is_instruction(cls, block: dict) -> bool:
        return block.get("type") == "text" and block.get("text", "").lstrip().startswith(cls.SUMMARY_MARKER)

    @classmethod
    def instructs_summary(cls, message: dict) -> bool:
        return message.get("role") == "user" and any(cls.is_instruction(b) for b in cls.blocks(message.get("content")))

    @staticmethod
    def placeholder_head() -> str:
        return AgentSession.IMAGE_PLACEHOLDER.partition("{")[0]

    @classmethod
    def is_placeholder(cls, block: dict) -> bool:
        return block.get("type") == "text" and block.get("text", "").startswith(cls.placeholder_head())

    @classmethod
    def placeholder_of(cls, block: dict) -> Optional[str]:
        return block.get("text") if cls.is_placeholder(block) else None

    @classmethod
    def holds_placeholder(cls, messages: list) -> bool:
        """Whether a picture is still a placeholder after rewriting: the model would read a caption, not the camera."""
        return any(cls.is_placeholder(b) for m in messages for b in cls.blocks(m.get("content")))

    @classmethod
    def pictures_arrived(cls, turn: Turn, messages: list) -> bool:
        """Whether every picture of the turn is somewhere in the request as the picture itself."""
        if not turn.images:
            return True
        sent = [b.get("source", {}).get("data") for m in messages for b in cls.blocks(m.get("content")) if b.get("type") == "image"]
        return all(img["source"]["data"] in sent for img in turn.images.values())

    @staticmethod
    def event_of(frame: bytes) -> dict:
        for line in frame.split(b"\n"):
            if line.startswith(b"data:"):
                try:
                    return json.loads(line[5:])
                except ValueError:
                    return {}
        return {}

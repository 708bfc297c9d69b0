"""One conversation of an agent process, turn by turn.

The agent is a command-line program that speaks the Messages form to a base URL from its environment
(``ANTHROPIC_BASE_URL``) and the line protocol of such CLIs on its pipes: one JSON object a line on stdin for every user
message (``{"type": "user", "message": {...}}``) and for control requests (``{"type": "control_request", "request":
{"subtype": "interrupt"}}``), one JSON object a line on stdout for what it does (``system`` notes such as the boundary of a
compaction, ``assistant`` messages, and a ``result`` that ends the turn). Upstream drives its CLI through that CLI's SDK
(pear/deploy/harness/claude_code/session.py:124-428); this session owns the process and the pipes itself, so any agent that
speaks the two protocols fits, the scripted one of ``scripted_agent.py`` included.

A session has at most one turn at a time. Its model requests reach the model server only through the proxy, which asks the
session for the turn they belong to; a session whose agent process ended is lost for good.
"""

from __future__ import annotations

import asyncio
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Optional


class SessionLost(RuntimeError):
    """The session's agent process is gone: its conversation cannot go on."""


class TurnUsage:
    """What a turn's model requests cost: the context the last main request held, output tokens, cache hits, compactions."""

    def __init__(self, context_limit: int):
        self.context_limit = context_limit
        self.context_tokens: Optional[int] = None  # prompt tokens of the latest main request
        self.requests: dict[str, dict] = {}  # open and finished requests by id
        self.compactions = 0
        self.started = time.time()

    def open_request(self, request_id: str, kind: str) -> None:
        self.requests[request_id] = {"kind": kind, "prompt_tokens": 0, "cached_tokens": 0, "output_tokens": 0}

    def update(self, request_id: str, **counts: Any) -> None:
        self.requests.setdefault(request_id, {}).update({k: v for k, v in counts.items() if v is not None})

    def measure_context(self, prompt_tokens: int) -> None:
        self.context_tokens = prompt_tokens

    def compact(self) -> None:
        self.compactions += 1

    def snapshot(self, is_final: bool, engine: Optional[dict] = None) -> dict:
        rs = list(self.requests.values())
        out = {"requests": len(rs), "prompt_tokens": sum(r.get("prompt_tokens", 0) for r in rs), "cached_tokens": sum(r.get("cached_tokens", 0) for r in rs),
               "output_tokens": sum(r.get("output_tokens", 0) for r in rs), "context_tokens": self.context_tokens, "context_limit": self.context_limit,
               "compactions": self.compactions, "seconds": round(time.time() - self.started, 3), "is_final": is_final}
        if engine:
            out["engine"] = engine
        return out


@dataclass
class Turn:
    id: str
    content: list  # the user message's blocks as the agent is given them (pictures as placeholders)
    images: dict  # placeholder text -> image block
    usage: TurnUsage
    events: asyncio.Queue = field(default_factory=asyncio.Queue)
    done: asyncio.Event = field(default_factory=asyncio.Event)
    cancellation: asyncio.Event = field(default_factory=asyncio.Event)
    refusal: Optional[str] = None  # why the turn ends without an action, once something went wrong on the way


class AgentSession:
    IMAGE_PLACEHOLDER = "[camera image {key}]"  # what the agent's history holds of a picture; the proxy puts the picture back
    RESULT_EVENT, TEXT_EVENT, USAGE_EVENT, NOTE_EVENT = "result", "text", "usage", "note"
    INTERRUPT_GRACE_S = 10.0  # an agent that has not ended its turn this long after an interrupt is stopped
    START_TIMEOUT_S = 60.0

    def __init__(self, session_id: str, system: str, command: list[str], proxy, context_limit: int, env: Optional[dict] = None):
        self.id, self.system, self.command, self.proxy, self.context_limit = session_id, system, list(command), proxy, context_limit
        self.env = dict(env or {})
        self.images: dict[str, dict] = {}  # every picture the conversation still holds, by placeholder
        self.references: list[dict] = []  # the task's own pictures: at the head of the first user message of every request
        self.turn: Optional[Turn] = None
        self.lost_reason: Optional[str] = None
        self.process: Optional[asyncio.subprocess.Process] = None
        self.started: asyncio.Future = asyncio.get_event_loop().create_future()
        self._inbox: asyncio.Queue = asyncio.Queue()
        self._task = asyncio.ensure_future(self._own())

    # -- the service's side -----------------------------------------------------------------------------------------------
    def submit(self, turn_id: str, content: list, images: dict, references: list) -> Turn:
        if self.lost_reason:
            raise SessionLost(self.lost_reason)
        if self.turn is not None and not self.turn.done.is_set():
            raise ValueError("The session runs a turn already")
        if references:
            self.references = list(references)
        self.images.update(images)
        turn = self.turn = Turn(turn_id, content, dict(images), TurnUsage(self.context_limit))
        self._inbox.put_nowait(turn)
        return turn

    async def interrupt(self, turn_id: str) -> None:
        """Stop a turn (before it starts too) and return once its result is out."""
        turn = self.turn
        if turn is None or turn.id != turn_id or turn.done.is_set():
            return
        turn.cancellation.set()
        await self.proxy.cancel(self.id)
        await self._send({"type": "control_request", "request_id": f"interrupt-{turn_id}", "request": {"subtype": "interrupt"}})
        try:
            await asyncio.wait_for(turn.done.wait(), self.INTERRUPT_GRACE_S)
        except asyncio.TimeoutError:
            await self._lose("The agent did not stop after an interrupt")
        if self.lost_reason:
            raise SessionLost(self.lost_reason)

    async def close(self) -> None:
        await self._lose("The session was closed")
        self._task.cancel()
        try:
            await self._task
        except (asyncio.CancelledError, Exception):  # noqa: BLE001
            pass
        await self.proxy.close(self.id)

    def report_usage(self, turn: Turn, is_final: bool = False) -> None:
        self._emit(turn, self.USAGE_EVENT, turn.usage.snapshot(is_final, self.proxy.engine_metrics()))

    # -- the agent process ------------------------------------------------------------------------------------------------
    async def _own(self) -> None:
        base_url = self.proxy.open(self)
        env = {**self.env, "ANTHROPIC_BASE_URL": base_url, "ANTHROPIC_API_KEY": "unused", "PEAR_SESSION_ID": self.id, "PEAR_SYSTEM_PROMPT": self.system}
        try:
            self.process = await asyncio.create_subprocess_exec(*self.command, stdin=asyncio.subprocess.PIPE, stdout=asyncio.subprocess.PIPE, env=env,
                                                                limit=64 * 1024 * 1024)
        except OSError as e:
            self.lost_reason = f"The agent did not start: {e}"
            self.started.set_exception(SessionLost(self.lost_reason))
            return
        self.started.set_result(True)
        try:
            while True:
                turn = await self._inbox.get()
                await self._run(turn)
        finally:
            await self._stop_process()

    async def _run(self, turn: Turn) -> None:
        result: Optional[dict] = None
        try:
            if not turn.cancellation.is_set():
                await self._send({"type": "user", "message": {"role": "user", "content": turn.content}, "turn_id": turn.id})
                result = await self._receive(turn)
        except SessionLost:
            pass
        self._finish(turn, result)

    async def _receive(self, turn: Turn) -> Optional[dict]:
        while True:
            line = await self.process.stdout.readline()
            if not line:
                await self._lose("The agent process ended")
                raise SessionLost(self.lost_reason)
            try:
                msg = json.loads(line)
            except ValueError:
                continue  # not the protocol's: an agent's own log line
            kind = msg.get("type")
            if kind == "result":
                return msg
            if kind == "system":
                if msg.get("subtype") == "compact_boundary":
                    turn.usage.compact()
                    self.report_usage(turn)
                self._emit(turn, self.NOTE_EVENT, {"subtype": msg.get("subtype"), "data": msg.get("data")})
            elif kind == "assistant":
                text = "".join(b.get("text", "") for b in (msg.get("message") or {}).get("content", []) if b.get("type") == "text")
                self._emit(turn, self.TEXT_EVENT, {"text": text})
                self.report_usage(turn)

    def _finish(self, turn: Turn, result: Optional[dict]) -> None:
        """The turn's last event: the agent's answer, or why there is none (interrupted, refused on the way, session lost)."""
        if turn.done.is_set():
            return
        data: dict[str, Any] = {"text": "", "is_error": False, "stop": "end_turn"}
        if self.lost_reason:
            data.update(is_error=True, stop="lost", message=self.lost_reason)
        elif turn.cancellation.is_set():
            data.update(stop="interrupted")
        elif turn.refusal:
            data.update(is_error=True, stop="refused", message=turn.refusal)
        elif result is None or result.get("is_error"):
            data.update(is_error=True, stop="error", message=str((result or {}).get("result") or "The agent reported an error"))
        else:
            data.update(text=str(result.get("result") or ""))
        data["usage"] = turn.usage.snapshot(True, self.proxy.engine_metrics())
        self._emit(turn, self.RESULT_EVENT, data)
        turn.done.set()

    def _emit(self, turn: Turn, kind: str, data: dict) -> None:
        turn.events.put_nowait({"type": kind, "turn_id": turn.id, **data})

    async def _send(self, obj: dict) -> None:
        p = self.process
        if p is None or p.returncode is not None:
            await self._lose("The agent process ended")
            raise SessionLost(self.lost_reason)
        try:
            p.stdin.write((json.dumps(obj) + "\n").encode())
            await p.stdin.drain()
        except (BrokenPipeError, ConnectionResetError):
            await self._lose("The agent process ended")
            raise SessionLost(self.lost_reason) from None

    async def _lose(self, reason: str) -> None:
        if not self.lost_reason:
            self.lost_reason = reason
        await self._stop_process()
        if self.turn is not None and not self.turn.done.is_set():
            self._finish(self.turn, None)

    async def _stop_process(self) -> None:
        p = self.process
        if p is None or p.returncode is not None:
            return
        try:
            p.stdin.close()
        except Exception:  # noqa: BLE001
            pass
        try:
            await asyncio.wait_for(p.wait(), 3.0)
        except asyncio.TimeoutError:
            p.kill()  # this session's own child, by its handle
            await p.wait()


def kept_environment(names=("PATH", "HOME", "LANG", "LC_ALL", "TMPDIR", "USER", "PYTHONPATH", "VIRTUAL_ENV")) -> dict:
    """What an agent process inherits of the service's environment: none of a login shell's keys or proxies."""
    return {k: os.environ[k] for k in names if k in os.environ}

"""The station's model clients: who holds the conversation and answers a turn.

``ModelClient.infer(model_input, on_event, cancellation)`` answers one turn (text + camera pictures + the task's reference
pictures) with the model's final answer. Two clients, as upstream has (pear/deploy/station/agent_loop/clients/client.py,
vllm.py, claude_code.py): ``MessagesClient`` keeps the conversation itself and asks the model server's Messages route directly;
``HarnessClient`` leaves the conversation to an agent behind the session service of ``deploy/harness`` (which compacts a full
context by itself) and streams the turn's events. Both stop a request in flight when ``cancellation`` is set or ``cancel()`` is
called, and both say for good when a conversation cannot go on (``ContextLimit``, ``SessionLost``).
"""

from __future__ import annotations

import base64
import io
import json
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np


class ContextLimit(ValueError):
    """The conversation no longer fits the model's context."""


class SessionLost(RuntimeError):
    """The service's session is gone; the task must be cleared."""


@dataclass
class ModelInput:
    text: str
    images: dict  # camera name -> uint8 [H, W, 3]
    reference_images: tuple = ()  # uint8 pictures of the task, sent with the first turn


@dataclass
class ModelOutput:
    answer: str
    seconds: float
    usage: dict = field(default_factory=dict)


def jpeg_b64(frame: np.ndarray, quality: int = 90) -> str:
    from PIL import Image

    buf = io.BytesIO()
    Image.fromarray(np.ascontiguousarray(frame)).save(buf, "JPEG", quality=quality)
    return base64.b64encode(buf.getvalue()).decode("ascii")


class ModelClient:
    CLEANUP_TIMEOUT_S = 15.0

    def __init__(self, system_prompt: str, timeout_s: float = 600.0):
        self.system_prompt, self.timeout_s = system_prompt, timeout_s

    def check(self) -> dict: ...
    def infer(self, model_input: ModelInput, on_event: Callable[[str, dict], None], cancellation: threading.Event) -> ModelOutput: ...
    def cancel(self) -> None: ...
    def close(self) -> None: ...

    def _watch(self, cancellation: threading.Event, response) -> threading.Thread:
        """Close ``response`` (a streaming HTTP response) once ``cancellation`` is set: the blocked read then ends."""
        done = threading.Event()

        def watch():
            while not done.wait(0.05):
                if cancellation.is_set() or self._cancelled.is_set():
                    response.close()
                    return

        t = threading.Thread(target=watch, daemon=True)
        t.done = done  # type: ignore[attr-defined]
        t.start()
        return t


class MessagesClient(ModelClient):
    """Asks ``/v1/messages`` of a model server directly; the history is this client's."""

    def __init__(self, base_url: str, model: str, system_prompt: str, max_tokens: int = 1024, timeout_s: float = 600.0, session=None):
        import requests

        super().__init__(system_prompt, timeout_s)
        self.url, self.model, self.max_tokens = base_url.rstrip("/"), model, max_tokens
        self.http = session or requests.Session()
        self.history: list[dict] = []
        self.user_id = str(uuid.uuid4())  # names the server's prefix-cache entry of this conversation
        self._cancelled = threading.Event()
        self._sent_references = False

    def check(self) -> dict:
        r = self.http.get(self.url + "/v1/models", timeout=5)
        r.raise_for_status()
        served = {m["id"]: m for m in r.json()["data"]}
        if self.model not in served:
            return {"status": "offline", "message": f"the server does not serve {self.model}"}
        return {"status": "ok", "model": self.model, "context_limit": served[self.model].get("max_model_len"), "capabilities": {"reference_images": True}}

    def infer(self, model_input, on_event, cancellation) -> ModelOutput:
        self._cancelled.clear()
        blocks: list[dict] = []
        if model_input.reference_images and not self._sent_references:
            blocks += [{"type": "image", "source": {"type": "base64", "media_type": "image/jpeg", "data": jpeg_b64(f)}} for f in model_input.reference_images]
        blocks.append({"type": "text", "text": model_input.text})
        for name, frame in model_input.images.items():
            blocks += [{"type": "text", "text": f"[{name}]"}, {"type": "image", "source": {"type": "base64", "media_type": "image/jpeg", "data": jpeg_b64(frame)}}]
        body = {"model": self.model, "system": self.system_prompt, "messages": self.history + [{"role": "user", "content": blocks}],
                "max_tokens": self.max_tokens, "metadata": {"user_id": self.user_id}}
        t0 = time.time()
        result: dict = {}

        def work():
            try:
                result["r"] = self.http.post(self.url + "/v1/messages", json=body, timeout=self.timeout_s)
            except Exception as e:  # noqa: BLE001
                result["e"] = e

        th = threading.Thread(target=work, daemon=True)
        th.start()
        while th.is_alive():
            th.join(0.05)
            if cancellation.is_set() or self._cancelled.is_set():
                raise InterruptedError("The model request was stopped")  # (the worker's answer, if one comes, is dropped)
        if "e" in result:
            raise RuntimeError(f"The model server did not answer: {result['e']}")
        r = result["r"]
        if r.status_code == 400 and "prompt is too long" in r.text:
            raise ContextLimit(r.json()["error"]["message"])
        r.raise_for_status()
        out = r.json()
        answer = "".join(b.get("text", "") for b in out.get("content", []) if b.get("type") == "text")
        if out.get("stop_reason") == "max_tokens":
            raise ValueError("The answer reached the model's token limit and was cut; no action executes")
        self.history += [{"role": "user", "content": blocks}, {"role": "assistant", "content": [{"type": "text", "text": answer}]}]
        self._sent_references = True
        on_event("usage", out.get("usage") or {})
        return ModelOutput(answer, time.time() - t0, out.get("usage") or {})

    def cancel(self) -> None:
        self._cancelled.set()

    def close(self) -> None:
        self.cancel()
        self.http.close()


class HarnessClient(ModelClient):
    """Drives a session of ``deploy/harness/service.py``: opened with the system prompt at the first turn, one turn per
    ``infer``, events streamed to ``on_event``, an interrupt when the turn is cancelled, the session deleted on ``close``."""

    SERVICE_NAME = "pear-agent-harness"

    def __init__(self, base_url: str, model: str, system_prompt: str, timeout_s: float = 600.0):
        import requests

        super().__init__(system_prompt, timeout_s)
        self.url, self.model = base_url.rstrip("/"), model
        self.http = requests.Session()
        self.session_id: Optional[str] = None
        self.turn_id: Optional[str] = None
        self._cancelled = threading.Event()
        self._sent_references = False

    def check(self) -> dict:
        r = self.http.get(self.url + "/health", timeout=5)
        h = r.json()
        if h.get("service") != self.SERVICE_NAME:
            return {"status": "offline", "message": "not an agent harness"}
        return h

    def _open(self) -> None:
        sid = str(uuid.uuid4())
        r = self.http.post(self.url + "/sessions", json={"session_id": sid, "model": self.model, "system": self.system_prompt}, timeout=120)
        if r.status_code != 200:
            raise SessionLost(f"The service opened no session: {r.status_code} {r.text}")
        self.session_id = sid

    def infer(self, model_input, on_event, cancellation) -> ModelOutput:
        self._cancelled.clear()
        if self.session_id is None:
            self._open()
        self.turn_id = str(uuid.uuid4())
        body = {"turn_id": self.turn_id, "text": model_input.text, "images": [{"role": n, "data": jpeg_b64(f)} for n, f in model_input.images.items()],
                "reference_images": [] if self._sent_references else [{"data": jpeg_b64(f)} for f in model_input.reference_images]}
        t0 = time.time()
        r = self.http.post(f"{self.url}/sessions/{self.session_id}/turns", json=body, stream=True, timeout=self.timeout_s)
        if r.status_code == 410:
            raise SessionLost(r.text)
        if r.status_code != 200:
            raise ValueError(f"The service refused the turn: {r.status_code} {r.text}")
        watcher = self._watch(cancellation, r)
        result = None
        try:
            for line in r.iter_lines():
                if not line:
                    continue
                ev = json.loads(line)
                if ev["type"] == "result":
                    result = ev
                    break
                on_event(ev["type"], ev)
        except Exception as e:  # noqa: BLE001 - the stream was closed under the read (a cancellation) or broke
            if cancellation.is_set() or self._cancelled.is_set():
                self._interrupt()
                raise InterruptedError("The model request was stopped") from e
            raise RuntimeError(f"The turn's stream broke: {e}") from e
        finally:
            watcher.done.set()  # type: ignore[attr-defined]
            r.close()
        if result is None:
            if cancellation.is_set() or self._cancelled.is_set():
                self._interrupt()
                raise InterruptedError("The model request was stopped")
            raise RuntimeError("The turn ended without a result")
        self._sent_references = True
        if result["stop"] == "lost":
            raise SessionLost(result.get("message", "session lost"))
        if result["stop"] == "interrupted":
            raise InterruptedError("The model request was stopped")
        if result["is_error"]:
            raise ValueError(result.get("message", "the agent reported an error"))
        return ModelOutput(result["text"], time.time() - t0, result.get("usage") or {})

    def _interrupt(self) -> None:
        try:
            self.http.post(f"{self.url}/sessions/{self.session_id}/turns/{self.turn_id}/interrupt", timeout=30)
        except Exception:  # noqa: BLE001 - the service is gone: nothing runs
            pass

    def cancel(self) -> None:
        self._cancelled.set()

    def close(self) -> None:
        self.cancel()
        if self.session_id is not None:
            try:
                self.http.delete(f"{self.url}/sessions/{self.session_id}", timeout=30)
            except Exception:  # noqa: BLE001
                pass
        self.http.close()

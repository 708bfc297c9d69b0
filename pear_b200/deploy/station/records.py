"""A task's records beside the turns file of the agent loop: every event of every step, one JSON line each with wall-clock and
monotonic times (``events.jsonl``), and the context usage of the model session turn by turn (``context_usage.json``: the
latest context size against the limit, output tokens, cached tokens, compactions). Upstream keeps the same two kinds of record
for its GUI and its post-hoc analysis (pear/deploy/station/records/task_events.py, context_usage.py); picture payloads never go
into them (frames are files of their own, written by the agent loop)."""

from __future__ import annotations

import json
import os
import threading
import time
from typing import Any


class TaskRecords:
    def __init__(self, directory: str):
        self.directory = str(directory)
        os.makedirs(self.directory, exist_ok=True)
        self.events_path = os.path.join(self.directory, "events.jsonl")
        self.usage_path = os.path.join(self.directory, "context_usage.json")
        self.lock = threading.Lock()  # events arrive from the step's thread and the model call's thread
        self.turns: list[dict] = []
        self._turn: dict = {}

    @staticmethod
    def _plain(value: Any) -> Any:
        """JSON-safe copy without bulky payloads: arrays and byte strings become their shape / length."""
        if isinstance(value, dict):
            return {str(k): TaskRecords._plain(v) for k, v in value.items()}
        if isinstance(value, (list, tuple)):
            return [TaskRecords._plain(v) for v in value]
        if hasattr(value, "shape") and hasattr(value, "dtype"):
            return {"array": list(value.shape), "dtype": str(value.dtype)}
        if isinstance(value, (bytes, bytearray)):
            return {"bytes": len(value)}
        if isinstance(value, (str, int, float, bool)) or value is None:
            return value
        return str(value)

    def on_event(self, kind: str, data: dict) -> None:
        """The agent loop's (and, through it, the model client's) event handler."""
        with self.lock:
            with open(self.events_path, "a") as f:
                f.write(json.dumps({"time": time.time(), "monotonic": time.monotonic(), "type": kind, "data": self._plain(data)}) + "\n")
            if kind == "observation":
                self._turn = {"turn_id": data.get("turn_id"), "started": time.time()}
                self.turns.append(self._turn)
            elif kind == "usage" and self.turns:
                keep = ("context_tokens", "context_limit", "output_tokens", "cached_tokens", "prompt_tokens", "requests", "compactions",
                        "input_tokens", "cache_read_input_tokens")
                self._turn.update({k: data[k] for k in keep if data.get(k) is not None})
            elif kind == "model_output" and self.turns:
                self._turn["model_seconds"] = data.get("seconds")
            if kind in ("usage", "model_output"):
                self._write_usage()

    def _write_usage(self) -> None:
        latest = next((t for t in reversed(self.turns) if t.get("context_tokens") is not None), {})
        limit = latest.get("context_limit")
        summary = {"turns": len(self.turns), "context_tokens": latest.get("context_tokens"), "context_limit": limit,
                   "context_fraction": (latest["context_tokens"] / limit) if limit and latest.get("context_tokens") is not None else None,
                   "compactions": sum(int(t.get("compactions") or 0) for t in self.turns),
                   "output_tokens": sum(int(t.get("output_tokens") or 0) for t in self.turns), "per_turn": self.turns}
        tmp = self.usage_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(summary, f, indent=1)
        os.replace(tmp, self.usage_path)

"""The environment tool: the single "tool" an episode talks to (upstream ``pear/envs/tool.py:22-127``).

``open / step / close`` forward to an ``EpisodeClient``; an observation is rendered as the user turn
``state JSON + reminder + "[camera]" + one image per camera`` (``:114-127``); every call is appended to a JSONL call
log (``:91-112``).
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ..sim.client import EpisodeClient
from ..sim.server import ServerPool
from ..utils.files import append_jsonl


def load_system_prompt() -> str:
    with open(os.path.join(os.path.dirname(__file__), "system_prompt.md")) as f:
        return f.read()


@dataclass
class Observation:
    text: str
    frames: list[np.ndarray] = field(default_factory=list)  # one [tokens, hidden] block per camera, in camera order
    cameras: list[str] = field(default_factory=list)  # the cameras' names, in the same order: each picture is rendered under its label
    done: bool = False
    success: bool = False
    info: dict = field(default_factory=dict)


def render_observation(result: dict) -> Observation:
    obs = result["observation"]
    lines = [json.dumps(obs["state"], sort_keys=True), obs.get("reminder", "")]
    cameras = sorted(obs.get("frames", {}))
    frames = [np.asarray(obs["frames"][cam]) for cam in cameras]
    info = dict(result.get("info", {}))
    for key in ("environment", "task"):  # what the family says about itself once, for the system prompt of the episode
        if key in obs:
            info[key] = obs[key]
    return Observation("\n".join(lines), frames, cameras, bool(result.get("done")), bool(result.get("success")), info)


def episode_system_prompt(base: str, first: Observation) -> str:
    """The system prompt of one episode: the general instructions, then what the environment family says about itself (one line
    per camera or rule) and the task of this episode, as sections of their own (upstream's prompts end with ``## ENVIRONMENT`` and
    ``## TASK``: tests/agent_loop/prompt_renderings/*.txt)."""
    parts = [base.rstrip("\n")]
    env_lines = first.info.get("environment")
    if env_lines:
        parts.append("## ENVIRONMENT\n\n" + "\n".join(f"- {line}" for line in env_lines))
    if first.info.get("task"):
        parts.append("## TASK\n\n" + str(first.info["task"]))
    return "\n\n".join(parts) + "\n"


class EnvTool:
    """One instance per episode."""

    def __init__(self, pool: ServerPool, family: str, log_path: Optional[str] = None):
        self.client = EpisodeClient(pool, family)
        self.family, self.log_path = family, log_path
        self.calls = 0

    def _log(self, call: str, payload: dict, result: Optional[dict], error: Optional[str], t0: float) -> None:
        if self.log_path:
            append_jsonl(self.log_path, {"episode": self.client.episode_id, "family": self.family, "call": call, "n": self.calls,
                                         "payload": payload, "done": None if result is None else result.get("done"),
                                         "success": None if result is None else result.get("success"), "error": error,
                                         "seconds": round(time.time() - t0, 4)})

    def _run(self, call: str, payload: dict, fn) -> Observation:
        t0 = time.time()
        self.calls += 1
        try:
            result = fn()
        except Exception as e:  # noqa: BLE001 - logged, then re-raised for the agent loop
            self._log(call, payload, None, f"{type(e).__name__}: {e}", t0)
            raise
        self._log(call, payload, result, None, t0)
        return render_observation(result)

    def open(self, env_args: dict) -> Observation:
        return self._run("open", env_args, lambda: self.client.open(env_args))

    def step(self, action: dict) -> Observation:
        return self._run("step", action, lambda: self.client.step(action))

    def close(self) -> None:
        self.client.close()

"""Environment base classes of the simulator runtime (upstream ``pear/sim/env.py:17,76,110``).

``BaseEnv`` is what a simulator family implements: ``reset(args) -> observation`` and ``step(action) -> (observation,
done, success, info)``. Two hosting modes wrap it:

* ``StatelessEnv``: no episode state is kept in the server process between calls; each call carries the episode's
  arguments and its action history and the environment is REPLAYED from reset (seeded, so deterministic). Any server
  process can serve any call, and a failed call can be retried once on another process.
* ``StatefulEnv``: one episode lives in one process from ``open`` to ``close``; losing the process loses the episode
  (``EpisodeLost``), and the agent loop restarts the trajectory.

An observation is a dict: ``state`` (JSON-able), ``frames`` (per camera: an array; for the synthetic family a block of
vision-embedding placeholders), ``reminder`` (text).
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any


class EpisodeLost(RuntimeError):
    """The process holding an episode died or timed out; the trajectory has to restart."""


class BaseEnv(ABC):
    family: str = "base"

    @abstractmethod
    def reset(self, args: dict) -> dict:
        """Start an episode described by ``args`` (task id, seed ...). Returns the first observation."""

    @abstractmethod
    def step(self, action: dict) -> tuple[dict, bool, bool, dict]:
        """Apply one action. Returns (observation, done, success, info)."""

    def close(self) -> None:
        pass

    @classmethod
    def action_schema(cls) -> dict:
        """JSON schema of an action (the agent loop validates answers against it)."""
        return {"type": "object"}


class StatelessEnv:
    """Hosts a ``BaseEnv`` class without per-episode state: every call replays the history."""

    mode = "stateless"

    def __init__(self, env_cls: type[BaseEnv], **kwargs: Any):
        self.env_cls, self.kwargs = env_cls, kwargs

    def rollout(self, args: dict, actions: list[dict]) -> dict:
        env = self.env_cls(**self.kwargs)
        try:
            obs = env.reset(args)
            done = success = False
            info: dict = {}
            for a in actions:
                if done:
                    break
                obs, done, success, info = env.step(a)
            return {"observation": obs, "done": done, "success": success, "info": info, "steps": len(actions)}
        finally:
            env.close()


class StatefulEnv:
    """Hosts one live episode per process."""

    mode = "stateful"

    def __init__(self, env_cls: type[BaseEnv], **kwargs: Any):
        self.env_cls, self.kwargs = env_cls, kwargs
        self.env: BaseEnv | None = None
        self.episode_id: str | None = None

    def open(self, episode_id: str, args: dict) -> dict:
        if self.env is not None:
            self.env.close()
        self.env = self.env_cls(**self.kwargs)
        self.episode_id = episode_id
        return {"observation": self.env.reset(args), "done": False, "success": False, "info": {}}

    def step(self, episode_id: str, action: dict) -> dict:
        if self.env is None or episode_id != self.episode_id:
            raise EpisodeLost(f"episode {episode_id} is not held by this process")
        obs, done, success, info = self.env.step(action)
        return {"observation": obs, "done": done, "success": success, "info": info}

    def close(self, episode_id: str) -> None:
        if self.env is not None and episode_id == self.episode_id:
            self.env.close()
            self.env, self.episode_id = None, None

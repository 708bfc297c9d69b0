"""Episode-side client of the simulator servers (upstream ``pear/sim/client.py:53-86``): opens an episode on a server
of its family, forwards steps, and turns every infrastructure failure into ``EpisodeLost`` so the agent loop can
restart the trajectory. Stateless families keep the action history here and replay it on every call."""

from __future__ import annotations

import uuid
from typing import Optional

from .env import EpisodeLost
from .server import Server, ServerPool


class EpisodeClient:
    def __init__(self, pool: ServerPool, family: str):
        self.server: Server = pool.get(family)
        self.family = family
        self.episode_id = uuid.uuid4().hex
        self.args: Optional[dict] = None
        self.actions: list[dict] = []
        self.slot = None

    def open(self, args: dict) -> dict:
        self.args, self.actions = dict(args), []
        if self.server.mode == "stateless":
            return self.server.rollout(self.args, [])
        self.slot = self.server.acquire(self.episode_id)
        try:
            return self.server._call(self.slot, "open", (self.episode_id, self.args))
        except EpisodeLost:
            self._drop_slot()
            raise

    def step(self, action: dict) -> dict:
        self.actions.append(action)
        if self.server.mode == "stateless":
            return self.server.rollout(self.args, self.actions)
        if self.slot is None:
            raise EpisodeLost("episode has no process")
        try:
            return self.server._call(self.slot, "step", (self.episode_id, action))
        except EpisodeLost:
            self._drop_slot()
            raise

    def close(self) -> None:
        if self.slot is not None:
            try:
                self.server._call(self.slot, "close", (self.episode_id,), timeout_s=5.0)
            except (EpisodeLost, RuntimeError):
                pass
            self._drop_slot()

    def _drop_slot(self) -> None:
        if self.slot is not None:
            self.server.release(self.slot)
            self.slot = None

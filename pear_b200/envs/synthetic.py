"""Seeded synthetic environment family.

Stands in for the simulator families of upstream ``pear/envs/{libero*,robodojo,robolab}`` (MuJoCo / Isaac Sim behind a
graphics stack) with the same contract and shapes: an episode is described by its arguments (task, seed, horizon), an
observation carries a JSON-able state, one frame per camera and a reminder, an action is a JSON object checked against
a schema, the reward is the episode's success flag. Frames are blocks of N(0, 1) vision-embedding placeholders
(``[tokens_per_image, hidden]``) instead of rendered pixels, drawn from the episode's seed, so rollouts are
reproducible and no renderer is needed.

The task is solvable, so rewards are not constant: the state holds a hidden target in ``[0, 10)`` and a cursor; the
action ``{"move": d}`` with ``d`` in {-1, 0, +1} moves the cursor, ``{"submit": true}`` ends the episode, success iff
the cursor sits on the target (whose distance is revealed in the state).
"""

from __future__ import annotations

import numpy as np

from ..sim.env import BaseEnv


class SyntheticEnv(BaseEnv):
    family = "synthetic"

    def __init__(self, cameras: tuple[str, ...] = ("front",), tokens_per_image: int = 16, hidden: int = 64,
                 fail_after: int = -1, hang_after: int = -1, pixels: int = 0):
        """``pixels`` > 0: the cameras deliver ``[pixels, pixels, 3]`` uint8 pictures (the agent loop's vision encoder turns them
        into embedding rows) instead of finished embedding blocks; the picture changes only when the cursor moves."""
        self.cameras, self.tokens_per_image, self.hidden, self.pixels = tuple(cameras), tokens_per_image, hidden, int(pixels)
        # host-side fault injection for the supervision tests: raise / sleep after this many steps
        self.fail_after, self.hang_after = fail_after, hang_after
        self.rng = np.random.default_rng(0)
        self.t = 0

    @classmethod
    def action_schema(cls) -> dict:
        return {"type": "object", "properties": {"move": {"type": "integer", "minimum": -1, "maximum": 1},
                                                 "submit": {"type": "boolean"}},
                "additionalProperties": False, "minProperties": 1}

    def _observe(self) -> dict:
        if self.pixels:
            frames = {}
            for ci, cam in enumerate(self.cameras):  # a function of (task seed, camera, cursor): a scene that did not move looks the same
                g = np.random.default_rng([self.target, ci, self.cursor])
                frames[cam] = g.integers(0, 256, (self.pixels, self.pixels, 3), dtype=np.uint8)
        else:
            frames = {cam: self.rng.standard_normal((self.tokens_per_image, self.hidden)).astype(np.float32) for cam in self.cameras}
        state = {"task": self.task, "step": self.t, "cursor": self.cursor, "distance": self.target - self.cursor,
                 "horizon": self.horizon}
        return {"state": state, "frames": frames, "reminder": "Answer with one JSON action in a ```json block."}

    def reset(self, args: dict) -> dict:
        self.task = str(args.get("task", "reach"))
        self.horizon = int(args.get("horizon", 8))
        self.rng = np.random.default_rng(int(args.get("seed", 0)))
        self.target = int(self.rng.integers(0, 10))
        self.cursor = int(self.rng.integers(0, 10))
        self.t = 0
        first = self._observe()
        # said once, in the system prompt of the episode: what the cameras show and what is to be done
        first["environment"] = [f"{cam}: a synthetic camera; its picture changes only when the cursor moves" for cam in self.cameras] + [
            "the episode ends by itself when you submit or when the horizon is reached"]
        first["task"] = f"{self.task}: move the cursor until the distance is 0, then submit"
        return first

    def step(self, action: dict) -> tuple[dict, bool, bool, dict]:
        self.t += 1
        if 0 <= self.fail_after < self.t:
            raise RuntimeError("synthetic environment failure (injected)")
        if 0 <= self.hang_after < self.t:
            import time
            time.sleep(3600)
        done = bool(action.get("submit", False))
        self.cursor = int(np.clip(self.cursor + int(action.get("move", 0)), 0, 9))
        if self.t >= self.horizon:
            done = True
        success = done and self.cursor == self.target
        return self._observe(), done, success, {"steps": self.t}

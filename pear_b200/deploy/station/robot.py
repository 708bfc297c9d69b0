"""What the station's agent loop needs of a robot, and a simulated arm that offers it.

Upstream's station drives real arms (YAM, SO-101: pear/deploy/station/control/**) behind one robot interface that the agent
loop uses: wait until the arms rest, observe (camera frames + joint state), execute one Cartesian action from the observed
pose and report how it ended, stop. That hardware is not here; the interface is, with ``SimulatedArm`` behind it: a gripper in
a box-shaped workspace with one top camera, enough to run the whole deployment chain (station loop -> model client -> harness
-> model server) and its records on a CPU box.
"""

from __future__ import annotations

import math
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

COMPLETED, REJECTED, FAILED, STOPPED = "completed", "rejected", "failed", "stopped"


@dataclass(frozen=True)
class ActionFormat:
    """The parts of an action and each part's quantities, exactly as the model must write them, with a bound per quantity."""

    name: str
    schema: dict  # part -> tuple of quantity names
    bounds: dict = field(default_factory=dict)  # "part.quantity" -> (low, high)

    def describe(self) -> str:
        lines = [f'  "{p}": {{' + ", ".join(f'"{q}": <number>' for q in qs) + "}" for p, qs in self.schema.items()]
        return "```json\n{\n" + ",\n".join(lines) + "\n}\n```"

    def result_feedback(self, result: "MotionResult", dispatched: bool) -> str:
        """What the next turn tells the model of the last action."""
        if result.status == COMPLETED:
            return "The last action completed."
        where = "was sent to the robot and" if dispatched else "was not sent to the robot: it"
        return f"The last action {where} ended as {result.status}: {result.detail}"


CARTESIAN = ActionFormat("cartesian_delta", {"arm": ("dx", "dy", "dz"), "gripper": ("opening",)},
                         {"arm.dx": (-0.2, 0.2), "arm.dy": (-0.2, 0.2), "arm.dz": (-0.2, 0.2), "gripper.opening": (0.0, 1.0)})


@dataclass
class Observation:
    observation_id: str
    captured_s: float
    cameras: dict  # camera name -> uint8 [H, W, 3]
    state: dict  # what the model reads of the robot, as numbers


@dataclass
class MotionResult:
    status: str
    detail: str
    state: dict
    seconds: float = 0.0

    def to_record(self) -> dict:
        return {"status": self.status, "detail": self.detail, "state": self.state, "seconds": round(self.seconds, 4)}


class Robot:
    """The interface of the agent loop's robot."""

    action_format: ActionFormat = CARTESIAN

    def wait_stationary(self, cancellation: Optional[threading.Event] = None) -> None: ...
    def observe(self) -> Observation: ...
    def execute(self, action: dict, cancellation: Optional[threading.Event] = None) -> MotionResult: ...
    def stop(self) -> None: ...

    def failure_result(self, error: BaseException, status: str = FAILED) -> MotionResult:
        return MotionResult(status, str(error), self.observe().state)


class SimulatedArm(Robot):
    """A gripper at (x, y, z) in the unit box and a target on the table; one camera looks down. An action moves the gripper by
    (dx, dy, dz) in steps of ``speed`` per tick and sets its opening; a move that would leave the workspace is rejected whole."""

    def __init__(self, start=(0.2, 0.2, 0.5), target=(0.7, 0.6, 0.0), speed: float = 0.05, tick_s: float = 0.0, image: int = 64):
        self.pos, self.opening = np.array(start, dtype=np.float64), 1.0
        self.target, self.speed, self.tick_s, self.image = np.array(target, dtype=np.float64), speed, tick_s, image
        self._halt = threading.Event()
        self.moves = 0

    def wait_stationary(self, cancellation=None) -> None:
        return None  # every execute returns at rest

    def state(self) -> dict:
        return {"x": round(float(self.pos[0]), 4), "y": round(float(self.pos[1]), 4), "z": round(float(self.pos[2]), 4), "opening": round(self.opening, 3)}

    def observe(self) -> Observation:
        n = self.image
        frame = np.full((n, n, 3), 235, dtype=np.uint8)

        def dot(p, color, r):
            cy, cx = int(p[1] * (n - 1)), int(p[0] * (n - 1))
            frame[max(cy - r, 0):cy + r + 1, max(cx - r, 0):cx + r + 1] = color

        dot(self.target, (30, 160, 30), 3)
        dot(self.pos, (200, 40, 40), 2 + int(3 * self.opening))
        return Observation(str(uuid.uuid4()), time.monotonic(), {"top": frame}, self.state())

    def distance(self) -> float:
        return float(np.linalg.norm(self.pos[:2] - self.target[:2]))

    def execute(self, action: dict, cancellation=None) -> MotionResult:
        t0 = time.time()
        self._halt.clear()
        delta = np.array([action["arm"]["dx"], action["arm"]["dy"], action["arm"]["dz"]], dtype=np.float64)
        goal = self.pos + delta
        if (goal < 0).any() or (goal > 1).any():
            return MotionResult(REJECTED, f"the move would leave the workspace (goal {np.round(goal, 3).tolist()})", self.state(), time.time() - t0)
        steps = max(1, math.ceil(float(np.linalg.norm(delta)) / self.speed))
        for _ in range(steps):
            if self._halt.is_set() or (cancellation is not None and cancellation.is_set()):
                return MotionResult(STOPPED, "the move was stopped on the way", self.state(), time.time() - t0)
            self.pos = self.pos + delta / steps
            if self.tick_s:
                time.sleep(self.tick_s)
        self.opening = float(action["gripper"]["opening"])
        self.moves += 1
        return MotionResult(COMPLETED, "", self.state(), time.time() - t0)

    def stop(self) -> None:
        self._halt.set()

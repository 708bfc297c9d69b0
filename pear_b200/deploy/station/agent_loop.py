"""A task's model session on a robot: each step observes the robot at rest, asks the model, reads the action at the end of its
answer and has the robot execute it; the conversation itself is the client's (pear/deploy/station/agent_loop/agent_loop.py:
146-346 upstream).

What a step guarantees: one step at a time; nothing reaches the robot unless the whole answer parsed as an action of the
format; the robot is stopped on every way out that is not a completed action; a model that takes longer than ``timeout_s`` or
an operator's cancellation ends the model request itself (the client's ``cancel``), not just the wait for it; a conversation
that cannot go on (context limit, lost session) blocks every later step with its reason; every turn leaves a record (the
frames the model saw as JPEG files, and one JSON line with the state, the text, the answer, the action and the result), and the
next turn tells the model how the last action ended.
"""

from __future__ import annotations

import json
import os
import threading
import time
import uuid
from dataclasses import dataclass
from typing import Callable, Optional

from .action_parser import parse_action
from .clients import ContextLimit, ModelClient, ModelInput, ModelOutput, SessionLost
from .robot import COMPLETED, FAILED, REJECTED, STOPPED, ActionFormat, MotionResult, Robot


class OperatorPaused(RuntimeError):
    """The operator stopped the step."""


def system_prompt(instruction: str, fmt: ActionFormat) -> str:
    return (f"You control a robot arm. The task: {instruction}\n\nEvery turn you are shown the robot's state and its camera pictures. Reason briefly, then end your "
            f"answer with exactly one fenced json block holding the next action in this form and nothing after it:\n{fmt.describe()}\n"
            "Quantities are metres (arm) and a fraction (gripper opening). A move that would leave the workspace is refused.")


@dataclass
class Turn:
    attempt_id: str
    model_input: ModelInput
    model_output: Optional[ModelOutput] = None
    action: Optional[dict] = None
    dispatched: bool = False
    result: Optional[MotionResult] = None


class StationAgentLoop:
    def __init__(self, robot: Robot, client: ModelClient, action_format: ActionFormat, timeout_s: float, directory: str, reference_images: tuple = ()):
        if not (timeout_s > 0 and timeout_s < float("inf")):
            raise ValueError("Model timeout must be finite and positive")
        self.robot, self.client, self.action_format, self.timeout_s = robot, client, action_format, timeout_s
        self.directory, self.reference_images = str(directory), tuple(reference_images)
        os.makedirs(self.directory, exist_ok=True)
        self.episode_id = str(uuid.uuid4())
        self.turn_count = 0
        self.last_turn: Optional[Turn] = None
        self.previous_result: Optional[MotionResult] = None
        self.blocked_reason: Optional[str] = None
        self._feedback: Optional[str] = None
        self._request_cancellation = threading.Event()
        self._step_lock = threading.Lock()

    # -- one step -----------------------------------------------------------------------------------------------------------
    def step(self, cancellation: threading.Event, on_event: Callable[[str, dict], None], attempt_id: Optional[str] = None) -> MotionResult:
        if not self._step_lock.acquire(blocking=False):
            raise RuntimeError("A model step is already running")
        turn = None
        self._request_cancellation = threading.Event()
        try:
            self._check(cancellation)
            if self.blocked_reason:
                raise ContextLimit(self.blocked_reason)
            attempt_id = attempt_id or str(uuid.uuid4())
            on_event("phase", {"phase": "observing"})
            self.robot.wait_stationary(cancellation)
            obs = self.robot.observe()
            turn = self.last_turn = Turn(attempt_id, self._model_input(obs, attempt_id))
            self.turn_count += 1
            on_event("observation", {"turn_id": attempt_id, "observation_id": obs.observation_id, "state": obs.state, "text": turn.model_input.text,
                                     "previous_result": self.previous_result.to_record() if self.previous_result else None})
            on_event("phase", {"phase": "thinking"})
            turn.model_output = self._call_model(turn, cancellation, on_event)
            on_event("model_output", {"answer": turn.model_output.answer, "seconds": turn.model_output.seconds})
            self._check(cancellation)
            turn.action = parse_action(turn.model_output.answer, self.action_format)
            on_event("action", turn.action)
            self._check(cancellation)
            turn.dispatched = True
            on_event("phase", {"phase": "moving"})
            result = self.robot.execute(turn.action, cancellation)
            if result.status != COMPLETED:
                self.robot.stop()
            return self._record(turn, result)
        except (ContextLimit, SessionLost) as e:
            self.blocked_reason = str(e)
            self.robot.stop()
            if turn is not None:
                self._record(turn, self.robot.failure_result(e))
            raise
        except OperatorPaused as e:
            self.robot.stop()
            if turn is not None:
                self._record(turn, self.robot.failure_result(e, STOPPED))
            raise
        except Exception as e:  # noqa: BLE001 - the turn ends without a completed action; the session goes on
            self.robot.stop()
            if turn is None:
                raise
            return self._record(turn, self.robot.failure_result(e, REJECTED if isinstance(e, ValueError) else FAILED))
        except BaseException:
            self.robot.stop()
            raise
        finally:
            self._step_lock.release()

    def close(self) -> None:
        self._request_cancellation.set()
        self.client.cancel()
        if not self._step_lock.acquire(timeout=ModelClient.CLEANUP_TIMEOUT_S):
            raise RuntimeError("Model step still running; cleanup incomplete")
        try:
            self.client.close()
        finally:
            self._step_lock.release()

    # -- parts --------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _check(cancellation: threading.Event) -> None:
        if cancellation.is_set():
            raise OperatorPaused("The operator stopped the step")

    def _model_input(self, obs, attempt_id: str) -> ModelInput:
        from PIL import Image

        for name, frame in obs.cameras.items():  # the frames the model is shown, kept with the task
            Image.fromarray(frame).save(os.path.join(self.directory, f"{self.turn_count:04d}_{attempt_id}_{name}.jpg"), "JPEG")
        lines = [f"Turn {self.turn_count + 1}."]
        if self._feedback:
            lines.append(self._feedback)
        lines.append("State: " + json.dumps(obs.state))
        return ModelInput("\n".join(lines), dict(obs.cameras), self.reference_images)

    def _call_model(self, turn: Turn, cancellation: threading.Event, on_event) -> ModelOutput:
        """The client's ``infer`` on a thread of its own, watched for the timeout and the operator's stop; either one ends the
        request itself and waits for the thread, so no answer arrives after the step has moved on."""
        box: dict = {}

        def work():
            try:
                box["out"] = self.client.infer(turn.model_input, on_event, self._request_cancellation)
            except BaseException as e:  # noqa: BLE001
                box["err"] = e

        th = threading.Thread(target=work, daemon=True)
        th.start()
        t0 = t_stop = time.time()
        stopped: Optional[BaseException] = None
        while th.is_alive():
            th.join(0.02)
            if stopped is None and cancellation.is_set():
                stopped = OperatorPaused("The operator stopped the step")
            elif stopped is None and time.time() - t0 > self.timeout_s:
                stopped = TimeoutError(f"The model did not answer within {self.timeout_s:g} s")
            if stopped is not None and not self._request_cancellation.is_set():
                self._request_cancellation.set()
                self.client.cancel()
                t_stop = time.time()
            if stopped is not None and time.time() - t_stop > ModelClient.CLEANUP_TIMEOUT_S:
                break
        if stopped is not None:
            raise stopped
        if "err" in box:
            raise box["err"]
        return box["out"]

    def _record(self, turn: Turn, result: MotionResult) -> MotionResult:
        turn.result = result
        self.previous_result = result
        self._feedback = self.action_format.result_feedback(result, turn.dispatched)
        rec = {"episode_id": self.episode_id, "turn": self.turn_count, "attempt_id": turn.attempt_id, "text": turn.model_input.text,
               "answer": turn.model_output.answer if turn.model_output else None, "model_seconds": turn.model_output.seconds if turn.model_output else None,
               "usage": turn.model_output.usage if turn.model_output else None, "action": turn.action, "dispatched": turn.dispatched, "result": result.to_record()}
        with open(os.path.join(self.directory, "turns.jsonl"), "a") as f:
            f.write(json.dumps(rec) + "\n")
        return result

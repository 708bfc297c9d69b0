"""Replay buffer of the separate-async trainer: prompt groups in flight, staleness, DAPO filtering, session caps.

Behaviour of upstream ``pear/trainer/replay_buffer.py`` (over verl's ``ReplayBufferAsync``) and the hooks of patches
0005/0007/0008:
  * a prompt group = ``n`` sessions of one prompt; it is sampleable once all its sessions are sealed in the queue;
  * ``is_stale``: a group whose issuing policy version is more than ``max_off_policy_threshold - 1`` versions behind
    the trainer is dropped (threshold 5 = staleness <= 4 plus the issuing version) and replaced;
  * the DAPO filter evicts groups whose rewards have no variance and refills one for one;
  * two refills while waiting: for evicted groups and for free room under the global / per-tool caps of sessions kept
    generating (``_refill_free_room`` :64-77, ``_inflight_sessions`` :79-91);
  * restored groups wait as QUEUED and are refilled before fresh prompts (:14);
  * pass-rate metrics avg@n / zero / one, overall and per tool (:93-113).
"""

from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Optional

import torch

from . import grpo


class GroupStatus(str, Enum):
    QUEUED = "queued"        # restored from a snapshot, not yet re-issued
    IN_FLIGHT = "in_flight"
    FINISHED = "finished"
    CONSUMED = "consumed"
    DROPPED = "dropped"


@dataclass
class PromptGroup:
    uid: str
    prompt: dict
    n: int
    issued_version: int
    tool: Optional[str] = None
    status: GroupStatus = GroupStatus.IN_FLIGHT
    session_ids: list[str] = field(default_factory=list)
    unfinished: Optional[list[str]] = None  # resume: only these sessions are (re-)run
    rewards: Optional[list[float]] = None

    def keys(self) -> list[str]:
        return [f"{self.uid}/{s}" for s in self.session_ids]


class ReplayBuffer:
    def __init__(self, queue, n: int, max_off_policy_threshold: int = 5, max_off_policy_strategy: str = "drop",
                 filter_groups: bool = True, max_inflight_sessions: Optional[int] = None,
                 tool_session_caps: Optional[dict[str, int]] = None):
        self.queue, self.n = queue, n
        self.threshold, self.strategy = max_off_policy_threshold, max_off_policy_strategy
        self.filter_groups = filter_groups
        self.max_inflight_sessions = max_inflight_sessions
        self.tool_caps = dict(tool_session_caps or {})
        self.groups: "OrderedDict[str, PromptGroup]" = OrderedDict()
        self.metrics: dict[str, float] = {}
        self.dropped_stale = self.evicted_filtered = 0
        self._judged: list[tuple[Optional[str], list[float]]] = []

    # -- bookkeeping --------------------------------------------------------------------------------------------------
    def add_group(self, g: PromptGroup) -> None:
        if not g.session_ids:
            g.session_ids = [str(i) for i in range(g.n)]
        self.groups[g.uid] = g

    def is_stale(self, g: PromptGroup, step_version: int) -> bool:
        return step_version - g.issued_version >= self.threshold

    def inflight_sessions(self, tool: Optional[str] = None) -> int:
        """Sessions being generated: every in-flight group counts as its ``n`` sessions (or its unfinished ones)."""
        total = 0
        for g in self.groups.values():
            if g.status != GroupStatus.IN_FLIGHT or (tool is not None and g.tool != tool):
                continue
            total += len(g.unfinished) if g.unfinished is not None else g.n
        return total

    def free_room(self, tool: Optional[str] = None) -> int:
        """How many more GROUPS may be issued under the global cap and (if given) the tool's cap."""
        rooms = []
        if self.max_inflight_sessions is not None:
            rooms.append((self.max_inflight_sessions - self.inflight_sessions()) // self.n)
        if tool is not None and tool in self.tool_caps:
            rooms.append((self.tool_caps[tool] - self.inflight_sessions(tool)) // self.n)
        return max(0, min(rooms)) if rooms else 1 << 30

    def queued(self) -> list[PromptGroup]:
        return [g for g in self.groups.values() if g.status == GroupStatus.QUEUED]

    # -- completion ---------------------------------------------------------------------------------------------------
    def _collect_finished(self) -> None:
        for g in self.groups.values():
            if g.status != GroupStatus.IN_FLIGHT:
                continue
            if all(self.queue.has(k) for k in g.keys()):
                g.rewards = [float(self.queue.get(k)["reward"]) for k in g.keys()]
                g.status = GroupStatus.FINISHED
                g.unfinished = None

    def _judge(self, g: PromptGroup) -> bool:
        """DAPO: keep a finished group only when its rewards vary. Records the pass-rate sample either way."""
        self._judged.append((g.tool, list(g.rewards)))
        if not self.filter_groups:
            return True
        return max(g.rewards) - min(g.rewards) > 0

    def _drop(self, g: PromptGroup, status: GroupStatus = GroupStatus.DROPPED) -> None:
        self.queue.clear(g.keys())
        g.status = status

    # -- sampling -----------------------------------------------------------------------------------------------------
    def sample(self, step_version: int, batch_groups: int, refill: Optional[Callable[[int, bool], int]] = None,
               timeout_s: float = 600.0, poll_s: float = 0.01, progress: Optional[Callable[[], None]] = None) -> list[PromptGroup]:
        """Block until ``batch_groups`` usable groups exist, then hand them out (oldest first).

        ``refill(k, evicted)``: ask the trainer to issue up to ``k`` more groups (``evicted``: replacements of dropped
        groups, otherwise free room under the caps); it returns how many it issued. ``progress`` is called while
        waiting (a synchronous driver steps the rollout engine there).
        """
        deadline = time.time() + timeout_s
        usable: list[PromptGroup] = []
        while True:
            self._collect_finished()
            need_replacement = 0
            for g in list(self.groups.values()):
                if g.status == GroupStatus.FINISHED and g not in usable:
                    if self.is_stale(g, step_version) and self.strategy == "drop":
                        self._drop(g)
                        self.dropped_stale += 1
                        need_replacement += 1
                    elif not self._judge(g):
                        self._drop(g)
                        self.evicted_filtered += 1
                        need_replacement += 1
                    else:
                        usable.append(g)
                elif g.status == GroupStatus.IN_FLIGHT and self.is_stale(g, step_version) and self.strategy == "drop":
                    # an unfinished group already too old to ever train: its sessions are cancelled by the trainer
                    self._drop(g)
                    self.dropped_stale += 1
                    need_replacement += 1
            if len(usable) >= batch_groups:
                break
            if refill is not None:
                if need_replacement:
                    refill(need_replacement, True)
                room = self.free_room()
                pending = sum(1 for g in self.groups.values() if g.status == GroupStatus.IN_FLIGHT)
                short = batch_groups - len(usable) - pending
                if room > 0 and (short > 0 or self.max_inflight_sessions is not None):
                    refill(min(room, max(short, 1)) if self.max_inflight_sessions is None else room, False)
            if progress is not None:
                progress()
            else:
                time.sleep(poll_s)
            if time.time() > deadline:
                raise TimeoutError(f"replay buffer: {len(usable)}/{batch_groups} groups after {timeout_s}s")
        out = usable[:batch_groups]
        for g in out:
            g.status = GroupStatus.CONSUMED
        self._flush_metrics()
        return out

    def release(self, groups: list[PromptGroup]) -> None:
        """After the step trained on them: clear their trajectories from the queue and forget them."""
        for g in groups:
            self.queue.clear(g.keys())
            self.groups.pop(g.uid, None)
        for uid in [u for u, g in self.groups.items() if g.status == GroupStatus.DROPPED]:
            self.groups.pop(uid)

    # -- metrics ------------------------------------------------------------------------------------------------------
    def _flush_metrics(self) -> None:
        if not self._judged:
            return
        n = self.n
        allr = torch.tensor([r for _, r in self._judged if len(r) == n])
        self.metrics = {}
        if allr.numel():
            self.metrics.update(grpo.pass_rate_metrics(allr, "train/filter_groups"))
        tools = sorted({t for t, _ in self._judged if t is not None})
        for t in tools:
            tr = torch.tensor([r for tt, r in self._judged if tt == t and len(r) == n])
            if tr.numel():
                for k, v in grpo.pass_rate_metrics(tr, "train/filter_groups").items():
                    self.metrics[f"{k}/{t}"] = v
        self.metrics["train/dropped_stale"] = float(self.dropped_stale)
        self.metrics["train/evicted_filtered"] = float(self.evicted_filtered)
        self._judged = []

    # -- snapshot / resume --------------------------------------------------------------------------------------------
    def state(self) -> dict:
        return {"groups": [dict(uid=g.uid, prompt=g.prompt, n=g.n, issued_version=g.issued_version, tool=g.tool,
                                status=g.status.value, session_ids=g.session_ids) for g in self.groups.values()
                           if g.status in (GroupStatus.IN_FLIGHT, GroupStatus.FINISHED, GroupStatus.QUEUED)]}

    def restore(self, state: dict, step_version: int) -> dict:
        """Rebuild in-flight groups from a snapshot taken before a crash: sessions already sealed in the queue are
        kept, the others are marked unfinished, groups already too stale restart from scratch as fresh prompts, and
        trajectories whose group is gone are cleared. Restored groups wait as QUEUED."""
        report = {"kept_sessions": 0, "rerun_sessions": 0, "restarted_groups": 0, "cleared_orphans": 0}
        self.groups.clear()
        known = set()
        for d in state["groups"]:
            g = PromptGroup(d["uid"], d["prompt"], d["n"], d["issued_version"], d.get("tool"), GroupStatus.QUEUED, d["session_ids"])
            if self.is_stale(g, step_version):
                self.queue.clear(g.keys())
                g.issued_version = step_version
                g.unfinished = None
                report["restarted_groups"] += 1
            else:
                done = [s for s in g.session_ids if self.queue.has(f"{g.uid}/{s}")]
                g.unfinished = [s for s in g.session_ids if s not in done]
                report["kept_sessions"] += len(done)
                report["rerun_sessions"] += len(g.unfinished)
            self.groups[g.uid] = g
            known.update(g.keys())
        for k in self.queue.keys(sealed_only=False):
            if k not in known:
                self.queue.clear([k])
                report["cleared_orphans"] += 1
        return report

"""The training loop: rollout -> replay buffer -> GRPO step -> weight sync -> checkpoint.

Two modes, as in upstream ``pear/trainer/trainer.py:120-313`` (``trainer.v1.trainer_mode``):

* ``sync``: a step issues exactly its batch of prompt groups, waits for them, trains, synchronises weights.
* ``separate_async``: rollout replicas keep generating under session caps while the trainer trains; a group is usable
  while its issuing policy version is at most ``max_off_policy_threshold - 1`` versions old; stale groups are dropped
  and replaced; groups whose rewards are all equal are filtered (DAPO) and replaced.

Resume (``_reissue_prompt_groups`` ``:159-244``): the replay buffer and the transfer queue come back from the
checkpoint; sealed sessions are kept, unfinished sessions are re-run, half-written keys were dropped by the queue,
groups already too stale restart as fresh prompts; restored groups are re-issued before fresh ones (``:251-297``).
The run end cancels background groups (``runner.py:44-53``).
"""

from __future__ import annotations

import itertools
import logging
import os
import time
import uuid
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch

from ..utils import nvtx
from . import grpo
from .engine import PackedBatch, TrainEngine
from .replay_buffer import GroupStatus, PromptGroup, ReplayBuffer


@dataclass
class TrainerConfig:
    total_training_steps: int = 1
    train_batch_size: int = 4            # prompt groups per step
    ppo_mini_batch_size: int = 0         # prompt groups per optimizer step (0 or >= the batch: one update per step)
    n: int = 4                           # sessions per group
    trainer_mode: str = "separate_async"
    parameter_sync_step: int = 1
    max_token_len_per_gpu: int = 69632
    save_freq: int = -1
    norm_adv_by_std: bool = True
    sample_timeout_s: float = 600.0
    topk_heads: int = 0

    @classmethod
    def from_config(cls, cfg) -> "TrainerConfig":
        tr, v1 = cfg.trainer, cfg.trainer.v1
        return cls(total_training_steps=int(tr.total_training_steps), train_batch_size=int(cfg.data.train_batch_size),
                   ppo_mini_batch_size=int(cfg.actor_rollout_ref.actor.get("ppo_mini_batch_size", 0) or 0),
                   n=int(cfg.actor_rollout_ref.rollout.n), trainer_mode=str(v1.trainer_mode),
                   parameter_sync_step=int(v1.separate_async.parameter_sync_step),
                   max_token_len_per_gpu=int(cfg.actor_rollout_ref.actor.ppo_max_token_len_per_gpu), save_freq=int(tr.save_freq),
                   norm_adv_by_std=bool(cfg.algorithm.norm_adv_by_std_in_grpo),
                   topk_heads=int(cfg.actor_rollout_ref.rollout.get("topk_log_probs", 0)))


def trajectory_to_rows(tr: dict, advantage: float, hidden: int, topk: int, train_vision: bool = False):
    """One trajectory -> per-token training rows (inputs t, labels t+1). ``train_vision``: blocks that came from pictures are
    handed over as pictures (the trainer's tower computes their rows with gradients), the others as finished rows."""
    tokens = torch.from_numpy(np.asarray(tr["tokens"])).long()
    n = tokens.numel()
    mask = torch.from_numpy(np.asarray(tr["response_mask"])).float()
    lp = torch.from_numpy(np.asarray(tr["rollout_logprobs"])).float()
    labels = torch.cat([tokens[1:], tokens[:1]])
    loss_mask = torch.cat([mask[1:], mask.new_zeros(1)])       # position t is trained iff token t+1 was sampled
    slp = torch.cat([lp[1:], lp.new_zeros(1)])
    pos = tr.get("position_ids")  # [3, n] when the rollout used the checkpoint's picture positions
    out = dict(input_ids=tokens, position_ids=torch.arange(n) if pos is None else torch.from_numpy(np.asarray(pos)).long(), labels=labels, loss_mask=loss_mask,
               advantages=torch.full((n,), float(advantage)) * loss_mask, sampler_log_probs=slp)
    if topk > 0:
        ids = torch.from_numpy(np.asarray(tr["topk_ids"])).reshape(n, -1)[:, :topk]
        hlp = torch.from_numpy(np.asarray(tr["topk_logprobs"])).float().reshape(n, -1)[:, :topk]
        out["head_ids"] = torch.cat([ids[1:], ids[:1]]).int()
        out["head_log_probs"] = torch.cat([hlp[1:], hlp[:1]])
    from_pixels = {int(p) for p, _ in tr.get("images", [])} if train_vision else set()
    if from_pixels:
        out["images"] = [(int(p), torch.from_numpy(np.ascontiguousarray(img))) for p, img in tr["images"]]
    if tr.get("embeds") and any(int(p) not in from_pixels for p, _ in tr["embeds"]):
        e = torch.zeros(n, hidden)
        m = torch.zeros(n, dtype=torch.bool)
        for pos, block in tr["embeds"]:
            if int(pos) in from_pixels:
                continue
            b = torch.from_numpy(np.asarray(block, dtype=np.float32))
            e[pos:pos + b.shape[0]] = b
            m[pos:pos + b.shape[0]] = True
        out["inputs_embeds"], out["embeds_mask"] = e, m
    return out


def pack_rows(rows: list[dict]) -> PackedBatch:
    cu = [0]
    for r in rows:
        cu.append(cu[-1] + r["input_ids"].numel())
    def cat(k):
        if any(k not in r for r in rows):
            if all(k not in r for r in rows):
                return None
            raise ValueError(f"field {k} present in some trajectories only")
        return torch.cat([r[k] for r in rows])
    emb, em = None, None
    if any("inputs_embeds" in r for r in rows):
        h = next(r["inputs_embeds"].shape[1] for r in rows if "inputs_embeds" in r)
        emb = torch.cat([r.get("inputs_embeds", torch.zeros(r["input_ids"].numel(), h)) for r in rows])
        em = torch.cat([r.get("embeds_mask", torch.zeros(r["input_ids"].numel(), dtype=torch.bool)) for r in rows])
    images = [(cu[i] + pos, img) for i, r in enumerate(rows) for pos, img in r.get("images", [])]
    positions = [r["position_ids"] for r in rows]
    if any(p.dim() == 2 for p in positions):  # some sequences carry (temporal, row, column) positions: all three axes for everyone
        positions = torch.cat([p if p.dim() == 2 else p.expand(3, -1) for p in positions], dim=1)
    else:
        positions = torch.cat(positions)
    return PackedBatch(cat("input_ids"), positions, cu, cat("labels"), cat("loss_mask"), cat("advantages"),
                       sampler_log_probs=cat("sampler_log_probs"), head_ids=cat("head_ids"), head_log_probs=cat("head_log_probs"),
                       inputs_embeds=emb, embeds_mask=em, images=images or None)


def balanced_partition(sizes: list[int], parts: int) -> list[list[int]]:
    """Longest-first greedy: indices per part with near-equal token sums (data-parallel ranks do equal work)."""
    bins: list[list[int]] = [[] for _ in range(parts)]
    load = [0] * parts
    for i in sorted(range(len(sizes)), key=lambda j: -sizes[j]):
        b = min(range(parts), key=lambda j: load[j])
        bins[b].append(i)
        load[b] += sizes[i]
    return [sorted(b) for b in bins]


def micro_batches(rows: list[dict], max_tokens: int) -> list[list[dict]]:
    out: list[list[dict]] = [[]]
    size = 0
    for r in rows:
        n = r["input_ids"].numel()
        if out[-1] and size + n > max_tokens:
            out.append([])
            size = 0
        out[-1].append(r)
        size += n
    return [mb for mb in out if mb]


_log = logging.getLogger("pear_b200.trainer")

# dense bf16 peak FLOP/s per device name (nominal; a measured peak file beside the package overrides the entry of the GPU
# the process runs on). Upstream keeps such a table in verl's flops counter (patch 0016: GB300 = 2.5e15).
DEVICE_PEAK_FLOPS = {"B200": 2.25e15, "GB200": 2.5e15, "GB300": 2.5e15, "H100": 0.989e15, "H200": 0.989e15, "A100": 0.312e15}


def device_peak_flops(name: Optional[str] = None) -> float:
    if name is None:
        name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    measured = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if "B200" in name and os.path.exists(measured):
        try:
            import json

            return float(json.load(open(measured))["bf16_tflops_sustained"]) * 1e12
        except (OSError, KeyError, ValueError):
            pass
    for key, val in DEVICE_PEAK_FLOPS.items():
        if key in name:
            return val
    return 1e12  # unknown device (CPU tests): the ratio is then only a scaled throughput


class Trainer:
    def __init__(self, cfg: TrainerConfig, engine: TrainEngine, dataset, manager, replay: ReplayBuffer, queue, weight_sync=None,
                 checkpoints=None, log: Optional[Callable[[int, dict], None]] = None, progress: Optional[Callable[[], None]] = None):
        self.cfg, self.engine, self.dataset, self.manager = cfg, engine, dataset, manager
        self.replay, self.queue, self.weight_sync, self.checkpoints = replay, queue, weight_sync, checkpoints
        self.log = log or (lambda step, m: None)
        self.progress = progress
        self.step = 0
        self._uid = itertools.count()
        self.run_id = uuid.uuid4().hex[:6]
        self.history: list[dict] = []
        # With several trainer ranks, rank 0 drives: it owns the replay buffer, the agent-loop manager and the weight sync,
        # builds every data-parallel rank's micro-batches and broadcasts them; the other ranks only compute.
        self.is_driver = engine.rank == 0

    # -- issuing prompt groups ----------------------------------------------------------------------------------------
    def _issue(self, g: PromptGroup) -> None:
        sessions = g.unfinished if g.unfinished is not None else g.session_ids
        g.status = GroupStatus.IN_FLIGHT
        g.unfinished = None
        if sessions:
            self.manager.dispatch_group(g.uid, g.prompt["family"], g.prompt["env_args"], list(sessions))

    def _refill(self, k: int, evicted: bool) -> int:
        issued = 0
        for g in self.replay.queued():                 # restored groups first
            if issued >= k:
                return issued
            self._issue(g)
            issued += 1
        while issued < k:
            row = self.dataset.next()
            g = PromptGroup(uid=f"{self.run_id}-{next(self._uid)}", prompt={"family": row.family, "env_args": row.env_args},
                            n=self.cfg.n, issued_version=self.engine.policy_version, tool=row.tool)
            self.replay.add_group(g)
            self._issue(g)
            issued += 1
        return issued

    def _while_waiting(self) -> None:
        """Called by the replay buffer while it waits for groups: surface a failed episode worker at once."""
        errs = getattr(self.manager, "errors", None)
        if errs:
            raise RuntimeError("an agent-loop worker failed:\n" + errs[0])
        if self.progress is not None:
            self.progress()
        else:
            time.sleep(0.01)

    # -- one step -----------------------------------------------------------------------------------------------------
    def _build(self, groups: list[PromptGroup]) -> tuple[list[PackedBatch], dict]:
        rows, rewards_all, lengths = [], [], []
        hidden = self.engine.model_cfg.hidden_size
        for g in groups:
            trs = [self.queue.get(k) for k in g.keys()]
            rewards = torch.tensor([float(t["reward"]) for t in trs])
            adv = grpo.group_advantages(rewards[None], self.cfg.norm_adv_by_std)[0]
            rewards_all += rewards.tolist()
            for t, a in zip(trs, adv.tolist()):
                rows.append(trajectory_to_rows(t, a, hidden, self.cfg.topk_heads, train_vision=self.engine.model.visual is not None))
                lengths.append(len(t["tokens"]))
        dp = self.engine.dp_size
        parts = [[pack_rows(mb) for mb in micro_batches([rows[i] for i in mine], self.cfg.max_token_len_per_gpu)]
                 for mine in balanced_partition(lengths, dp)]  # one list of packed micro-batches per data-parallel rank
        total_loss_tokens = int(sum(float(r["loss_mask"].sum()) for r in rows))
        stats = {"data/reward_mean": float(np.mean(rewards_all)), "data/sessions": float(len(rows)), "data/tokens": float(sum(lengths)),
                 "data/response_tokens": float(total_loss_tokens), "data/max_len": float(max(lengths)),
                 # whole-context lengths of the trained sessions (prompt + every turn): upstream verl patch 0012
                 "ctx_total_length/mean": float(np.mean(lengths)), "ctx_total_length/max": float(max(lengths))}
        return parts, dict(stats, _total_loss_tokens=total_loss_tokens)

    def train_step(self) -> dict:
        t0 = time.time()
        cap = None if self.cfg.trainer_mode == "sync" else self.replay.max_inflight_sessions
        groups, chunks = [], None
        if self.is_driver:
            groups = self.replay.sample(self.engine.policy_version, self.cfg.train_batch_size, refill=self._refill,
                                        timeout_s=self.cfg.sample_timeout_s, progress=self._while_waiting)
            # the batch is trained in mini-batches of `ppo_mini_batch_size` prompt groups, one optimizer step each (upstream's
            # update loop); advantages are per group, so a group never straddles two updates
            mini = self.cfg.ppo_mini_batch_size if 0 < self.cfg.ppo_mini_batch_size < len(groups) else len(groups)
            chunks = [self._build(groups[i:i + mini]) for i in range(0, len(groups), mini)]
        t_gen = time.time() - t0
        if self.engine.world > 1:
            import torch.distributed as dist

            box = [chunks]
            dist.broadcast_object_list(box, src=dist.get_global_rank(self.engine.group, 0), group=self.engine.group)
            chunks = box[0]
        t1 = time.time()
        version = self.engine.policy_version
        metrics, stats = {}, {}
        for ci, (parts, cstats) in enumerate(chunks):
            mbs = parts[self.engine.dp_rank]
            total = cstats.pop("_total_loss_tokens")
            with nvtx.annotate("trainer/forward_backward"):
                m = self.engine.forward_backward_batch(mbs, total_loss_tokens=total) if mbs else {}
            with nvtx.annotate("trainer/optimizer_step"):
                m.update(self.engine.optimizer_step())
            w = cstats["data/sessions"]
            for k, v in m.items():  # update metrics: session-weighted means over the mini-batches
                metrics[k] = metrics.get(k, 0.0) + float(v) * w
            for k, v in cstats.items():
                if k in ("data/sessions", "data/tokens", "data/response_tokens"):
                    stats[k] = stats.get(k, 0.0) + v
                elif k.endswith("/max") or k == "data/max_len":
                    stats[k] = max(stats.get(k, 0.0), v)
                else:
                    stats[k] = stats.get(k, 0.0) + v * w
        n_sessions = max(1.0, stats.get("data/sessions", 1.0))
        metrics = {k: v / n_sessions for k, v in metrics.items()}
        stats = {k: (v if k in ("data/sessions", "data/tokens", "data/response_tokens", "data/max_len") or k.endswith("/max") else v / n_sessions) for k, v in stats.items()}
        metrics["actor/updates"] = float(len(chunks))
        # one policy version per trained batch, however many updates it took (none when every update was skipped)
        self.engine.policy_version = version + (1 if self.engine.policy_version > version else 0)
        t_train = time.time() - t1
        stale = [self.engine.policy_version - 1 - g.issued_version for g in groups]
        if self.is_driver:
            self.replay.release(groups)
        self.step += 1
        if self.step % self.cfg.parameter_sync_step == 0 and (self.weight_sync is not None or self.engine.world > 1):
            state = self.engine.full_state_dict(torch.float32)  # collective: every trainer rank takes part
            if self.weight_sync is not None:
                with nvtx.annotate("trainer/weight_sync"):
                    metrics.update(self.weight_sync.sync(state, self.engine.policy_version))
            del state
        metrics.update(stats)
        metrics.update(self.replay.metrics)
        # model FLOPs utilisation of the trainer ranks against the device table (upstream verl patch 0016 adds its GPU there)
        tokens = stats.get("data/tokens", 0.0)
        if t_train > 0 and tokens:
            ctx = stats["ctx_total_length/mean"] / 2.0
            flops = 3.0 * self.engine.model_cfg.flops_per_token(context=int(ctx)) * tokens
            metrics["perf/mfu"] = flops / t_train / (device_peak_flops() * max(1, self.engine.world))
            metrics["perf/tokens_per_s"] = tokens / t_train
        for name, secs in (("wait_rollout", t_gen), ("train", t_train)):
            _log.info("phase %s %.3fs (step %d)", name, secs, self.step)  # one line per timed phase (upstream verl patch 0013)
        metrics.update({"timing/wait_rollout_s": t_gen, "timing/train_s": t_train, "timing/step_s": time.time() - t0,
                        "train/staleness_mean": float(np.mean(stale)) if stale else 0.0, "train/policy_version": float(self.engine.policy_version),
                        "train/inflight_sessions": float(self.replay.inflight_sessions()), "train/session_cap": float(cap or 0)})
        return metrics

    # -- the run ------------------------------------------------------------------------------------------------------
    def resume(self) -> Optional[dict]:
        if self.checkpoints is None:
            return None
        report = self.checkpoints.load(self.engine, self.dataset, self.replay, self.queue)
        if report is not None:
            self.step = report["step"]
            if self.weight_sync is not None or self.engine.world > 1:  # replicas start from the restored policy, not from the base model
                state = self.engine.full_state_dict(torch.float32)
                if self.weight_sync is not None:
                    self.weight_sync.sync(state, self.engine.policy_version)
        return report

    def fit(self) -> list[dict]:
        self.resume()
        try:
            while self.step < self.cfg.total_training_steps:
                m = self.train_step()
                if self.checkpoints is not None and self.cfg.save_freq > 0 and self.step % self.cfg.save_freq == 0:
                    t0 = time.time()
                    self.checkpoints.save(self.step, self.engine, self.dataset, self.replay, self.queue)
                    m["timing/checkpoint_s"] = time.time() - t0
                self.history.append(m)
                if self.is_driver:
                    self.log(self.step, m)
        finally:
            self.cancel_background()
        return self.history

    def cancel_background(self) -> None:
        """Run end: groups still generating are cancelled so no worker outlives the run."""
        if self.manager is None:
            return
        for g in list(self.replay.groups.values()):
            if g.status in (GroupStatus.IN_FLIGHT, GroupStatus.QUEUED):
                self.manager.cancel_group(g.uid)

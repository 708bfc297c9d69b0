"""Checkpoint / resume of a training run.

Layout and rules of the upstream run directory (``RUN/ckpt/global_step_<k>/actor/...``, ``run_stage1.sh:99``):

* one model+optimizer shard file per rank, ``model_world_size_<N>_rank_<r>.pt`` (a checkpoint of another world size is
  refused with both sizes named);
* ``extra_state.pt`` (step, policy version, RNG), ``data.pt`` (dataset cursor + replay-buffer groups), a transfer-queue
  snapshot (one file per storage unit) so that in-flight prompt groups survive a restart;
* ``latest_checkpointed_iteration.txt`` is written LAST and atomically: a crash mid-save leaves the previous
  checkpoint current;
* ``max_ckpt_to_keep``: older steps are pruned BEFORE the new snapshot is written (a disk sized for two checkpoints
  never holds three), and retention also counts checkpoints written before a resume;
* resumed LR = the configured LR at the restored schedule position (the engine applies it).

Export: ``export_model`` gathers the full state and writes a Hugging Face safetensors directory.
"""

from __future__ import annotations

import os
import re
import shutil
from typing import Optional

import torch

from ..models import io as model_io
from ..utils.files import atomic_write

LATEST = "latest_checkpointed_iteration.txt"


class CheckpointManager:
    def __init__(self, run_dir: str, rank: int = 0, world_size: int = 1, max_ckpt_to_keep: Optional[int] = None,
                 barrier=None):
        self.root = os.path.join(run_dir, "ckpt")
        self.rank, self.world, self.keep = rank, world_size, max_ckpt_to_keep
        self.barrier = barrier or (lambda: None)

    # -- paths --------------------------------------------------------------------------------------------------------
    def step_dir(self, step: int) -> str:
        return os.path.join(self.root, f"global_step_{step}")

    def steps_on_disk(self) -> list[int]:
        if not os.path.isdir(self.root):
            return []
        out = []
        for d in os.listdir(self.root):
            m = re.fullmatch(r"global_step_(\d+)", d)
            if m:
                out.append(int(m.group(1)))
        return sorted(out)

    def latest(self) -> Optional[int]:
        p = os.path.join(self.root, LATEST)
        if not os.path.exists(p):
            return None
        with open(p) as f:
            step = int(f.read().strip())
        return step if os.path.isdir(self.step_dir(step)) else None

    # -- save ---------------------------------------------------------------------------------------------------------
    def _prune(self, new_step: int) -> list[int]:
        if self.keep is None or self.rank != 0:
            return []
        old = [s for s in self.steps_on_disk() if s != new_step]
        victims = old[: max(0, len(old) - (self.keep - 1))]
        for s in victims:
            shutil.rmtree(self.step_dir(s), ignore_errors=True)
        return victims

    def save(self, step: int, engine, dataset=None, replay=None, queue=None, extra: Optional[dict] = None) -> str:
        self._prune(step)
        self.barrier()
        d = self.step_dir(step)
        actor = os.path.join(d, "actor")
        os.makedirs(actor, exist_ok=True)
        st = engine.train_state()
        # HSDP: the first replica (the ranks below the shard group size) writes; the other replicas hold copies of its shards
        # (upstream: 3rdparty/verl/patches/0021)
        if self.rank < int(getattr(engine, "shard_world", self.world)):
            torch.save(st, os.path.join(actor, f"model_world_size_{self.world}_rank_{self.rank}.pt"))
        if self.rank == 0:
            torch.save({"step": step, "policy_version": st["policy_version"], "world_size": self.world,
                        "rng": torch.get_rng_state(), **(extra or {})}, os.path.join(actor, "extra_state.pt"))
            torch.save({"dataset": dataset.state() if dataset is not None else None,
                        "replay": replay.state() if replay is not None else None}, os.path.join(d, "data.pt"))
            if queue is not None:
                queue.snapshot(os.path.join(d, "transfer_queue"))
        self.barrier()
        if self.rank == 0:
            atomic_write(os.path.join(self.root, LATEST), str(step))
        self.barrier()
        return d

    # -- load ---------------------------------------------------------------------------------------------------------
    def load(self, engine, dataset=None, replay=None, queue=None, step: Optional[int] = None) -> Optional[dict]:
        step = self.latest() if step is None else step
        if step is None:
            return None
        d = self.step_dir(step)
        actor = os.path.join(d, "actor")
        mine = os.path.join(actor, f"model_world_size_{self.world}_rank_{self.rank % int(getattr(engine, 'shard_world', self.world))}.pt")
        if not os.path.exists(mine):
            sizes = sorted({int(m.group(1)) for f in os.listdir(actor) if (m := re.match(r"model_world_size_(\d+)_rank_", f))})
            raise ValueError(f"checkpoint {d} was written by world size {sizes}, this run has world size {self.world}")
        engine.load_train_state(torch.load(mine, map_location="cpu", weights_only=False))
        extra = torch.load(os.path.join(actor, "extra_state.pt"), map_location="cpu", weights_only=False)
        data = torch.load(os.path.join(d, "data.pt"), map_location="cpu", weights_only=False)
        report = {"step": step, "extra": extra, "dropped_keys": 0, "replay": None}
        if queue is not None and os.path.isdir(os.path.join(d, "transfer_queue")):
            report["dropped_keys"] = queue.restore(os.path.join(d, "transfer_queue"))
        if dataset is not None:
            dataset.restore(data.get("dataset"))
        if replay is not None and data.get("replay") is not None:
            report["replay"] = replay.restore(data["replay"], extra["policy_version"])
        return report


def export_model(engine, directory: str, fp32_modules=(), drop_mtp: bool = True, rank: int = 0) -> None:
    """Full (unsharded) model as a safetensors directory; every rank takes part in the gather, rank 0 writes."""
    state = engine.full_state_dict(torch.float32)
    if rank == 0:
        model_io.save_model_dir(directory, engine.model_cfg, state, fp32_modules=fp32_modules, drop_mtp=drop_mtp)

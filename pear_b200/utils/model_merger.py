"""``python -m pear_b200.utils.model_merger <run_dir> <out_dir> [--step K] [--fp32-module NAME ...]``: merge the per-rank
shards of a training checkpoint into a Hugging Face safetensors model directory (upstream ``pear/utils/model_merger.py:
11-38`` around verl's FSDP merger; ``scripts/export_checkpoint.sh``). fp32 for the named modules, bf16 for the rest;
the MTP head is left out (the drafter always comes from the base model)."""

from __future__ import annotations

import argparse
import os
import re

import torch

from ..models import io as model_io
from ..models.config import HybridConfig


def merge_shards(actor_dir: str) -> dict[str, torch.Tensor]:
    files = sorted(f for f in os.listdir(actor_dir) if re.fullmatch(r"model_world_size_\d+_rank_\d+\.pt", f))
    if not files:
        raise FileNotFoundError(f"no shard files in {actor_dir}")
    world = int(re.match(r"model_world_size_(\d+)_", files[0]).group(1))
    first = torch.load(os.path.join(actor_dir, f"model_world_size_{world}_rank_0.pt"), map_location="cpu", weights_only=False)
    # HSDP: only the first replica (ranks [0, S)) writes shard files, the other replicas hold copies
    sharded_over = int(first.get("shard_world_size", world))
    if len(files) != sharded_over:
        raise ValueError(f"{actor_dir}: {len(files)} shard files for world size {world} sharded over {sharded_over} ranks")
    shards = [first["shards"]] + [torch.load(os.path.join(actor_dir, f"model_world_size_{world}_rank_{r}.pt"), map_location="cpu", weights_only=False)["shards"]
                                  for r in range(1, sharded_over)]
    out: dict[str, torch.Tensor] = {}
    for unit, meta in shards[0]["__layout__"].items():
        flat = torch.cat([s[unit] for s in shards])
        for name, (offset, shape) in meta.items():
            n = 1
            for d in shape:
                n *= d
            out[name] = flat[offset:offset + n].reshape(shape).clone()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("run_dir")
    ap.add_argument("out_dir")
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--config", default=None, help="model config.json (default: <run_dir>/model_config.json)")
    ap.add_argument("--fp32-module", action="append", default=[])
    a = ap.parse_args(argv)
    root = os.path.join(a.run_dir, "ckpt")
    step = a.step
    if step is None:
        with open(os.path.join(root, "latest_checkpointed_iteration.txt")) as f:
            step = int(f.read().strip())
    state = merge_shards(os.path.join(root, f"global_step_{step}", "actor"))
    cfg = HybridConfig.load(a.config or os.path.join(a.run_dir, "model_config.json"))
    model_io.save_model_dir(a.out_dir, cfg, state, fp32_modules=a.fp32_module)
    print(f"wrote {len(state)} tensors of step {step} to {a.out_dir}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

"""Tensor parallelism for the rollout replicas (upstream runs its Blackwell rollout backend at TP2 and the Hopper one
at TP4: ``rollout/blackwell/model.py:45-346``, ``rollout/hopper/*``).

Megatron-style sharding of the hybrid model: attention heads, GDN heads and the FFN width are split over the ranks;
q/k/v, the GDN input projections and gate/up are column-parallel (no communication), o_proj / out_proj / down_proj are
row-parallel and their partial sums are all-reduced (``models.hybrid.row_linear``; on B200s the fused
all-reduce + residual add + RMSNorm kernel of ``parallel/symm.py`` replaces the NCCL call). Norms, embedding and
lm_head stay replicated. Every rank runs the same scheduler on the same requests, so the ranks stay in lockstep
without a control channel.

``tp_config`` gives the per-rank model shape, ``shard_state`` cuts a full state dict for one rank.
"""

from __future__ import annotations

import dataclasses

import torch

from ..models.config import HybridConfig


def kv_heads_per_rank(cfg: HybridConfig, world: int) -> tuple[int, int]:
    """(KV heads a rank holds, ranks that share one KV head). With more ranks than KV heads every group of
    ``world / num_kv_heads`` ranks holds a copy of the same head (the 27B shape has 4 KV heads: at 8 ranks each rank holds
    one head and 3 of its 6 query heads)."""
    kv = cfg.num_kv_heads
    if kv % world == 0:
        return kv // world, 1
    group = cfg.num_attention_heads // kv
    if world % kv == 0 and group % (world // kv) == 0:
        return 1, world // kv
    raise ValueError(f"num_kv_heads={kv} can be neither split nor replicated over the tensor-parallel size {world}")


def tp_config(cfg: HybridConfig, world: int) -> HybridConfig:
    for name, v in (("num_attention_heads", cfg.num_attention_heads), ("gdn_qk_heads", cfg.gdn_qk_heads),
                    ("gdn_v_heads", cfg.gdn_v_heads), ("intermediate_size", cfg.intermediate_size)):
        if v % world:
            raise ValueError(f"{name}={v} is not divisible by the tensor-parallel size {world}")
    kv_local, _ = kv_heads_per_rank(cfg, world)
    return dataclasses.replace(cfg, num_attention_heads=cfg.num_attention_heads // world, num_kv_heads=kv_local,
                               gdn_qk_heads=cfg.gdn_qk_heads // world, gdn_v_heads=cfg.gdn_v_heads // world,
                               intermediate_size=cfg.intermediate_size // world)


def _rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def _cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n]


def _sections(t: torch.Tensor, sizes: list[int], rank: int, world: int) -> torch.Tensor:
    """Row-shard a tensor whose rows are consecutive sections (q | k | v): each section is cut separately."""
    out, o = [], 0
    for s in sizes:
        out.append(_rows(t[o:o + s], rank, world))
        o += s
    return torch.cat(out, dim=0)


def shard_state(state: dict[str, torch.Tensor], cfg: HybridConfig, rank: int, world: int) -> dict[str, torch.Tensor]:
    kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
    _, kv_share = kv_heads_per_rank(cfg, world)
    out: dict[str, torch.Tensor] = {}
    for name, t in state.items():
        leaf = name.rsplit(".", 2)[-2] if name.endswith(".weight") else name.rsplit(".", 1)[-1]
        if leaf in ("k_proj", "v_proj") and kv_share > 1:
            head = rank // kv_share              # replicated KV head: every rank of the group takes the same rows
            t = t[head * cfg.head_dim:(head + 1) * cfg.head_dim]
        elif leaf in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "in_proj_z", "in_proj_b", "in_proj_a"):
            t = _rows(t, rank, world)          # q_proj rows are per head [q | gate]: head-major, so a plain row cut
        elif leaf in ("o_proj", "out_proj", "down_proj"):
            t = _cols(t, rank, world)
        elif leaf in ("in_proj_qkv", "conv1d"):
            t = _sections(t, [kd, kd, vd], rank, world)
        elif leaf in ("A_log", "dt_bias"):
            t = _rows(t, rank, world)
        out[name] = t.contiguous()
    return out

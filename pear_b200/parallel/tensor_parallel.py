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


def shard_pieces(name: str, shape: tuple, cfg: HybridConfig, rank: int, world: int) -> list[tuple[int, int, int, int]]:
    """Which blocks of a full tensor one tensor-parallel rank holds, in the order they are stacked along dim 0 of its shard:
    ``(row0, rows, col0, cols)`` of the tensor seen as a matrix ``[shape[0], prod(shape[1:])]``. Replicated tensors are one
    block. The weight-sync receiver pulls exactly these blocks; ``shard_state`` cuts them out of a full state dict."""
    rows = int(shape[0]) if len(shape) else 1
    cols = 1
    for d in shape[1:]:
        cols *= int(d)
    if world == 1:
        return [(0, rows, 0, cols)]
    kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
    _, kv_share = kv_heads_per_rank(cfg, world)
    leaf = name.rsplit(".", 2)[-2] if name.endswith(".weight") else name.rsplit(".", 1)[-1]
    if leaf in ("k_proj", "v_proj") and kv_share > 1:
        head = rank // kv_share              # replicated KV head: every rank of the group takes the same rows
        return [(head * cfg.head_dim, cfg.head_dim, 0, cols)]
    if leaf in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "in_proj_z", "in_proj_b", "in_proj_a", "A_log", "dt_bias"):
        n = rows // world                    # q_proj rows are per head [q | gate]: head-major, so a plain row cut
        return [(rank * n, n, 0, cols)]
    if leaf in ("o_proj", "out_proj", "down_proj"):
        n = cols // world
        return [(0, rows, rank * n, n)]
    if leaf in ("in_proj_qkv", "conv1d"):    # rows are consecutive sections (q | k | v): each section is cut separately
        out, o = [], 0
        for sec in (kd, kd, vd):
            n = sec // world
            out.append((o + rank * n, n, 0, cols))
            o += sec
        return out
    return [(0, rows, 0, cols)]


def shard_state(state: dict[str, torch.Tensor], cfg: HybridConfig, rank: int, world: int) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for name, t in state.items():
        pieces = shard_pieces(name, tuple(t.shape), cfg, rank, world)
        m = t.reshape(t.shape[0], -1) if t.dim() >= 1 else t.reshape(1, 1)
        cut = torch.cat([m[r0:r0 + r, c0:c0 + c] for r0, r, c0, c in pieces], dim=0) if len(pieces) > 1 else \
            m[pieces[0][0]:pieces[0][0] + pieces[0][1], pieces[0][2]:pieces[0][2] + pieces[0][3]]
        out[name] = cut.reshape(shard_shape(tuple(t.shape), pieces)).contiguous()
    return out


def shard_shape(shape: tuple, pieces: list[tuple[int, int, int, int]]) -> tuple:
    """Shape of the shard that ``pieces`` of a tensor of ``shape`` stack up to."""
    if not shape:
        return ()
    rows = sum(p[1] for p in pieces)
    if len(shape) == 1:
        return (rows,)
    full_cols = 1
    for d in shape[1:]:
        full_cols *= int(d)
    if pieces[0][3] == full_cols:
        return (rows, *shape[1:])
    assert len(shape) == 2, "a column cut of a tensor with more than two dimensions"
    return (rows, pieces[0][3])

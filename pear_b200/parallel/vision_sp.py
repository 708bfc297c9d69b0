"""Vision tower sharded over the sequence-parallel ranks (upstream ``verl patch 0025``): every rank encodes a share of a
micro-batch's images, the features are all-gathered so that each rank holds all image rows, and the tower's gradients
are summed over the group in fp32. Shares are dealt by patch count (longest first) so the ranks do similar work."""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def deal_images(sizes: list[int], world: int) -> list[list[int]]:
    bins: list[list[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(len(sizes)), key=lambda j: -sizes[j]):
        b = min(range(world), key=lambda j: load[j])
        bins[b].append(i)
        load[b] += sizes[i]
    return [sorted(b) for b in bins]


class _AllGatherRows(torch.autograd.Function):
    """Concatenate per-rank row blocks of different lengths; backward returns this rank's slice of the gradient summed
    over the ranks (every rank consumes every image's rows)."""

    @staticmethod
    def forward(ctx, local: torch.Tensor, counts: list[int], group):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        width = local.shape[1]
        pad = max(counts)
        buf = local.new_zeros(pad, width)
        buf[: local.shape[0]] = local
        out = [torch.empty_like(buf) for _ in range(world)]
        dist.all_gather(out, buf.contiguous(), group=group)
        ctx.group, ctx.counts, ctx.rank = group, counts, rank
        return torch.cat([o[:c] for o, c in zip(out, counts)], dim=0)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        g = g.contiguous().float()
        dist.all_reduce(g, group=ctx.group)
        lo = sum(ctx.counts[: ctx.rank])
        return g[lo: lo + ctx.counts[ctx.rank]], None, None


def encode_sharded(tower, images: list[torch.Tensor], group=None) -> list[torch.Tensor]:
    """Feature rows of every image on every rank, each image encoded once (by the rank it was dealt to)."""
    if group is None or dist.get_world_size(group) == 1:
        return tower(images)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    tokens = [tower.tokens_per_image(im.shape[1], im.shape[2]) for im in images]
    shares = deal_images(tokens, world)
    mine = tower([images[i] for i in shares[rank]]) if shares[rank] else []
    width = tower.cfg.out_hidden
    local = torch.cat(mine, dim=0) if mine else torch.zeros(0, width, device=images[0].device)
    counts = [sum(tokens[i] for i in s) for s in shares]
    rows = _AllGatherRows.apply(local, counts, group)
    out: list[Optional[torch.Tensor]] = [None] * len(images)
    off = 0
    for s in shares:
        for i in s:
            out[i] = rows[off: off + tokens[i]]
            off += tokens[i]
    return out  # type: ignore[return-value]


def reduce_tower_grads(tower, group=None) -> None:
    """fp32 all-reduce of the tower's gradients (each rank back-propagated only through its own images)."""
    if group is None or dist.get_world_size(group) == 1:
        return
    for p in tower.parameters():
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        g = p.grad.float()
        dist.all_reduce(g, group=group)
        p.grad.copy_(g)

"""Process-group plumbing and autograd-aware collectives (NCCL on GPUs, gloo on CPU ranks).

These are the baseline transport of every parallel path; the fused compute+collective kernels of
:mod:`pear_b200.parallel.symm` replace them on the hot paths when peer memory is available. gloo lacks
``reduce_scatter_tensor`` and is slow at ``all_to_all``; both are expressed through what it has, so the same code runs in
the CPU multi-process tests.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


def init_process_group(backend: Optional[str] = None, init_method: Optional[str] = None, rank: Optional[int] = None,
                       world_size: Optional[int] = None, timeout_s: float = 600.0) -> None:
    """One process per GPU. Without arguments the ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` environment is used; a
    ``file://`` init method avoids ports and hostname resolution (tests)."""
    if dist.is_initialized():
        return
    import datetime

    backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    kw = dict(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
    if init_method is not None:
        kw.update(init_method=init_method, rank=rank, world_size=world_size)
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", rank or 0))
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(**kw)


def backend_of(group) -> str:
    return dist.get_backend(group)


def all_gather_cat(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
    """Concatenation of every rank's ``x`` (equal shapes) along ``dim``; not differentiable."""
    n = dist.get_world_size(group)
    if n == 1:
        return x
    xc = x.contiguous()
    flat = torch.empty(n * xc.numel(), dtype=xc.dtype, device=xc.device)
    dist.all_gather_into_tensor(flat, xc.reshape(-1), group=group)
    out = flat.view((n,) + tuple(xc.shape))
    if dim == 0:
        return out.reshape((n * xc.shape[0],) + tuple(xc.shape[1:]))
    return torch.cat(list(out.unbind(0)), dim=dim)


def reduce_scatter_sum(x: torch.Tensor, group) -> torch.Tensor:
    """Sum over ranks of ``x`` [n * m, ...], this rank keeping rows [rank * m, (rank + 1) * m)."""
    n = dist.get_world_size(group)
    if n == 1:
        return x
    xc = x.contiguous()
    m = xc.shape[0] // n
    if backend_of(group) == "gloo":
        dist.all_reduce(xc, group=group)
        r = dist.get_rank(group)
        return xc[r * m : (r + 1) * m].clone()
    out = torch.empty((m,) + tuple(xc.shape[1:]), dtype=xc.dtype, device=xc.device)
    dist.reduce_scatter_tensor(out, xc, group=group)
    return out


class _AllGather(torch.autograd.Function):
    """Stacked all-gather [n, ...]; backward sums the incoming gradients and keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        xc = x.contiguous()
        flat = torch.empty(n * xc.numel(), dtype=xc.dtype, device=xc.device)
        dist.all_gather_into_tensor(flat, xc.reshape(-1), group=group)
        return flat.view((n,) + tuple(xc.shape))

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_sum(g.contiguous(), ctx.group).squeeze(0), None


def all_gather_stack(x: torch.Tensor, group) -> torch.Tensor:
    if dist.get_world_size(group) == 1:
        return x.unsqueeze(0)
    return _AllGather.apply(x, group)


_STARTED: list = []  # the work handle of the collective `_AllGatherStart.forward` just launched (taken by its caller at once)


class _AllGatherStart(torch.autograd.Function):
    """``_AllGather`` whose forward only launches the collective: the caller waits on the handle before it reads the result,
    and whatever it computes in between overlaps the transfer (NCCL runs it on its own stream)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        xc = x.contiguous()
        out = torch.empty((n,) + tuple(xc.shape), dtype=xc.dtype, device=xc.device)  # (returned as it is: the collective fills it later)
        _STARTED.append((dist.all_gather_into_tensor(out.view(-1), xc.reshape(-1), group=group, async_op=True), xc))  # xc stays alive until the wait
        return out

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_sum(g.contiguous(), ctx.group).squeeze(0), None


def all_gather_stack_start(x: torch.Tensor, group):
    """Start a stacked all-gather; returns (result, wait). ``result`` may be read only after ``wait()``."""
    if dist.get_world_size(group) == 1:
        return x.unsqueeze(0), (lambda: None)
    out = _AllGatherStart.apply(x, group)
    work, keep = _STARTED.pop()

    def wait() -> None:
        work.wait()
        keep.clear()

    keep = [keep]
    return out, wait


class _AllToAll(torch.autograd.Function):
    """x [n, chunk...] -> y [n, chunk...] with y[j] = rank j's x[rank]; its own transpose in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_to_all_equal(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all_equal(g, ctx.group), None


def _all_to_all_equal(x: torch.Tensor, group) -> torch.Tensor:
    xc = x.contiguous()
    out = torch.empty_like(xc)
    if backend_of(group) == "gloo":
        # gloo: pairwise exchange expressed as an all-gather (small CPU test sizes only)
        n, r = dist.get_world_size(group), dist.get_rank(group)
        flat = torch.empty(n * xc.numel(), dtype=xc.dtype)
        dist.all_gather_into_tensor(flat, xc.reshape(-1), group=group)
        return flat.view((n,) + tuple(xc.shape))[:, r].contiguous()
    dist.all_to_all_single(out, xc, group=group)
    return out


def all_to_all(x: torch.Tensor, group) -> torch.Tensor:
    """Differentiable equal-split all-to-all over the leading dimension (size = group size)."""
    if dist.get_world_size(group) == 1:
        return x
    return _AllToAll.apply(x, group)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        y = g.clone()
        dist.all_reduce(y, group=ctx.group)
        return y, None


def all_reduce_sum(x: torch.Tensor, group) -> torch.Tensor:
    if dist.get_world_size(group) == 1:
        return x
    return _AllReduceSum.apply(x, group)

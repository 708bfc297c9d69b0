"""Spawn helper for multi-process CPU tests: gloo ranks with a file:// rendezvous (no ports, no hostname lookups)."""

from __future__ import annotations

import os
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, path, fn, args, errors):
    try:
        os.environ["OMP_NUM_THREADS"] = "1"
        torch.set_num_threads(1)
        dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        errors.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, tmp_path, *args, timeout: float = 240.0):
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    path = os.path.join(str(tmp_path), "rdzv")
    procs = [ctx.Process(target=_entry, args=(r, world, path, fn, args, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    while not errors.empty():
        failed.append(errors.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            failed.append((-1, "rank timed out"))
    assert not failed, "\n".join(f"rank {r}: {tb}" for r, tb in failed)
    assert all(p.exitcode == 0 for p in procs)

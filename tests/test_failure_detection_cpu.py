"""Failure detection on the host with gloo ranks on CPU: a rank that leaves between steps is seen through the heartbeat
store before the next step; a rank that silently stops answering ends the survivor's collective with an error after a
short process-group timeout. No GPU is involved and nothing is made to hang."""

import datetime
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pear_b200.parallel.heartbeat import Heartbeat, PeerLost


def _leave_worker(rank, world, path, results):
    store = dist.FileStore(path, world)
    hb = Heartbeat(store, rank, world, timeout_s=5.0)
    try:
        hb.beat(0)
        hb.wait_all(0)
        if rank == 1:
            hb.leave(0)  # between steps: nothing of this rank is in flight
            return
        time.sleep(0.5)
        hb.check(min_step=None)  # what a survivor does before launching its next step
        results.put((rank, "alive"))
    except PeerLost as e:  # wherever the survivor notices, it is on the host and before its next launch
        results.put((rank, f"lost {e.ranks}"))


def test_rank_that_leaves_between_steps_is_seen_before_the_next_launch():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_leave_worker, args=(r, 3, path, results)) for r in range(3)]
        for p in procs:
            p.start()
        got = sorted(results.get(timeout=60) for _ in range(2))
        for p in procs:
            p.join(30)
    assert got == [(0, "lost [1]"), (2, "lost [1]")]


def test_stale_heartbeat_and_never_joined():
    with tempfile.TemporaryDirectory() as d:
        store = dist.FileStore(os.path.join(d, "s"), 2)
        hb0 = Heartbeat(store, 0, 2, timeout_s=0.2)
        with pytest.raises(PeerLost, match="never joined"):
            hb0.check()
        hb1 = Heartbeat(store, 1, 2, timeout_s=0.2)
        hb1.beat(3)
        hb0.check(min_step=3)
        with pytest.raises(PeerLost, match="still before step 4"):
            hb0.check(min_step=4)
        time.sleep(0.3)
        with pytest.raises(PeerLost, match="no heartbeat"):
            hb0.check()


def _silent_worker(rank, world, path, results):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)  # step 0: everybody answers
    if rank == 1:
        os._exit(0)  # the rank disappears without a word
    t0 = time.time()
    try:
        dist.all_reduce(t)  # step 1: the survivor's collective ends with an error, it does not wait forever
        results.put("no error")
    except Exception as e:  # noqa: BLE001
        results.put(f"error after {time.time() - t0:.0f}s: {type(e).__name__}")
    results.close()
    results.join_thread()  # the message is on its way before the process goes (no process-group teardown with a dead peer)
    os._exit(0)


@pytest.mark.timeout(120)
def test_silent_rank_ends_the_survivors_collective_with_an_error():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "rdzv")
        procs = [ctx.Process(target=_silent_worker, args=(r, 2, path, results)) for r in range(2)]
        for p in procs:
            p.start()
        msg = results.get(timeout=90)
        for p in procs:
            p.join(30)
    assert msg.startswith("error after"), msg

"""A tensor-parallel rollout replica behind one HTTP endpoint: the ranks run their engines in lock-step.

Every rank of the replica owns a shard of the model and a full copy of the scheduler state (block tables, queues, sampler
seed). Only rank 0 (the leader) talks to clients. Once per scheduler iteration the leader broadcasts the control events it
collected since the last one (new requests, pause, resume); every rank applies them in the same order and then takes the
same ``engine.step()``, whose collectives (the row-parallel reductions, the logits gather) meet inside the model. Because the
scheduler is a deterministic function of the event sequence and of the sampled tokens (identical on every rank: same logits,
same seed), the ranks never need to exchange scheduling decisions. An idle leader sends a heartbeat so that a follower's
blocking receive stays far from the process group's timeout.

Weights arrive on every rank through its own weight-sync receiver (``server.start_weight_receiver``); a rank applies the
``resume`` event only after it has loaded as many syncs as the leader had when the trainer asked to resume.

Upstream gets this from vLLM's executor (one driver worker broadcasting ``execute_model`` inputs to the tensor-parallel
workers: pear/rollout/server.py:14-82, pear/rollout/worker_extension.py:13-70).
"""

from __future__ import annotations

import time
from concurrent.futures import Future
from typing import Optional

import torch
import torch.distributed as dist

from .engine import SamplingParams
from .server import RolloutServer


class LockstepChannel:
    """Leader -> followers broadcast of picklable messages over a host-side (gloo) group, so that control traffic never
    queues behind kernels on a GPU stream."""

    def __init__(self, group=None, leader: int = 0):
        self.group, self.leader = group, leader
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    @property
    def is_leader(self) -> bool:
        return self.rank == self.leader

    def exchange(self, msg=None):
        box = [msg if self.is_leader else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, self.leader) if self.group is not None else self.leader, group=self.group)
        return box[0]

    def barrier(self) -> None:
        dist.barrier(group=self.group)


class LockstepServer(RolloutServer):
    """``RolloutServer`` whose engine calls all happen on the scheduling thread, in an order the leader fixes for every rank.
    The client API (``submit``, ``generate``, ``pause``, ``resume``) exists on the leader only."""

    def __init__(self, engine, channel: LockstepChannel, shard_fn=None, heartbeat_s: float = 2.0, load_wait_s: float = 600.0, **kw):
        self.channel, self.shard_fn = channel, shard_fn
        self.heartbeat_s, self.load_wait_s = heartbeat_s, load_wait_s
        self.events: list[tuple] = []
        self.tickets: dict[int, Future] = {}
        self._ticket = 0
        super().__init__(engine, **kw)

    # -- leader-side client API ---------------------------------------------------------------------------------------
    def _enqueue(self, kind: str, *payload) -> Future:
        if not self.channel.is_leader:
            raise RuntimeError(f"{self.name}: only rank {self.channel.leader} of a tensor-parallel replica takes requests")
        if self.error is not None:
            raise RuntimeError(f"{self.name}: scheduler stopped") from self.error
        fut: Future = Future()
        with self.lock:
            self._ticket += 1
            self.tickets[self._ticket] = fut
            self.events.append((kind, self._ticket) + payload)
        return fut

    def submit(self, prompt: list[int], params: Optional[SamplingParams] = None, session: Optional[str] = None,
               embeds=None, embeds_mask=None, position_ids=None) -> Future:
        cpu = lambda t: t.detach().cpu() if torch.is_tensor(t) else t  # noqa: E731 - events travel pickled
        return self._enqueue("add", list(prompt), params, session, cpu(embeds), cpu(embeds_mask), cpu(position_ids))

    def pause(self, abort: bool = True) -> int:
        return int(self._enqueue("pause", bool(abort)).result(timeout=self.load_wait_s))

    def resume(self) -> None:
        self._enqueue("resume", self.weight_loads).result(timeout=self.load_wait_s + 60)

    def update_weights(self, state: dict[str, torch.Tensor], version: int) -> None:
        """Called by this rank's weight-sync receiver while the replica is paused: full tensors are cut to this rank's shard."""
        super().update_weights(self.shard_fn(state) if self.shard_fn is not None else state, version)

    # -- scheduling thread (every rank) -------------------------------------------------------------------------------
    def _apply(self, ev: tuple):
        kind, ticket = ev[0], ev[1]
        fut = self.tickets.pop(ticket, None) if self.channel.is_leader else None
        if kind == "add":
            _, _, prompt, params, session, embeds, mask, position_ids = ev
            dev = self.engine.device
            req = self.engine.add_request(prompt, params, session, embeds=embeds.to(dev) if torch.is_tensor(embeds) else embeds,
                                          embeds_mask=mask.to(dev) if torch.is_tensor(mask) else mask, position_ids=position_ids)
            if fut is not None:
                if req.finish is not None:  # rejected by a paused engine
                    fut.set_result(req)
                else:
                    self.futures[req.request_id] = fut
            return None
        if kind == "pause":
            aborted = self.engine.pause(abort=ev[2])
            self._resolve(aborted)
            return (fut, len(aborted))
        if kind == "resume":
            t0 = time.time()
            while self.weight_loads < ev[2]:  # this rank's receiver has not loaded the sync the leader resumes from
                if time.time() - t0 > self.load_wait_s:
                    raise TimeoutError(f"{self.name} rank {self.channel.rank}: weights of sync {ev[2]} never arrived")
                time.sleep(0.001)
            return (fut, None)
        raise ValueError(f"unknown control event {kind!r}")

    def _loop(self) -> None:
        dev = next(self.engine.model.parameters()).device
        if dev.type == "cuda":
            torch.cuda.set_device(dev)  # a new host thread starts on device 0
        ch, last_msg = self.channel, time.time()
        try:
            while True:
                msg = None
                if ch.is_leader:
                    with self.lock:
                        events, self.events = self.events, []
                    stop = self.stop_flag
                    busy = self.engine.has_work() and not self.engine.paused
                    if not (events or stop or busy) and time.time() - last_msg < self.heartbeat_s:
                        time.sleep(self.idle_sleep_s)
                        continue
                    msg, last_msg = {"events": events, "stop": stop}, time.time()
                msg = ch.exchange(msg)
                control = []
                for ev in msg["events"]:  # in the leader's order
                    if ev[0] == "resume":  # waits for this rank's receiver, which needs the lock to load
                        control.append(self._apply(ev))
                        with self.lock:
                            self.engine.resume()
                        continue
                    with self.lock:
                        res = self._apply(ev)
                    if res is not None:
                        control.append(res)
                if control:  # the leader answers a pause / resume only once every rank has applied it
                    ch.barrier()
                    for fut, value in control:
                        if fut is not None:
                            fut.set_result(value)
                if msg["stop"]:
                    return
                with self.lock:
                    if self.engine.has_work() and not self.engine.paused:
                        self._resolve(self.engine.step())
        except BaseException as e:  # noqa: BLE001 - surfaced to every waiter
            self.error = e
            with self.lock:
                for f in list(self.futures.values()) + list(self.tickets.values()):
                    if not f.done():
                        f.set_exception(e)
                self.futures.clear()
                self.tickets.clear()

    def close(self) -> None:
        """Leader: tell the followers to stop, then join. Followers: join (their loop ends with the leader's stop message)."""
        self.stop_flag = True
        self.thread.join(timeout=30)


def build_tp_replica(path: str, cfg, name: str = "replica-0", fp32_modules=(), with_mtp: bool = True) -> LockstepServer:
    """One rank of a tensor-parallel replica; ``torch.distributed`` is initialised with the replica's ranks as its world
    (``torch.distributed.run --nproc-per-node <tp>``). Builds the full model on the host, keeps this rank's shard, routes the
    row-parallel reductions through the world (on GPUs: through the NVSwitch kernels of a ``SymmWorld`` as well) and opens a
    host-side control group for the lock-step channel."""
    import os

    from ..models import hybrid
    from ..models.hybrid import HybridForCausalLM
    from ..parallel.tensor_parallel import shard_state, tp_config
    from .engine import RolloutEngine
    from .server import load_rollout_model, to_rollout_dtypes

    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    device = f"cuda:{int(os.environ.get('LOCAL_RANK', rank))}" if cuda else "cpu"
    full = load_rollout_model(path, device="cpu", with_mtp=with_mtp)
    mcfg = full.config
    model = HybridForCausalLM(tp_config(mcfg, world), with_mtp=full.mtp is not None)
    model.load_state_dict(shard_state(full.state_dict(), mcfg, rank, world), strict=True)
    del full
    if cuda:
        torch.cuda.set_device(device)
        to_rollout_dtypes(model.to(device))
    hybrid.set_tensor_parallel_group(dist.group.WORLD)
    engine = RolloutEngine(model.eval(), cfg, device)
    if cuda:
        from ..parallel.symm import SymmWorld

        symm = SymmWorld()
        hybrid.set_tensor_parallel_fused(symm, 256, mcfg.hidden_size)
        engine.set_symm_world(symm)
    control = dist.new_group(backend="gloo")  # host-side: control messages never wait behind kernels
    return LockstepServer(engine, LockstepChannel(control), shard_fn=lambda s: shard_state(s, mcfg, rank, world), name=name,
                          fp32_modules=tuple(fp32_modules))

"""Trainer -> rollout weight synchronisation.

Every training step ends with the rollout replicas loading the new policy (upstream ``pear/rollout/checkpoint_engine.py:
15-43`` on verl's NCCL checkpoint engine; recipe keys ``checkpoint_engine.*`` in ``configs/base.yaml:89-99``):

1. replicas pause and abort in-flight requests (they are resubmitted afterwards and continue from the prefix cache of
   the NEW policy, i.e. from nothing: every KV tier is cleared after the sync);
2. cached allocator memory is released before the transfer buffers are prepared;
3. the full state is streamed in buckets of ``bucket_megabytes``: every float tensor is cast to the rollout dtype
   except the modules that must stay fp32;
4. replicas load in place, bump their policy version, clear their KV tiers and resume.

Transports:
* ``InProcessTransport``: trainer and replicas in one process (tests, the single-node synchronous recipe);
* ``BroadcastTransport``: a ``torch.distributed`` group of {trainer rank 0} + {replica ranks}; bucket payloads are
  flattened into one buffer per bucket and broadcast (NCCL on GPUs, gloo on CPU); the group may be rebuilt every sync.
The NVSwitch transport (P2P reads of the trainer's staging buffer fused with bf16 -> NVFP4 requantisation on the
receiver) lives in ``pear_b200/parallel/symm.py`` and plugs in through the same interface.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Iterable, Iterator, Optional

import torch
import torch.distributed as dist


@dataclass
class SyncConfig:
    bucket_megabytes: int = 512
    rollout_dtype: torch.dtype = torch.bfloat16
    fp32_modules: tuple = ()
    rebuild_group: bool = True


def cast_for_rollout(name: str, t: torch.Tensor, cfg: SyncConfig) -> torch.Tensor:
    if not t.is_floating_point() or any(m in name for m in cfg.fp32_modules):
        return t
    return t.to(cfg.rollout_dtype)


def buckets(state: Iterable[tuple[str, torch.Tensor]], cfg: SyncConfig) -> Iterator[list[tuple[str, torch.Tensor]]]:
    limit = cfg.bucket_megabytes << 20
    cur, size = [], 0
    for name, t in state:
        t = cast_for_rollout(name, t, cfg)
        n = t.numel() * t.element_size()
        if cur and size + n > limit:
            yield cur
            cur, size = [], 0
        cur.append((name, t))
        size += n
    if cur:
        yield cur


class InProcessTransport:
    def __init__(self, servers: list):
        self.servers = servers

    def send(self, bucket: list[tuple[str, torch.Tensor]], version: int, last: bool) -> None:
        for s in self.servers:
            s._pending = getattr(s, "_pending", {})
            s._pending.update({k: v for k, v in bucket})
            if last:
                s.update_weights(s._pending, version)
                s._pending = {}


class BroadcastTransport:
    """Rank ``src`` of ``group`` owns the weights; every other rank calls ``receive`` with the same manifest."""

    def __init__(self, group=None, src: int = 0, device="cpu"):
        self.group, self.src, self.device = group, src, torch.device(device)

    def send(self, bucket: list[tuple[str, torch.Tensor]], version: int, last: bool) -> None:
        manifest = [(n, tuple(t.shape), t.dtype, t.numel() * t.element_size()) for n, t in bucket]
        obj = [{"manifest": manifest, "version": version, "last": last}]
        dist.broadcast_object_list(obj, src=self.src, group=self.group)
        flat = torch.cat([t.detach().contiguous().view(-1).view(torch.uint8).to(self.device) for _, t in bucket])
        dist.broadcast(flat, src=self.src, group=self.group)

    def receive(self) -> tuple[dict[str, torch.Tensor], int, bool]:
        obj = [None]
        dist.broadcast_object_list(obj, src=self.src, group=self.group)
        info = obj[0]
        total = sum(m[3] for m in info["manifest"])
        flat = torch.empty(total, dtype=torch.uint8, device=self.device)
        dist.broadcast(flat, src=self.src, group=self.group)
        out, off = {}, 0
        for name, shape, dtype, nbytes in info["manifest"]:
            out[name] = flat[off:off + nbytes].view(dtype).reshape(shape)
            off += nbytes
        return out, info["version"], info["last"]


def receive_all(transport: BroadcastTransport, server) -> int:
    """Replica side of a broadcast sync: collect buckets until the last one, then load."""
    state: dict[str, torch.Tensor] = {}
    while True:
        part, version, last = transport.receive()
        state.update({k: v.clone() for k, v in part.items()})
        if last:
            server.update_weights(state, version)
            return version


class WeightSync:
    def __init__(self, cfg: SyncConfig, transport, servers: Optional[list] = None):
        self.cfg, self.transport, self.servers = cfg, transport, servers or []
        self.last_seconds = 0.0
        self.bytes_sent = 0

    def sync(self, state: dict[str, torch.Tensor], version: int) -> dict:
        t0 = time.time()
        aborted = sum(s.pause(abort=True) for s in self.servers)
        for s in self.servers:
            s.release_cached_memory()
        sent = 0
        bl = list(buckets(state.items(), self.cfg))
        for i, b in enumerate(bl):
            self.transport.send(b, version, last=(i == len(bl) - 1))
            sent += sum(t.numel() * t.element_size() for _, t in b)
        for s in self.servers:
            s.resume()
        self.last_seconds, self.bytes_sent = time.time() - t0, sent
        return {"weight_sync/seconds": self.last_seconds, "weight_sync/bytes": float(sent), "weight_sync/buckets": float(len(bl)),
                "weight_sync/aborted_requests": float(aborted)}

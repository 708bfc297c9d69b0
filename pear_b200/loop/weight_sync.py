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
* ``SymmTransport``: trainer rank and replica ranks of one node share symmetric memory (``parallel/symm.py``); the
  sender stages a bucket once, every replica rank pulls ONLY the blocks of its own tensor-parallel shard out of it with
  peer loads over NVSwitch (the sender's egress is one model, not one model per receiver), and a receiver that serves in
  NVFP4 quantises while it pulls (``bcast_quant_nvfp4_kernel``).
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


class StandaloneGroup:
    """A process group of its own world, beside whatever ``torch.distributed`` world the process already belongs to: the
    trainer's rank 0 (member of the training world) and the rollout replicas (each possibly the member of a tensor-parallel
    world) meet here for weight syncs only. Rank 0 of this group hosts the rendezvous store at ``master`` (``host:port``).
    Backends: ``gloo`` (host tensors) and ``nccl`` (tensors on ``device``). (Upstream names such a group per sync in its
    checkpoint engine: pear/rollout/checkpoint_engine.py:15-43.)"""

    def __init__(self, master: str, rank: int, world: int, backend: str = "gloo", device="cpu", timeout_s: float = 1800.0):
        from datetime import timedelta

        host, port = master.rsplit(":", 1)
        self.rank, self.world, self.backend, self.device = rank, world, backend, torch.device(device)
        timeout = timedelta(seconds=timeout_s)
        self.store = dist.TCPStore(host, int(port), world, is_master=(rank == 0), timeout=timeout)
        store = dist.PrefixStore("weight_sync", self.store)
        if backend == "nccl":
            torch.cuda.set_device(self.device)
            self.pg = dist.ProcessGroupNCCL(store, rank, world, timeout)
        elif backend == "gloo":
            self.pg = dist.ProcessGroupGloo(store, rank, world, timeout)
        else:
            raise ValueError(f"unknown backend {backend!r}")

    def broadcast(self, t: torch.Tensor, src: int) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank, opts.rootTensor = src, 0
        self.pg.broadcast([t], opts).wait()
        if t.is_cuda:
            torch.cuda.current_stream(t.device).synchronize()

    def broadcast_object(self, obj, src: int):
        """Pickled through two broadcasts (length, then bytes); returns the object on every rank."""
        import pickle

        dev = self.device if self.backend == "nccl" else torch.device("cpu")
        if self.rank == src:
            payload = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8).to(dev)
            n = torch.tensor([payload.numel()], dtype=torch.int64, device=dev)
        else:
            n = torch.zeros(1, dtype=torch.int64, device=dev)
        self.broadcast(n, src)
        if self.rank != src:
            payload = torch.empty(int(n.item()), dtype=torch.uint8, device=dev)
        self.broadcast(payload, src)
        return obj if self.rank == src else pickle.loads(payload.cpu().numpy().tobytes())

    def heartbeat(self, timeout_s: float = 30.0):
        """A :class:`pear_b200.parallel.heartbeat.Heartbeat` of this world over its rendezvous store: replica ranks beat from a
        thread of their own, the sender checks before every sync, so a replica that died is named on the host instead of being
        waited for inside a broadcast."""
        from ..parallel.heartbeat import Heartbeat

        return Heartbeat(self.store, self.rank, self.world, timeout_s, prefix="weight_sync_hb")

    def close(self) -> None:
        self.pg = None
        self.store = None


class BroadcastTransport:
    """Rank ``src`` of ``group`` owns the weights; every other rank calls ``receive`` with the same manifest. ``group`` is a
    ``torch.distributed`` group (None: the default world) or a :class:`StandaloneGroup`."""

    def __init__(self, group=None, src: int = 0, device="cpu"):
        self.group, self.src, self.device = group, src, torch.device(device)

    def _object(self, obj):
        if isinstance(self.group, StandaloneGroup):
            return self.group.broadcast_object(obj, self.src)
        box = [obj]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]

    def _tensor(self, t: torch.Tensor) -> None:
        if isinstance(self.group, StandaloneGroup):
            self.group.broadcast(t, self.src)
        else:
            dist.broadcast(t, src=self.src, group=self.group)

    def send(self, bucket: list[tuple[str, torch.Tensor]], version: int, last: bool) -> None:
        manifest = [(n, tuple(t.shape), t.dtype, t.numel() * t.element_size()) for n, t in bucket]
        self._object({"manifest": manifest, "version": version, "last": last})
        self._tensor(torch.cat([t.detach().contiguous().view(-1).view(torch.uint8).to(self.device) for _, t in bucket]))

    def receive(self) -> tuple[dict[str, torch.Tensor], int, bool]:
        info = self._object(None)
        total = sum(m[3] for m in info["manifest"])
        flat = torch.empty(total, dtype=torch.uint8, device=self.device)
        self._tensor(flat)
        out, off = {}, 0
        for name, shape, dtype, nbytes in info["manifest"]:
            out[name] = flat[off:off + nbytes].view(dtype).reshape(shape)
            off += nbytes
        return out, info["version"], info["last"]


class SymmTransport:
    """NVSwitch transport over a :class:`pear_b200.parallel.symm.SymmWorld` whose group holds the sending trainer rank and
    the replica ranks. Per bucket: the sender copies the (already cast) tensors into its symmetric staging buffer and
    publishes a manifest; after a device barrier every receiver pulls the blocks ``shard_pieces`` names for its
    tensor-parallel rank straight out of the sender's buffer (own kernel, 16-byte peer loads); a second barrier hands the
    buffer back. With ``nvfp4`` the 2-D weights whose inner size is a multiple of 256 arrive as ``(packed, scale)`` in the
    decode megakernel's stage layout, quantised during the pull; everything else stays in the rollout dtype.
    (Upstream broadcasts whole buckets with NCCL and casts on the receiver: pear/rollout/checkpoint_engine.py:15-43.)"""

    def __init__(self, symm, src: int, model_cfg=None, tp_rank: int = 0, tp_world: int = 1, bucket_megabytes: int = 512, nvfp4: bool = False):
        self.symm, self.src = symm, src
        self.model_cfg, self.tp_rank, self.tp_world, self.nvfp4 = model_cfg, tp_rank, tp_world, nvfp4
        self.capacity = (bucket_megabytes << 20) + (1 << 20)  # offsets are rounded up to 256 bytes per tensor
        self.staging = symm.alloc((self.capacity,), torch.uint8)
        self.bytes_pulled = 0

    # -- sender -------------------------------------------------------------------------------------------------------
    def send(self, bucket: list[tuple[str, torch.Tensor]], version: int, last: bool) -> None:
        manifest, off = [], 0
        for name, t in bucket:
            nbytes = t.numel() * t.element_size()
            if off + nbytes > self.capacity:
                raise ValueError(f"bucket of {off + nbytes} bytes exceeds the staging buffer ({self.capacity}); lower bucket_megabytes")
            self.staging.tensor[off:off + nbytes].copy_(t.detach().contiguous().view(-1).view(torch.uint8), non_blocking=True)
            manifest.append((name, tuple(t.shape), t.dtype, off))
            off = (off + nbytes + 255) // 256 * 256
        obj = [{"manifest": manifest, "version": version, "last": last}]
        dist.broadcast_object_list(obj, src=dist.get_global_rank(self.symm.group, self.src), group=self.symm.group)
        self.symm.device_barrier()  # the bucket is complete in the sender's buffer
        self.symm.device_barrier()  # every receiver has pulled what it needs: the buffer may be overwritten

    # -- receivers ----------------------------------------------------------------------------------------------------
    def receive(self) -> tuple[dict, int, bool]:
        import ctypes

        from ..ops import lib as _lib
        from ..parallel.tensor_parallel import shard_pieces, shard_shape

        obj = [None]
        dist.broadcast_object_list(obj, src=dist.get_global_rank(self.symm.group, self.src), group=self.symm.group)
        info = obj[0]
        self.symm.device_barrier()
        base = self.staging.ptrs[self.src]
        out: dict = {}
        for name, shape, dtype, off in info["manifest"]:
            es = torch.empty(0, dtype=dtype).element_size()
            pieces = shard_pieces(name, shape, self.model_cfg, self.tp_rank, self.tp_world) if self.model_cfg is not None and self.tp_world > 1 \
                else [(0, int(shape[0]) if shape else 1, 0, int(torch.Size(shape[1:]).numel()) if len(shape) > 1 else 1)]
            full_cols = int(torch.Size(shape[1:]).numel()) if len(shape) > 1 else 1
            local_shape = shard_shape(shape, pieces)
            if (self.nvfp4 and len(shape) == 2 and dtype == torch.bfloat16 and len(pieces) == 1 and pieces[0][3] == full_cols
                    and full_cols % 256 == 0):  # whole rows (a row cut or a replicated matrix): contiguous in the sender's buffer
                r0, r, c0, c = pieces[0]
                out[name] = self._pull_nvfp4(base + off + r0 * full_cols * es, r, c)
                self.bytes_pulled += r * c * es
                continue
            dst = torch.empty(local_shape, dtype=dtype, device=self.symm.device)
            dst_rows = dst.view(dst.shape[0], -1) if dst.dim() >= 1 and dst.numel() else dst.view(1, -1)
            row = 0
            for r0, r, c0, c in pieces:
                _lib.check(_lib.lib().pear_pull_block(ctypes.c_void_p(base + off + (r0 * full_cols + c0) * es), ctypes.c_longlong(full_cols * es),
                                                      ctypes.c_void_p(dst_rows.data_ptr() + row * dst_rows.shape[1] * es),
                                                      ctypes.c_longlong(dst_rows.shape[1] * es), r, ctypes.c_longlong(c * es), _lib.stream()),
                           "pull_block")
                _lib.count_launch()
                row += r
                self.bytes_pulled += r * c * es
            out[name] = dst
        self.symm.device_barrier()
        return out, info["version"], info["last"]

    def _pull_nvfp4(self, src_ptr: int, rows: int, k: int):
        import ctypes
        import math

        from ..ops import lib as _lib

        lib, dev = _lib.lib(), self.symm.device
        # the tensor scale needs the block's maximum first: one pass of peer loads for it, one for the quantisation
        amax = torch.zeros(1, dtype=torch.int32, device=dev)
        _lib.check(lib.pear_amax_bf16(ctypes.c_void_p(src_ptr), ctypes.c_size_t(rows * k), _lib.ptr(amax), _lib.stream()), "amax_bf16")
        a = float(amax.view(torch.float32).item())
        gs = 1.0 if (a <= 0.0 or not math.isfinite(a)) else 2.0 ** math.floor(math.log2(448.0 * 6.0 / a))
        packed = torch.zeros((rows + 127) // 128, k // 256, 18432, dtype=torch.uint8, device=dev)
        _lib.check(lib.pear_bcast_quant_nvfp4(ctypes.c_void_p(src_ptr), rows, k, k, ctypes.c_float(gs), _lib.ptr(packed), _lib.stream()),
                   "bcast_quant_nvfp4")
        _lib.count_launch(2)
        return packed, gs


def receive_all(transport, server) -> int:
    """Replica side of a broadcast sync: collect buckets until the last one, then load."""
    state: dict[str, torch.Tensor] = {}
    while True:
        part, version, last = transport.receive()
        state.update({k: (v.clone() if torch.is_tensor(v) else v) for k, v in part.items()})
        if last:
            server.update_weights(state, version)
            return version


class WeightSync:
    def __init__(self, cfg: SyncConfig, transport, servers: Optional[list] = None, heartbeat=None, listeners: Optional[list] = None):
        """``heartbeat``: checked before anything of a sync starts (``PeerLost`` names the replica ranks that are gone).
        ``listeners``: callables ``(state, version)`` of this process that also follow the policy (the agent loop's vision
        encoder), called with the trainer's full-precision state while the replicas are paused."""
        self.cfg, self.transport, self.servers, self.heartbeat = cfg, transport, servers or [], heartbeat
        self.listeners = listeners or []
        self.last_seconds = 0.0
        self.bytes_sent = 0

    def sync(self, state: dict[str, torch.Tensor], version: int) -> dict:
        t0 = time.time()
        if self.heartbeat is not None:
            self.heartbeat.beat(version)
            self.heartbeat.check()
        aborted = sum(s.pause(abort=True) for s in self.servers)
        for s in self.servers:
            s.release_cached_memory()
        sent = 0
        bl = list(buckets(state.items(), self.cfg))
        for i, b in enumerate(bl):
            self.transport.send(b, version, last=(i == len(bl) - 1))
            sent += sum(t.numel() * t.element_size() for _, t in b)
        for listen in self.listeners:
            listen(state, version)
        for s in self.servers:
            if hasattr(s, "wait_version"):  # a replica in another process loads on a thread of its own
                s.wait_version(version)
            s.resume()
        self.last_seconds, self.bytes_sent = time.time() - t0, sent
        return {"weight_sync/seconds": self.last_seconds, "weight_sync/bytes": float(sent), "weight_sync/buckets": float(len(bl)),
                "weight_sync/aborted_requests": float(aborted)}

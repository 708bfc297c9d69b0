"""ZeRO-3 style parameter sharding owned by the trainer (no wrapper framework).

Each unit (one decoder layer, or the root: embedding + final norm + head + MTP) flattens its parameters into one
buffer, keeps an fp32 master SHARD of it as the optimizer's parameter, all-gathers the compute-dtype copy right before
the unit runs and frees it right after, and reduce-scatters the unit's gradients as soon as its backward finishes.
Units are driven explicitly by the layer runner (:mod:`pear_b200.train.checkpointing`), which also recomputes the layer
in backward, so gather / recompute / reduce-scatter / release happen in one place per layer.

Behaviours kept from the upstream FSDP2 setup (``3rdparty/verl/patches``): named ``fp32_modules`` become their own fp32
units (0027); with a replicate group (HSDP) the replica all-reduce runs on the last micro-batch only while the
reduce-scatter runs on every micro-batch (0019); the replicate communicator is warmed right after sharding (0020).
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from . import collectives as C


_COMM_STREAMS: dict = {}


def comm_stream(device) -> "torch.cuda.Stream":
    """The side stream (one per device) on which prefetched all-gathers and gradient reduce-scatters run."""
    key = torch.device(device)
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(key)
    return _COMM_STREAMS[key]


class FlatUnit:
    overlap = True  # multi-rank CUDA runs: gathers are prefetched and gradients reduced on the side stream

    def __init__(self, name: str, params: list[tuple[str, nn.Parameter]], shard_group=None, replicate_group=None,
                 compute_dtype: torch.dtype = torch.bfloat16, device=None, average: bool = False, src_rank: Optional[int] = None):
        """``src_rank``: only that rank of the shard group holds real parameters (the others built the model on the meta
        device); the unit's fp32 flat buffer is broadcast from it and every rank keeps its own shard (upstream:
        3rdparty/verl/patches/0031 — meta-device ranks receive the weights by broadcast)."""
        self.name = name
        self.average = average  # False: gradients are SUMMED over ranks (the loss is already normalised globally)
        self.names = [n for n, _ in params]
        self.params = [p for _, p in params]
        self.group, self.replicate_group = shard_group, replicate_group
        self.world = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.rank = dist.get_rank(shard_group) if shard_group is not None else 0
        self.compute_dtype = compute_dtype
        self.shapes = [tuple(getattr(p, "_full_shape", p.shape)) for p in self.params]  # (meta-built ranks: see ShardedModel)
        self.numels = [int(torch.Size(s).numel()) for s in self.shapes]
        total = sum(self.numels)
        align = 8 * self.world  # 16-byte aligned bf16 shards
        self.padded = (total + align - 1) // align * align
        self.shard_numel = self.padded // self.world
        device = device or self.params[0].device
        flat = torch.zeros(self.padded, dtype=torch.float32, device=device)
        if src_rank is None or self.rank == src_rank:
            o = 0
            for p, n in zip(self.params, self.numels):
                flat[o : o + n] = p.detach().reshape(-1).float().to(device)
                o += n
        if src_rank is not None and self.world > 1:
            dist.broadcast(flat, dist.get_global_rank(shard_group, src_rank), group=shard_group)
        # the optimizer's parameter: this rank's fp32 master shard
        self.shard = nn.Parameter(flat[self.rank * self.shard_numel : (self.rank + 1) * self.shard_numel].clone())
        self.full: Optional[torch.Tensor] = None
        self._empty = torch.empty(0, dtype=compute_dtype, device=device)
        for p in self.params:
            p.data = self._empty
        self.gathered = False
        self._pending = None  # (full buffer, ready event) of a prefetched gather
        self._grad_pending = False

    def _overlapped(self) -> bool:
        return FlatUnit.overlap and self.world > 1 and self.shard.is_cuda

    # -- parameter lifetime -----------------------------------------------------------------------------------------
    def prefetch(self) -> None:
        """Start this unit's all-gather on the side stream (the layer before it is still computing); ``gather`` picks the
        result up. Without overlap (one rank, CPU) it does nothing and ``gather`` runs the collective itself."""
        if self.gathered or self._pending is not None or not self._overlapped():
            return
        cur, side = torch.cuda.current_stream(self.shard.device), comm_stream(self.shard.device)
        side.wait_stream(cur)  # the shard as the optimizer (or a load) on the compute stream left it
        with torch.cuda.stream(side):
            local = self.shard.detach().to(self.compute_dtype)
            full = torch.empty(self.padded, dtype=self.compute_dtype, device=local.device)
            dist.all_gather_into_tensor(full, local.contiguous(), group=self.group)
            ready = torch.cuda.Event()
            ready.record(side)
        self._pending = (full, ready)

    def gather(self, stream=None) -> None:
        if self.gathered:
            return
        if self._pending is not None:
            full, ready = self._pending
            self._pending = None
            cur = torch.cuda.current_stream(full.device)
            cur.wait_event(ready)
            full.record_stream(cur)  # allocated on the side stream, used (and freed) on the compute stream
        else:
            local = self.shard.detach().to(self.compute_dtype)
            if self.world > 1:
                full = torch.empty(self.padded, dtype=self.compute_dtype, device=local.device)
                dist.all_gather_into_tensor(full, local.contiguous(), group=self.group)
            else:
                full = local if local.data_ptr() != self.shard.data_ptr() else local.clone()
        self.full = full
        o = 0
        for p, n, shp in zip(self.params, self.numels, self.shapes):
            p.data = full[o : o + n].view(shp)
            o += n
        self.gathered = True

    def release(self) -> None:
        for p in self.params:
            p.data = self._empty
        self.full = None
        self.gathered = False

    # -- gradients ----------------------------------------------------------------------------------------------------
    def reduce_grads(self, last_micro_batch: bool = True) -> None:
        """Flatten the unit's full gradients, reduce-scatter over the shard group into the master shard's ``.grad``
        (accumulating over micro-batches), and all-reduce over the replicate group on the last micro-batch."""
        average = self.average
        # one pass over the unit: every gradient is converted straight into its slice (no fp32 temporary, no memset of the whole
        # buffer); only a parameter without a gradient and the alignment tail are zeroed
        flat = torch.empty(self.padded, dtype=torch.float32, device=self.shard.device)
        o = 0
        for p, n in zip(self.params, self.numels):
            if p.grad is not None:
                flat[o : o + n].copy_(p.grad.reshape(-1))
                p.grad = None
            else:
                flat[o : o + n].zero_()
            o += n
        if o < self.padded:
            flat[o:].zero_()

        def finish(flat):
            if self.world > 1:
                piece = C.reduce_scatter_sum(flat, self.group)
                if average:
                    piece = piece / self.world
            else:
                piece = flat
            if self.shard.grad is None:
                self.shard.grad = piece.clone()
            else:
                self.shard.grad.add_(piece)
            if last_micro_batch and self.replicate_group is not None and dist.get_world_size(self.replicate_group) > 1:
                dist.all_reduce(self.shard.grad, group=self.replicate_group)
                if average:
                    self.shard.grad.div_(dist.get_world_size(self.replicate_group))

        if self._overlapped():
            # the reduce-scatter (and the accumulation into the shard's gradient) runs on the side stream under the backward
            # of the next layer; `wait_grads` joins it before anything on the compute stream reads the gradient
            cur, side = torch.cuda.current_stream(flat.device), comm_stream(flat.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                finish(flat)
            flat.record_stream(side)
            self._grad_pending = True
        else:
            finish(flat)

    def wait_grads(self) -> None:
        if self._grad_pending:
            torch.cuda.current_stream(self.shard.device).wait_stream(comm_stream(self.shard.device))
            self._grad_pending = False

    # -- full state (checkpoint export, weight sync) ------------------------------------------------------------------
    def full_state(self, dtype=torch.float32) -> dict[str, torch.Tensor]:
        local = self.shard.detach().to(dtype)
        if self.world > 1:
            full = torch.empty(self.padded, dtype=dtype, device=local.device)
            dist.all_gather_into_tensor(full, local.contiguous(), group=self.group)
        else:
            full = local
        out, o = {}, 0
        for name, n, shp in zip(self.names, self.numels, self.shapes):
            out[name] = full[o : o + n].view(shp).clone()
            o += n
        return out

    def load_full_state(self, state: dict[str, torch.Tensor]) -> None:
        flat = torch.zeros(self.padded, dtype=torch.float32, device=self.shard.device)
        o = 0
        for name, n in zip(self.names, self.numels):
            flat[o : o + n] = state[name].reshape(-1).float().to(flat.device)
            o += n
        with torch.no_grad():
            self.shard.copy_(flat[self.rank * self.shard_numel : (self.rank + 1) * self.shard_numel])


class ShardedModel:
    """The model's parameters as flat sharded units: one per decoder layer, fp32 units for ``fp32_modules``, one root."""

    def __init__(self, model: nn.Module, shard_group=None, replicate_group=None, compute_dtype=torch.bfloat16,
                 fp32_modules: Iterable[str] = (), device=None, src_rank: Optional[int] = None):
        """``src_rank``: the one rank whose ``model`` holds real weights (see :class:`FlatUnit`); the units are built in the
        same order on every rank, one broadcast each, so no rank but the source ever holds more than one unit in full."""
        self.model = model
        # a rank that built the model on the meta device: every parameter becomes an empty real tensor that remembers its
        # shape (a meta tensor cannot be given storage later)
        swapped: dict[int, nn.Parameter] = {}  # a parameter shared by two modules stays shared
        for mod in model.modules():
            for pname, p in list(mod._parameters.items()):
                if p is not None and p.is_meta:
                    if id(p) not in swapped:
                        real = nn.Parameter(torch.empty(0, dtype=p.dtype, device=device), requires_grad=p.requires_grad)
                        real._full_shape = tuple(p.shape)
                        swapped[id(p)] = real
                    mod._parameters[pname] = swapped[id(p)]
        self.units: dict[str, FlatUnit] = {}
        taken: set[int] = set()
        named = dict(model.named_parameters())
        fp32_modules = tuple(fp32_modules)

        def make(name: str, items: list[tuple[str, nn.Parameter]], dtype) -> None:
            items = [(n, p) for n, p in items if id(p) not in taken]
            if not items:
                return
            taken.update(id(p) for _, p in items)
            self.units[name] = FlatUnit(name, items, shard_group, replicate_group, dtype, device, src_rank=src_rank)

        for pat in fp32_modules:
            make(f"fp32:{pat}", [(n, p) for n, p in named.items() if pat in n], torch.float32)
        self.layer_units: list[FlatUnit] = []
        for i, layer in enumerate(model.model.layers):
            make(f"layer{i}", [(f"model.layers.{i}.{n}", p) for n, p in layer.named_parameters()], compute_dtype)
            self.layer_units.append(self.units[f"layer{i}"])
        make("root", [(n, p) for n, p in named.items()], compute_dtype)
        self.root = self.units.get("root")
        if replicate_group is not None and dist.get_world_size(replicate_group) > 1:
            # warm the replicate communicator while memory is still free
            dist.all_reduce(torch.zeros(1, device=self.root.shard.device), group=replicate_group)

    def parameters(self) -> list[nn.Parameter]:
        return [u.shard for u in self.units.values()]

    def gather_static(self) -> None:
        for name, u in self.units.items():
            if not name.startswith("layer"):
                u.gather()

    def release_static(self) -> None:
        for name, u in self.units.items():
            if not name.startswith("layer"):
                u.release()

    def reduce_static_grads(self, last_micro_batch: bool = True) -> None:
        for name, u in self.units.items():
            if not name.startswith("layer"):
                u.reduce_grads(last_micro_batch)

    def wait_grads(self) -> None:
        """Join the side stream: every unit's reduced gradient is complete for the compute stream."""
        for u in self.units.values():
            u.wait_grads()

    def full_state_dict(self, dtype=torch.float32) -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        for u in self.units.values():
            out.update(u.full_state(dtype))
        return out

    def load_full_state_dict(self, state: dict[str, torch.Tensor]) -> None:
        for u in self.units.values():
            u.load_full_state(state)

    def shard_state(self) -> dict:
        """This rank's flat shards plus the layout (unit -> parameter name -> (offset, shape) in the unit's full flat
        buffer) an offline merger needs to rebuild the tensors from all ranks' files."""
        out: dict = {name: u.shard.detach().clone() for name, u in self.units.items()}
        layout = {}
        for uname, u in self.units.items():
            o, meta = 0, {}
            for name, n, shp in zip(u.names, u.numels, u.shapes):
                meta[name] = (o, tuple(shp))
                o += n
            layout[uname] = meta
        out["__layout__"] = layout
        return out

    def load_shard_state(self, state: dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for name, u in self.units.items():
                u.shard.copy_(state[name])

"""Symmetric memory over NVLink / NVSwitch and the kernels that use it.

Every rank of a process group allocates the same buffers (``torch.distributed._symmetric_memory``) and learns every
peer's address; the kernels of ``ops/csrc/comm_kernels.cu`` and ``ops/csrc/gemm_collective.cu`` then read or write peer
memory directly. This module owns the buffers, the flag protocol (slots x source ranks of monotonically growing
epochs) and the Python entry points:

* ``all_reduce_add_rmsnorm``: tensor-parallel partial rows -> all-reduce + fp32 residual add + (1 + w) RMSNorm, one
  kernel (upstream ``rollout/blackwell/csrc/ar_norm.cu`` at TP2; here any power of two up to 8);
* ``ag_gemm``: all-gather -> GEMM with the A tiles pulled from their owners by the GEMM's own TMA producer;
* ``gemm_rs``: GEMM -> reduce-scatter with the epilogue adding tiles into the owner's buffer;
* ``pull_quantize_nvfp4``: weight broadcast fused with bf16 -> NVFP4 requantisation on the receiver (the NVSwitch
  transport of the trainer -> rollout weight sync; upstream broadcasts with NCCL and casts afterwards,
  ``rollout/checkpoint_engine.py:36-43``).

Every device-side wait is bounded; ``check()`` raises if a kernel recorded a timeout.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import lib as _lib

SLOTS = 32
SLOT_AR, SLOT_AG, SLOT_RS_DONE, SLOT_SYNC, SLOT_LOGITS, SLOT_ARGMAX = 0, 1, 3, 4, 5, 6
DEFAULT_BUDGET = 1 << 22  # polls of >= 100 ns: a few hundred milliseconds, then the kernel gives up


class SymmBuffer:
    def __init__(self, tensor: torch.Tensor, ptrs: list[int]):
        self.tensor, self.ptrs = tensor, ptrs
        self.c_ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)


class SymmWorld:
    def __init__(self, group=None, device: Optional[torch.device] = None, reductions: bool = True):
        """``reductions=False``: a world that only allocates, signals and pulls (the weight-sync group of one trainer rank and
        the replica ranks, e.g. 1 + 4) may have any size up to 8; the reduction kernels need a power of two."""
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8 or (reductions and self.world & (self.world - 1)):
            raise ValueError(f"world size {self.world}: the NVSwitch kernels take a power of two up to 8")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.flags = self.alloc((SLOTS * 8,), torch.int32)
        self.flags.tensor.zero_()
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.epochs = [0] * SLOTS
        self._dev_counters: dict = {}
        self._ag_bufs: dict = {}
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    # -- memory -------------------------------------------------------------------------------------------------------
    def alloc(self, shape, dtype) -> SymmBuffer:
        t = self._symm.empty(shape, dtype=dtype, device=self.device)
        h = self._symm.rendezvous(t, self.group.group_name)
        buf = SymmBuffer(t, [int(p) for p in h.buffer_ptrs])
        buf.handle = h
        # the NVLS multicast address of the buffer (0 when the platform gives none): `multimem` loads from it return the sum over
        # all ranks' buffers, stores to it land in all of them
        try:
            buf.mc_ptr = int(getattr(h, "multicast_ptr", 0) or 0)
        except Exception:  # noqa: BLE001
            buf.mc_ptr = 0
        return buf

    def device_counter(self, slot: int) -> torch.Tensor:
        """The device-resident epoch of a flag slot (kernels that must replay inside a CUDA graph read and advance it
        themselves). One counter per slot for the whole ``SymmWorld``: every user of the slot continues the same epoch
        sequence, so flags left by an earlier user can never satisfy a later user's wait."""
        if slot not in self._dev_counters:
            self._dev_counters[slot] = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self._dev_counters[slot]

    def check(self) -> None:
        code = int(self.status[0].item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"rank {self.rank}: a device-side wait on a peer gave up (status {code})")

    # -- flags --------------------------------------------------------------------------------------------------------
    def next_epoch(self, slot: int) -> int:
        self.epochs[slot] += 1
        return self.epochs[slot]

    def signal(self, slot: int, epoch: int) -> None:
        _lib.check(_lib.lib().pear_symm_signal(self.flags.c_ptrs, self.rank, self.world, slot, epoch, _lib.stream()), "symm_signal")

    def wait(self, slot: int, epoch: int, budget: int = DEFAULT_BUDGET) -> None:
        _lib.check(_lib.lib().pear_symm_wait(_lib.ptr(self.flags.tensor), self.world, slot, epoch, budget, _lib.ptr(self.status),
                                              _lib.stream()), "symm_wait")

    def device_barrier(self, slot: int = SLOT_SYNC) -> None:
        """All ranks' streams meet: everything issued before on any rank is visible to everything issued after."""
        e = self.next_epoch(slot)
        self.signal(slot, e)
        self.wait(slot, e)

    # -- all-reduce + residual add + RMSNorm --------------------------------------------------------------------------
    def make_ar_workspace(self, max_rows: int, hidden: int) -> SymmBuffer:
        return self.alloc((2, max_rows, hidden), torch.bfloat16)

    def all_reduce_add_rmsnorm(self, ws: SymmBuffer, partial: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                               eps: float = 1e-6, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += sum_ranks(partial)`` (fp32, in place); returns ``rmsnorm(residual) * (1 + weight)`` in bf16."""
        t, h = partial.shape
        e = self.next_epoch(SLOT_AR)
        ws.tensor[e & 1, :t].copy_(partial)
        out = out if out is not None else torch.empty(t, h, dtype=torch.bfloat16, device=self.device)
        buf_elems = ws.tensor.shape[1] * ws.tensor.shape[2]
        if ws.tensor.shape[2] != h:
            raise ValueError("workspace hidden size mismatch")
        _lib.check(_lib.lib().pear_ar_add_rmsnorm(ws.c_ptrs, self.flags.c_ptrs, self.rank, self.world, SLOT_AR, e, _lib.ptr(residual),
                                                   _lib.ptr(weight), _lib.ptr(out), t, h, ctypes.c_size_t(buf_elems), ctypes.c_float(eps),
                                                   DEFAULT_BUDGET, _lib.ptr(self.status), 2 * self.num_sms, _lib.stream()), "ar_add_rmsnorm")
        _lib.LAUNCH_COUNT += 1
        return out

    # -- all-gather -> GEMM -------------------------------------------------------------------------------------------
    def ag_gemm(self, a_shard: SymmBuffer, b: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
        """``C = concat_ranks(A_shard) @ B^T``. ``a_shard.tensor`` [M / world, K] bf16 must be written on this stream
        before the call; the call publishes it and the kernel pulls the other shards from their owners."""
        ml, k = a_shard.tensor.shape
        n = b.shape[0]
        m = ml * self.world
        c = torch.empty(m, n, dtype=out_dtype, device=self.device)
        key = (m, k)
        if key not in self._ag_bufs:  # local full-A buffer + one flag per 128-row block, kept across calls
            self._ag_bufs[key] = (torch.empty(m, k, dtype=torch.bfloat16, device=self.device),
                                  torch.zeros(m // 128, dtype=torch.int32, device=self.device))
        a_full, chunk_flags = self._ag_bufs[key]
        chunk_flags.zero_()  # piece counters of the remote blocks
        e = self.next_epoch(SLOT_AG)
        self.signal(SLOT_AG, e)
        _lib.check(_lib.lib().pear_ag_gemm_bf16(a_shard.c_ptrs, _lib.ptr(b), _lib.ptr(c), m, n, k, a_shard.tensor.stride(0), b.stride(0),
                                                 c.stride(0), 1 if out_dtype == torch.bfloat16 else 0, self.rank, self.world,
                                                 _lib.ptr(self.flags.tensor), SLOT_AG, e, DEFAULT_BUDGET, _lib.ptr(self.status), self.num_sms,
                                                 _lib.ptr(a_full), _lib.ptr(chunk_flags), _lib.stream()), "ag_gemm")
        _lib.LAUNCH_COUNT += 1
        return c

    def ag_gemm_done(self) -> None:
        """Call before overwriting the A shard again: every rank has finished pulling it."""
        self.device_barrier()

    # -- GEMM -> reduce-scatter ---------------------------------------------------------------------------------------
    def make_rs_accumulator(self, rows_local: int, n: int) -> SymmBuffer:
        """Staging for ``gemm_rs``: one bf16 slot of this rank's rows per source rank, plus per-tile flags."""
        buf = self.alloc((self.world, rows_local, n), torch.bfloat16)
        tiles = (rows_local // 128) * ((n + 255) // 256)
        buf.flags = self.alloc((self.world, tiles), torch.int32)
        buf.flags.tensor.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        return buf

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, acc: SymmBuffer) -> torch.Tensor:
        """``sum_ranks(A_r @ B_r^T)`` restricted to this rank's rows, fp32 [M / world, N]."""
        m, k = a.shape
        n = b.shape[0]
        out = torch.empty(m // self.world, n, dtype=torch.float32, device=self.device)
        self.device_barrier()  # every rank has finished reading what the previous call pushed into its staging buffer
        e = self.next_epoch(SLOT_RS_DONE)
        stage = (ctypes.c_void_p * self.world)(*acc.ptrs)
        flags = (ctypes.c_void_p * self.world)(*acc.flags.ptrs)
        _lib.check(_lib.lib().pear_gemm_rs_bf16(_lib.ptr(a), _lib.ptr(b), stage, flags, _lib.ptr(out), m, n, k, a.stride(0), b.stride(0), out.stride(0),
                                                 self.rank, self.world, e, DEFAULT_BUDGET, _lib.ptr(self.status), self.num_sms, _lib.stream()), "gemm_rs")
        _lib.LAUNCH_COUNT += 1
        return out

    # -- projection GEMM -> all-to-all (Ulysses: token-sharded in, head-sharded out) -----------------------------------
    def make_a2a_buffer(self, rows_local: int, cols_per_rank: int) -> SymmBuffer:
        return self.alloc((self.world * rows_local, cols_per_rank), torch.bfloat16)

    def gemm_a2a(self, a: torch.Tensor, b: torch.Tensor, out: SymmBuffer) -> torch.Tensor:
        """``a`` [M, K]: this rank's tokens, ``b`` [N, K]: the full projection weight. Column group p of ``a @ b^T`` (width
        N / world: the heads of rank p) is stored by the GEMM's epilogue into rank p's ``out`` at rows [rank * M, ...):
        after the call ``out.tensor`` [world * M, N / world] holds every rank's tokens for this rank's heads."""
        m, k = a.shape
        n = b.shape[0]
        self.device_barrier()  # every rank has finished reading what the previous call stored into its buffer
        _lib.check(_lib.lib().pear_gemm_a2a_bf16(_lib.ptr(a), _lib.ptr(b), out.c_ptrs, m, n, k, a.stride(0), b.stride(0), out.tensor.stride(0),
                                                  self.rank, self.world, _lib.ptr(self.status), self.num_sms, _lib.stream()), "gemm_a2a")
        _lib.LAUNCH_COUNT += 1
        self.device_barrier()  # every rank's stores have landed here
        return out.tensor

    # -- all-to-all -> GEMM (Ulysses: head-sharded attention output in, token-sharded output projection out) -----------
    def a2a_gemm(self, src: SymmBuffer, b: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
        """``src.tensor`` [world * M, K / world] (all tokens, this rank's columns: written on this stream before the call).
        Returns ``C`` [M, N] = this rank's tokens over the whole K times ``b^T``; the peers' column groups are pulled by
        the GEMM's copier warps while it already multiplies the local group."""
        rows, kg = src.tensor.shape
        m, k, n = rows // self.world, kg * self.world, b.shape[0]
        c = torch.empty(m, n, dtype=out_dtype, device=self.device)
        key = ("a2a", m, k)
        if key not in self._ag_bufs:
            self._ag_bufs[key] = (torch.empty(m, k, dtype=torch.bfloat16, device=self.device),
                                  torch.zeros(m // 128 * self.world, dtype=torch.int32, device=self.device))
        a_full, chunk_flags = self._ag_bufs[key]
        chunk_flags.zero_()
        e = self.next_epoch(SLOT_AG)
        self.signal(SLOT_AG, e)
        _lib.check(_lib.lib().pear_a2a_gemm_bf16(src.c_ptrs, _lib.ptr(b), _lib.ptr(c), m, n, k, b.stride(0), c.stride(0),
                                                  1 if out_dtype == torch.bfloat16 else 0, self.rank, self.world, _lib.ptr(self.flags.tensor),
                                                  SLOT_AG, e, DEFAULT_BUDGET, _lib.ptr(self.status), self.num_sms, _lib.ptr(a_full),
                                                  _lib.ptr(chunk_flags), _lib.stream()), "a2a_gemm")
        _lib.LAUNCH_COUNT += 1
        return c

    def a2a_gemm_done(self) -> None:
        """Call before overwriting ``src`` again: every rank has finished pulling from it."""
        self.device_barrier()

    # -- vocab-parallel logits all-gather -----------------------------------------------------------------------------
    def all_gather_logits(self, shard: torch.Tensor, full: SymmBuffer) -> torch.Tensor:
        """Write this rank's fp32 logits shard [T, V / world] into every rank's ``full`` [T, V]; returns the local full
        buffer once every rank's shard has landed in it. Reuse contract: the call starts with a device barrier, so a rank that
        is still reading the previous call's ``full`` (its sampler) is never overwritten by a faster peer's next call."""
        t, vs = shard.shape
        self.device_barrier()
        _lib.check(_lib.lib().pear_logits_allgather(_lib.ptr(shard.contiguous()), full.c_ptrs, self.rank, self.world, t, vs,
                                                     full.tensor.stride(0), _lib.stream()), "logits_allgather")
        _lib.LAUNCH_COUNT += 1
        e = self.next_epoch(SLOT_LOGITS)
        self.signal(SLOT_LOGITS, e)
        self.wait(SLOT_LOGITS, e)
        return full.tensor[:t]

    # -- sharded argmax (drafter's greedy token under vocabulary parallelism) -------------------------------------------
    def make_argmax_buffer(self, max_rows: int) -> SymmBuffer:
        return self.alloc((max_rows, 8), torch.int64)

    def sharded_argmax(self, logits_shard: torch.Tensor, xbuf: SymmBuffer) -> tuple[torch.Tensor, torch.Tensor]:
        """Global (token, value) of the row-wise maximum over the vocabulary, each rank holding columns
        ``[rank * Vs, (rank + 1) * Vs)``; ties go to the lower token id. Starts with a device barrier (same reuse contract as
        :meth:`all_gather_logits`: ``xbuf`` of the previous call may still be read by a slower peer's ``argmax_finish``)."""
        rows, vs = logits_shard.shape
        lib = _lib.lib()
        self.device_barrier()
        _lib.check(lib.pear_argmax_shard(_lib.ptr(logits_shard), rows, vs, logits_shard.stride(0), self.rank * vs, xbuf.c_ptrs, self.rank,
                                         self.world, _lib.stream()), "argmax_shard")
        e = self.next_epoch(SLOT_ARGMAX)
        self.signal(SLOT_ARGMAX, e)
        self.wait(SLOT_ARGMAX, e)
        tok = torch.empty(rows, dtype=torch.int32, device=self.device)
        val = torch.empty(rows, dtype=torch.float32, device=self.device)
        _lib.check(lib.pear_argmax_finish(_lib.ptr(xbuf.tensor), rows, self.world, _lib.ptr(tok), _lib.ptr(val), _lib.stream()), "argmax_finish")
        _lib.LAUNCH_COUNT += 2
        return tok.long(), val

    # -- weight sync: pull bf16 from the sender, write NVFP4 ----------------------------------------------------------
    def pull_quantize_nvfp4(self, staging: SymmBuffer, src_rank: int, rows: int, k: int) -> tuple[torch.Tensor, float]:
        """Receiver side: read ``[rows, k]`` bf16 from ``src_rank``'s staging buffer over NVLink and return the weight in
        the decode megakernel's NVFP4 stage layout plus its power-of-two tensor scale. The sender must have published
        the buffer (``device_barrier`` after writing it)."""
        import math

        src = staging.ptrs[src_rank]
        bits = torch.zeros(1, dtype=torch.int32, device=self.device)
        lib = _lib.lib()
        _lib.check(lib.pear_amax_bf16(ctypes.c_void_p(src), ctypes.c_size_t(rows * k), _lib.ptr(bits), _lib.stream()), "amax_bf16")
        amax = float(bits.view(torch.float32).item())
        gs = 1.0 if (amax <= 0.0 or not math.isfinite(amax)) else 2.0 ** math.floor(math.log2(448.0 * 6.0 / amax))
        tiles = (rows + 127) // 128
        packed = torch.zeros(tiles, k // 256, 18432, dtype=torch.uint8, device=self.device)
        _lib.check(lib.pear_bcast_quant_nvfp4(ctypes.c_void_p(src), rows, k, k, ctypes.c_float(gs), _lib.ptr(packed), _lib.stream()),
                   "bcast_quant_nvfp4")
        _lib.LAUNCH_COUNT += 2
        return packed, gs


class FusedShardedAdamW:
    """ZeRO-style optimizer step over NVSwitch in two kernels (``ops/csrc/optim_collective.cu``): gradient reduce-scatter +
    scale + norm, then clip + AdamW on the owned shard + all-gather of the new bf16 parameters by peer stores.

    Every rank writes its full flat gradient into ``grads.tensor`` (symmetric memory) and reads the current parameters
    from ``params.tensor``; the fp32 master weights and moments exist only for the owned range. Upstream does the same
    work as an NCCL reduce-scatter, ``_multi_tensor_adam`` on the shards and an NCCL all-gather
    (pear/trainer/engine.py:155-236)."""

    def __init__(self, symm: SymmWorld, numel: int, grads_dtype=torch.bfloat16, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_norm: float = 1.0):
        self.symm = symm
        unit = 8 * symm.world
        self.numel = numel
        self.padded = (numel + unit - 1) // unit * unit
        self.shard = self.padded // symm.world
        self.lo = symm.rank * self.shard
        self.grads = symm.alloc((self.padded,), grads_dtype)
        self.params = symm.alloc((self.padded,), torch.bfloat16)
        self.norms = symm.alloc((8,), torch.float32)
        self.grads.tensor.zero_()
        self.params.tensor.zero_()
        self.norms.tensor.zero_()
        dev = symm.device
        self.master = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.reduced = torch.zeros_like(self.master)
        self.block_sums = torch.zeros(592, dtype=torch.float32, device=dev)
        self.norm_out = torch.zeros(1, dtype=torch.float32, device=dev)
        self.lr, self.betas, self.eps, self.weight_decay, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.t = 0
        torch.cuda.synchronize(dev)
        dist.barrier(symm.group)

    def load_parameters(self, flat: torch.Tensor) -> None:
        """``flat``: the full fp32 parameter vector (same on every rank)."""
        self.master.zero_()
        hi = min(self.lo + self.shard, self.numel)
        if hi > self.lo:
            self.master[: hi - self.lo].copy_(flat[self.lo:hi])
        self.params.tensor[: self.numel].copy_(flat)
        self.symm.device_barrier()

    def step(self, grad_scale: float = 1.0) -> torch.Tensor:
        """One optimizer step over the gradients currently in ``grads.tensor`` on every rank; returns the global gradient
        norm before clipping (device scalar)."""
        s, lib = self.symm, _lib.lib()
        self.t += 1
        b1, b2 = self.betas
        s.device_barrier()  # every rank's gradient bucket is complete
        _lib.check(lib.pear_rs_sumsq(self.grads.c_ptrs, 1 if self.grads.tensor.dtype == torch.bfloat16 else 0, s.rank, s.world,
                                     ctypes.c_size_t(self.lo), ctypes.c_size_t(self.shard), ctypes.c_float(grad_scale), _lib.ptr(self.reduced),
                                     _lib.ptr(self.block_sums), self.norms.c_ptrs, _lib.stream()), "rs_sumsq")
        s.device_barrier()  # every rank's partial norm has landed here; every rank is done reading this rank's gradients
        _lib.check(lib.pear_adamw_bcast(_lib.ptr(self.reduced), _lib.ptr(self.master), _lib.ptr(self.m), _lib.ptr(self.v), _lib.ptr(self.norms.tensor),
                                        self.params.c_ptrs, s.world, ctypes.c_size_t(self.lo), ctypes.c_size_t(self.shard), ctypes.c_float(self.lr),
                                        ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(self.eps), ctypes.c_float(self.weight_decay),
                                        ctypes.c_float(1.0 - b1 ** self.t), ctypes.c_float(1.0 - b2 ** self.t), ctypes.c_float(self.max_norm),
                                        _lib.ptr(self.norm_out), _lib.stream()), "adamw_bcast")
        s.device_barrier()  # the new parameters are visible in every rank's bucket
        _lib.LAUNCH_COUNT += 3
        return self.norm_out

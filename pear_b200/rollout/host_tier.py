"""Host-DRAM tier of the KV cache: evicted prefix blocks (and their recurrent-state snapshots) live on in pinned host
memory and are promoted back on a prefix hit.

It owns the behaviours the upstream stack gets from its LMCache sidecar and the five patches it carries
(``pear/rollout/lmcache.py``, ``3rdparty/LMCache/patches``):
  * LRU with eviction rounds of 5 % of the entries once the tier is 80 % full (``lmcache.py:30-35``);
  * recurrent-state pages that fall outside the load window of a session (a later boundary of the same session was
    stored) are DEMOTED to the cold end of the LRU and never promoted again by touches (patch 0002);
  * a STORE pins every device block it reads from the moment it is scheduled until the copy is done, so blocks freed by
    preemption / finish cannot be reused mid-copy (patch 0001), and it reads the CURRENT block table: freed slots appear
    as the null block and are neither pinned nor stored (patch 0005);
  * a lookup miss on a scheduler retry clears the earlier hit watermark (patch 0004);
  * the whole tier is force-cleared after a weight sync (``lmcache.py:263-274``).
Copies are per-block gathers over the layer caches into a pinned staging row (one ``cudaMemcpyAsync`` per layer cache on
a side stream); on CPU tensors they are plain copies.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .block_manager import NULL_BLOCK


@dataclass
class HostEntry:
    slot: int
    has_state: bool
    demoted: bool = False
    session: Optional[str] = None
    position: int = 0  # block index within its session's sequence


class HostTier:
    def __init__(self, capacity_blocks: int, kv_caches: list[torch.Tensor], state_caches: Optional[list[torch.Tensor]] = None,
                 watermark: float = 0.8, eviction_ratio: float = 0.05, pin: bool = True):
        """``kv_caches``: per layer [num_blocks, ...] device tensors (K and V separately or fused);
        ``state_caches``: per layer [num_slots, ...] recurrent-state / conv-state pools."""
        self.capacity = capacity_blocks
        self.kv_caches = kv_caches
        self.state_caches = state_caches or []
        self.watermark, self.eviction_ratio = watermark, eviction_ratio
        use_pin = pin and torch.cuda.is_available()
        self.kv_host = [torch.empty((capacity_blocks,) + tuple(c.shape[1:]), dtype=c.dtype, pin_memory=use_pin) for c in kv_caches]
        self.state_host = [torch.empty((capacity_blocks,) + tuple(c.shape[1:]), dtype=c.dtype, pin_memory=use_pin)
                           for c in self.state_caches]
        self.entries: "OrderedDict[bytes, HostEntry]" = OrderedDict()  # coldest first
        self.free_slots = list(range(capacity_blocks - 1, -1, -1))
        self.pinned: dict[int, int] = {}  # device block -> outstanding stores reading it
        self.stream = torch.cuda.Stream() if (torch.cuda.is_available() and kv_caches and kv_caches[0].is_cuda) else None
        self.hit_watermark: dict[str, int] = {}
        self._stage: dict = {}  # cache tensor index -> (device staging, pinned staging) of the batched store path
        self.stores = self.loads = self.evicted = 0
        self.release_block: Optional[Callable[[int], None]] = None

    @staticmethod
    def bytes_per_block(kv_caches: list[torch.Tensor], state_caches: Optional[list[torch.Tensor]] = None) -> int:
        """Host bytes one cached block takes: its KV pages of every layer plus one recurrent-state snapshot per state pool."""
        return sum(c[0].numel() * c.element_size() for c in list(kv_caches) + list(state_caches or []))

    def prefault(self, node: Optional[int] = None) -> Optional[float]:
        """Touch every page of the tier now (the first touch decides the NUMA node of a page, and a tier that faults its pages
        in under load stalls the stores) and report the fraction of it that sits on ``node`` (None: not asked / no answer).
        Upstream's sidecar waits until its tier is fully pinned and >= 95 % local before the replica serves
        (pear/rollout/lmcache.py:152-187)."""
        from ..utils.process import numa_locality

        local, total = 0.0, 0
        for t in self.kv_host + self.state_host:
            t.view(torch.uint8).reshape(-1)[::4096].zero_()
            if node is not None:
                nbytes = t.numel() * t.element_size()
                frac = numa_locality(t.data_ptr(), nbytes, node)
                if frac is not None:
                    local, total = local + frac * nbytes, total + nbytes
        return (local / total) if total else None

    # -- store --------------------------------------------------------------------------------------------------------
    def schedule_store(self, block_table: list[int], hashes: list[Optional[bytes]], state_slots: list[Optional[int]],
                       session: Optional[str] = None) -> list[tuple]:
        """Plan a store from the CURRENT block table. Null / unhashed blocks are skipped. Returns the work items and
        pins their device blocks until :meth:`run_store` finished them."""
        work = []
        for pos, (blk, h, st) in enumerate(zip(block_table, hashes, state_slots)):
            if blk == NULL_BLOCK or h is None or h in self.entries:
                continue
            self.pinned[blk] = self.pinned.get(blk, 0) + 1
            work.append((pos, blk, h, st))
        return [(session,) + w for w in work]

    def run_store(self, work: list[tuple]) -> int:
        if self.stream is not None and len(work) > 1:
            return self._run_store_batched(work)
        done = 0
        for session, pos, blk, h, st in work:
            try:
                if h in self.entries:
                    continue
                slot = self._host_slot()
                if slot is None:
                    continue
                self._copy_out(blk, st, slot)
                self.entries[h] = HostEntry(slot, st is not None, session=session, position=pos)
                if st is not None and session is not None:
                    self._demote_superseded(session, pos)
                self.stores += 1
                done += 1
            finally:
                self._unpin(blk)
        return done

    def _run_store_batched(self, work: list[tuple]) -> int:
        """GPU path of a store of several blocks: per cache tensor ONE gather kernel packs the blocks into a device staging
        buffer (``kv_blocks_copy_kernel``) and ONE copy moves it to pinned host memory, instead of one copy per block and
        tensor; the host then files the rows into their tier slots."""
        from ..ops import rollout_ops

        plan = []
        for session, pos, blk, h, st in work:
            if h in self.entries or any(p[3] == h for p in plan):
                self._unpin(blk)
                continue
            slot = self._host_slot()
            if slot is None:
                self._unpin(blk)
                continue
            plan.append((session, pos, blk, h, st, slot))
        if not plan:
            return 0
        n = len(plan)
        dev = self.kv_caches[0].device
        ids = torch.tensor([p[2] for p in plan], dtype=torch.int32, device=dev)
        self.stream.wait_stream(torch.cuda.current_stream())
        staged = []
        with torch.cuda.stream(self.stream):
            for ci, (cache, host) in enumerate(zip(self.kv_caches, self.kv_host)):
                shape = tuple(cache.shape[1:])
                if ci not in self._stage or self._stage[ci][0].shape[0] < n:  # persistent staging per cache tensor, grown on demand
                    cap = max(n, 64)
                    self._stage[ci] = (torch.empty((cap,) + shape, dtype=cache.dtype, device=dev),
                                       torch.empty((cap,) + shape, dtype=cache.dtype, pin_memory=True))
                sd, sh = self._stage[ci]
                rollout_ops.kv_blocks_copy(cache, sd, ids, to_staging=True)
                sh[:n].copy_(sd[:n], non_blocking=True)
                staged.append((host, sh))
            for i, (_, _, _, _, st, slot) in enumerate(plan):
                if st is not None:
                    for cache, host in zip(self.state_caches, self.state_host):
                        host[slot].copy_(cache[st], non_blocking=True)
        self.stream.synchronize()
        torch.cuda.current_stream().wait_stream(self.stream)  # the blocks may be reused right after
        for host, sh in staged:
            for i, p in enumerate(plan):
                host[p[5]].copy_(sh[i])
        for session, pos, blk, h, st, slot in plan:
            self.entries[h] = HostEntry(slot, st is not None, session=session, position=pos)
            if st is not None and session is not None:
                self._demote_superseded(session, pos)
            self.stores += 1
            self._unpin(blk)
        return n

    def offer(self, h: bytes, blk: int, state_slot: Optional[int]) -> None:
        """Eviction hook of the block manager: keep the block's contents on the host before it is reused."""
        work = self.schedule_store([blk], [h], [state_slot])
        self.run_store(work)

    def _unpin(self, blk: int) -> None:
        n = self.pinned.get(blk, 0) - 1
        if n <= 0:
            self.pinned.pop(blk, None)
        else:
            self.pinned[blk] = n

    def is_pinned(self, blk: int) -> bool:
        return self.pinned.get(blk, 0) > 0

    # -- LRU ----------------------------------------------------------------------------------------------------------
    def _host_slot(self) -> Optional[int]:
        used = self.capacity - len(self.free_slots)
        if used >= self.watermark * self.capacity or not self.free_slots:
            self._evict_round()
        return self.free_slots.pop() if self.free_slots else None

    def _evict_round(self) -> None:
        n = max(1, int(self.eviction_ratio * self.capacity))
        for _ in range(min(n, len(self.entries))):
            _, e = self.entries.popitem(last=False)
            self.free_slots.append(e.slot)
            self.evicted += 1

    def _demote_superseded(self, session: str, newest_pos: int) -> None:
        """State pages of earlier boundaries of the same session can no longer start a load: cold end, and sticky."""
        for h, e in list(self.entries.items()):
            if e.session == session and e.has_state and e.position < newest_pos and not e.demoted:
                e.demoted = True
                self.entries.move_to_end(h, last=False)

    def touch(self, h: bytes) -> None:
        e = self.entries.get(h)
        if e is not None and not e.demoted:
            self.entries.move_to_end(h, last=True)

    def end_session(self, session: str, usable_hashes: list[bytes]) -> None:
        """Only the keys a later turn can actually use are refreshed (patch 0002)."""
        for h in usable_hashes:
            self.touch(h)

    # -- load ---------------------------------------------------------------------------------------------------------
    def find(self, h: bytes) -> Optional[HostEntry]:
        return self.entries.get(h)

    def lookup(self, request_id: str, hashes: list[bytes]) -> int:
        """Number of leading blocks present on the host. A retry that now misses clears the earlier watermark."""
        n = 0
        for h in hashes:
            if h not in self.entries:
                break
            n += 1
        if n == 0:
            self.hit_watermark.pop(request_id, None)
        else:
            self.hit_watermark[request_id] = n
        return n

    def load(self, h: bytes, blk: int, state_slot: Optional[int]) -> None:
        e = self.entries[h]
        self._copy_in(e.slot, blk, state_slot if e.has_state else None)
        self.touch(h)
        self.loads += 1

    # -- copies -------------------------------------------------------------------------------------------------------
    def _copy_out(self, blk: int, state_slot: Optional[int], slot: int) -> None:
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                self._copy_out_impl(blk, state_slot, slot)
            torch.cuda.current_stream().wait_stream(self.stream)  # the block may be reused right after
        else:
            self._copy_out_impl(blk, state_slot, slot)

    def _copy_out_impl(self, blk, state_slot, slot) -> None:
        for dev, host in zip(self.kv_caches, self.kv_host):
            host[slot].copy_(dev[blk], non_blocking=True)
        if state_slot is not None:
            for dev, host in zip(self.state_caches, self.state_host):
                host[slot].copy_(dev[state_slot], non_blocking=True)

    def _copy_in(self, slot: int, blk: int, state_slot: Optional[int]) -> None:
        for dev, host in zip(self.kv_caches, self.kv_host):
            dev[blk].copy_(host[slot], non_blocking=True)
        if state_slot is not None:
            for dev, host in zip(self.state_caches, self.state_host):
                dev[state_slot].copy_(host[slot], non_blocking=True)

    def clear(self) -> None:
        for e in self.entries.values():
            self.free_slots.append(e.slot)
        self.entries.clear()
        self.hit_watermark.clear()

    def stats(self) -> dict:
        return {"host_blocks": len(self.entries), "host_stores": self.stores, "host_loads": self.loads, "host_evicted": self.evicted}

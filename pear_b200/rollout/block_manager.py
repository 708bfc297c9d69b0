"""Paged KV-cache block manager with hash-based prefix caching and block-aligned recurrent-state snapshots.

Cache semantics reproduced from the upstream rollout stack (vLLM block manager in ``mamba_cache_mode align`` with
``prefix_cache_retention_interval None``, ``pear/configs/base.yaml:77-80``): attention KV lives in fixed-size token
blocks; a full block is published in the prefix cache under the hash of (parent hash, its tokens, the policy version
salt); the Gated-DeltaNet state is only meaningful at block boundaries, so a snapshot slot can be attached to a block
and a cached prefix is only usable up to the LAST boundary that carries a snapshot; every finished turn's boundary keeps
its snapshot so a session's next turn resumes right after the previous answer. A weight sync invalidates everything
(``pear/rollout/lmcache.py:263-274``). Blocks are reference counted; unreferenced cached blocks sit in an LRU list and
are the eviction victims (optionally demoted to the host tier first).
"""

from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

NULL_BLOCK = 0  # never allocated: freed slots of a block table read as the null block


@dataclass
class Block:
    idx: int
    ref: int = 0
    hash: Optional[bytes] = None
    state_slot: Optional[int] = None  # snapshot of the recurrent state at the END of this block
    num_tokens: int = 0


def block_hash(parent: Optional[bytes], tokens, salt: bytes = b"", extra: bytes = b"") -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(parent or b"root")
    h.update(salt)
    h.update(extra)
    h.update(b",".join(str(int(t)).encode() for t in tokens))
    return h.digest()


@dataclass
class PrefixHit:
    blocks: list[int] = field(default_factory=list)  # cached blocks, in order
    tokens: int = 0  # tokens usable (up to the last boundary with a state snapshot)
    state_slot: Optional[int] = None
    host_blocks: int = 0  # of which were promoted from the host tier


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int = 16, num_state_slots: int = 0, enable_prefix_caching: bool = True,
                 needs_state: bool = True, host_tier=None):
        self.block_size = block_size
        self.blocks = [Block(i) for i in range(num_blocks)]
        self.free: list[int] = list(range(num_blocks - 1, 0, -1))  # block 0 is the null block
        self.cached: dict[bytes, int] = {}
        self.lru: "OrderedDict[int, None]" = OrderedDict()  # unreferenced cached blocks, oldest first
        self.free_slots: list[int] = list(range(num_state_slots - 1, -1, -1))
        self.slot_ref: dict[int, int] = {}
        self.enable_prefix_caching = enable_prefix_caching
        self.needs_state = needs_state
        self.host_tier = host_tier
        self.salt = b"v0"
        # metrics (the counters the monitor scrapes)
        self.queries = self.hits = self.host_hits = self.evictions = 0

    # -- capacity -----------------------------------------------------------------------------------------------------
    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.lru)

    def can_allocate(self, n: int) -> bool:
        return self.num_free >= n

    def _evict_one(self) -> int:
        idx, _ = self.lru.popitem(last=False)
        b = self.blocks[idx]
        if self.host_tier is not None and b.hash is not None:
            self.host_tier.offer(b.hash, idx, b.state_slot)
        self._unpublish(b)
        self.evictions += 1
        return idx

    def _unpublish(self, b: Block) -> None:
        if b.hash is not None and self.cached.get(b.hash) == b.idx:
            del self.cached[b.hash]
        b.hash = None
        if b.state_slot is not None:
            self.release_slot(b.state_slot)
            b.state_slot = None
        b.num_tokens = 0

    def allocate(self) -> int:
        if self.free:
            idx = self.free.pop()
        elif self.lru:
            idx = self._evict_one()
        else:
            raise MemoryError("out of KV blocks")
        b = self.blocks[idx]
        b.ref, b.hash, b.state_slot, b.num_tokens = 1, None, None, 0
        return idx

    def retain(self, idx: int) -> None:
        b = self.blocks[idx]
        if b.ref == 0:
            self.lru.pop(idx, None)
        b.ref += 1

    def release(self, idx: int) -> None:
        if idx == NULL_BLOCK:
            return
        b = self.blocks[idx]
        b.ref -= 1
        assert b.ref >= 0, f"block {idx} released too often"
        if b.ref == 0:
            if b.hash is not None and self.enable_prefix_caching:
                self.lru[idx] = None  # stays cached until evicted
            else:
                self._unpublish(b)
                self.free.append(idx)

    # -- recurrent-state snapshot slots ----------------------------------------------------------------------------------
    def allocate_slot(self) -> Optional[int]:
        if not self.free_slots:
            # steal the snapshot of the oldest unreferenced cached block
            for idx in self.lru:
                b = self.blocks[idx]
                if b.state_slot is not None and self.slot_ref.get(b.state_slot, 0) == 1:
                    slot = b.state_slot
                    b.state_slot = None
                    self.slot_ref.pop(slot, None)
                    self.slot_ref[slot] = 1
                    return slot
            return None
        slot = self.free_slots.pop()
        self.slot_ref[slot] = 1
        return slot

    def release_slot(self, slot: int) -> None:
        self.slot_ref[slot] = self.slot_ref.get(slot, 1) - 1
        if self.slot_ref[slot] <= 0:
            self.slot_ref.pop(slot, None)
            self.free_slots.append(slot)

    # -- prefix cache -------------------------------------------------------------------------------------------------
    def publish(self, idx: int, parent: Optional[bytes], tokens, state_slot: Optional[int] = None, extra: bytes = b"") -> bytes:
        """Register a FULL block under its content hash. ``state_slot``: snapshot of the recurrent state at its end
        (ownership moves to the block)."""
        h = block_hash(parent, tokens, self.salt, extra)
        b = self.blocks[idx]
        b.num_tokens = len(tokens)
        if not self.enable_prefix_caching:
            if state_slot is not None:
                self.release_slot(state_slot)
            return h
        if h in self.cached and self.cached[h] != idx:
            # an identical block exists already: keep ours private, but move a snapshot over if the cached one lacks it
            other = self.blocks[self.cached[h]]
            if state_slot is not None:
                if other.state_slot is None:
                    other.state_slot = state_slot
                else:
                    self.release_slot(state_slot)
            return h
        b.hash = h
        self.cached[h] = idx
        if state_slot is not None:
            if b.state_slot is not None:
                self.release_slot(b.state_slot)
            b.state_slot = state_slot
        return h

    def lookup(self, tokens, extra_fn=None, count: bool = True) -> PrefixHit:
        """Longest cached prefix of ``tokens`` (whole blocks). Retains the returned blocks. With a recurrent model the
        hit is cut back to the last block carrying a state snapshot."""
        hit = PrefixHit()
        if count:
            self.queries += len(tokens)
        if not self.enable_prefix_caching:
            return hit
        parent: Optional[bytes] = None
        chain: list[int] = []
        bs = self.block_size
        for i in range(len(tokens) // bs):
            extra = extra_fn(i) if extra_fn is not None else b""
            h = block_hash(parent, tokens[i * bs : (i + 1) * bs], self.salt, extra)
            idx = self.cached.get(h)
            if idx is None and self.host_tier is not None:
                idx = self._promote(h)
                if idx is not None:
                    hit.host_blocks += 1
            if idx is None:
                break
            # retained as soon as it is matched: a later promotion in this loop allocates device blocks and state slots, and
            # neither the LRU eviction nor the snapshot stealing of those may take a block that is already part of the chain
            self.retain(idx)
            chain.append(idx)
            parent = h
        usable = len(chain)
        if self.needs_state:
            while usable > 0 and self.blocks[chain[usable - 1]].state_slot is None:
                usable -= 1
        for idx in chain[usable:]:  # the tail past the last state snapshot is not used
            self.release(idx)
        hit.blocks = chain[:usable]
        hit.tokens = usable * bs
        hit.state_slot = self.blocks[chain[usable - 1]].state_slot if (usable and self.needs_state) else None
        if count:
            self.hits += hit.tokens
            self.host_hits += min(hit.host_blocks, usable) * bs
        return hit

    def _promote(self, h: bytes) -> Optional[int]:
        """Bring a block back from the host tier into a free device block (the tier copies the payload)."""
        if not self.can_allocate(1):
            return None
        entry = self.host_tier.find(h)
        if entry is None:
            return None
        idx = self.allocate()
        slot = self.allocate_slot() if entry.has_state else None
        # the allocation may have evicted a device block into the host tier, whose own eviction round may have dropped `h`
        if (entry.has_state and slot is None) or self.host_tier.find(h) is None:
            if slot is not None:
                self.release_slot(slot)
            self.release(idx)
            return None
        self.host_tier.load(h, idx, slot)
        b = self.blocks[idx]
        b.hash, b.state_slot, b.num_tokens = h, slot, self.block_size
        self.cached[h] = idx
        self.release(idx)  # cached, unreferenced until the caller retains it
        return idx

    def chain_hash(self, tokens, upto_blocks: int, extra_fn=None) -> Optional[bytes]:
        parent = None
        bs = self.block_size
        for i in range(upto_blocks):
            parent = block_hash(parent, tokens[i * bs : (i + 1) * bs], self.salt, extra_fn(i) if extra_fn else b"")
        return parent

    # -- invalidation -------------------------------------------------------------------------------------------------
    def reset_prefix_cache(self, new_salt: Optional[bytes] = None) -> int:
        """Drop every cached (unreferenced) block and change the salt so blocks still in use can never be matched by a
        request under the new weights. Returns the number of dropped blocks."""
        dropped = 0
        for idx in list(self.lru):
            self.lru.pop(idx)
            self._unpublish(self.blocks[idx])
            self.free.append(idx)
            dropped += 1
        for b in self.blocks:
            if b.hash is not None:
                self.cached.pop(b.hash, None)
                b.hash = None
        if new_salt is not None:
            self.salt = new_salt
        if self.host_tier is not None:
            self.host_tier.clear()
        return dropped

    def stats(self) -> dict:
        return {"prefix_cache_queries": self.queries, "prefix_cache_hits": self.hits, "external_prefix_cache_hits": self.host_hits,
                "evictions": self.evictions, "free_blocks": self.num_free, "cached_blocks": len(self.cached)}

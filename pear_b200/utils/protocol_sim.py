"""CPU simulator of the peer-memory flag protocols, with a happens-before race detector.

The NVSwitch kernels (``ops/csrc/comm_kernels.cu``, ``decode_step.cu``, ``gemm_collective.cu``) synchronise ranks with epoch
flags: a rank publishes "my slot reached epoch e" to every peer with a release store and a waiter polls ITS OWN copy with
acquire loads until the epoch is reached. Whether a buffer may be reused is an argument about which release is ordered before
which acquire, and such arguments are easy to get wrong (a buffer pushed into by peers and read by a later kernel, with
nothing ordering the peer's NEXT push after that read, was one). This module states each protocol as a small per-rank program
over four operations and checks it mechanically:

* ``write(buffer, tag)`` / ``read(buffer, expect)``: plain stores / loads of a (whole) buffer in some rank's memory;
* ``signal(dst, slot, epoch)``: release store of ``epoch`` into ``dst``'s copy of this rank's flag of ``slot``;
* ``wait(slot, src, epoch)``: acquire-poll of this rank's copy of ``src``'s flag until it is ``>= epoch``.

Every rank carries a vector clock; a signal stores the sender's clock beside the epoch and the wait that observes it joins
that clock (release / acquire). A read must be ordered after the last write of its buffer and must find the tag the protocol
expects; a write must be ordered after every read of the previous contents and after the previous write. An unordered pair is
reported as a race whatever order the scheduler happened to run it in, so a few random schedules per protocol are enough;
a schedule in which every rank waits is reported as a deadlock (on the device: the bounded wait's timeout status).

Upstream has no such tool (its only race check is a static launch-argument test, tests/test_kernel_launch_checks_on_cpu.py);
the protocols modelled here are this build's own.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Callable, Generator, Iterable, Optional


class ProtocolError(AssertionError):
    pass


@dataclass
class _Cell:
    write: Optional[tuple[int, tuple, object]] = None  # (rank, clock, tag)
    reads: list[tuple[int, tuple]] = field(default_factory=list)


def _before(a: tuple, b: tuple) -> bool:
    return all(x <= y for x, y in zip(a, b))


class Sim:
    def __init__(self, world: int, seed: int = 0):
        self.world, self.rng = world, random.Random(seed)
        self.clock = [[0] * world for _ in range(world)]
        self.flags: dict[tuple[int, int, int], tuple[int, tuple]] = {}  # (owner, slot, src) -> (epoch, clock of the release)
        self.cells: dict[object, _Cell] = {}
        self.trace: list[tuple] = []

    # -- operations (executed by `run` on behalf of a rank) -----------------------------------------------------------
    def _tick(self, r: int) -> tuple:
        self.clock[r][r] += 1
        return tuple(self.clock[r])

    def _write(self, r: int, buf, tag) -> None:
        now = self._tick(r)
        c = self.cells.setdefault(buf, _Cell())
        for rr, rc in c.reads:
            if rr != r and not _before(rc, now):
                raise ProtocolError(f"rank {r} overwrites {buf!r} (tag {tag!r}) while rank {rr}'s read of {c.write and c.write[2]!r} is not ordered before it")
        if c.write is not None and c.write[0] != r and not _before(c.write[1], now):
            raise ProtocolError(f"rank {r} and rank {c.write[0]} write {buf!r} without an order between them")
        c.write, c.reads = (r, now, tag), []

    def _read(self, r: int, buf, expect) -> None:
        now = self._tick(r)
        c = self.cells.setdefault(buf, _Cell())
        if c.write is None:
            raise ProtocolError(f"rank {r} reads {buf!r} before anything wrote it (expected {expect!r})")
        if c.write[0] != r and not _before(c.write[1], now):
            raise ProtocolError(f"rank {r} reads {buf!r} while rank {c.write[0]}'s write of {c.write[2]!r} is not ordered before it (expected {expect!r})")
        if c.write[2] != expect:
            raise ProtocolError(f"rank {r} reads {c.write[2]!r} from {buf!r}, expected {expect!r}")
        c.reads.append((r, now))

    def _signal(self, r: int, dst: int, slot: int, epoch: int) -> None:
        now = self._tick(r)
        old = self.flags.get((dst, slot, r))
        if old is not None and old[0] > epoch:
            raise ProtocolError(f"rank {r} moves its flag of slot {slot} at rank {dst} backwards ({old[0]} -> {epoch})")
        self.flags[(dst, slot, r)] = (epoch, now)

    def _ready(self, r: int, slot: int, src: int, epoch: int) -> bool:
        f = self.flags.get((r, slot, src))
        return f is not None and f[0] >= epoch

    def _acquire(self, r: int, slot: int, src: int) -> None:
        _, fc = self.flags[(r, slot, src)]
        self.clock[r] = [max(a, b) for a, b in zip(self.clock[r], fc)]
        self._tick(r)

    # -- scheduler ----------------------------------------------------------------------------------------------------
    def run(self, programs: list[Generator]) -> None:
        """``programs[r]`` yields rank r's operations: ("write", buf, tag), ("read", buf, expect), ("signal", dst, slot, epoch),
        ("wait", slot, src, epoch). Ranks advance one operation at a time in a random order."""
        pending: list[Optional[tuple]] = [None] * self.world
        live = set(range(self.world))
        for r in list(live):
            pending[r] = next(programs[r], None)
            if pending[r] is None:
                live.discard(r)
        while live:
            runnable = [r for r in live if pending[r][0] != "wait" or self._ready(r, *pending[r][1:])]
            if not runnable:
                raise ProtocolError("deadlock: " + "; ".join(f"rank {r} waits for slot {pending[r][1]} of rank {pending[r][2]} to reach {pending[r][3]}"
                                                             for r in sorted(live)))
            r = self.rng.choice(runnable)
            op = pending[r]
            self.trace.append((r,) + op)
            if op[0] == "write":
                self._write(r, op[1], op[2])
            elif op[0] == "read":
                self._read(r, op[1], op[2])
            elif op[0] == "signal":
                self._signal(r, op[1], op[2], op[3])
            elif op[0] == "wait":
                self._acquire(r, op[1], op[2])
            else:
                raise ValueError(op)
            pending[r] = next(programs[r], None)
            if pending[r] is None:
                live.discard(r)


def check(protocol: Callable[..., Generator], world: int, schedules: int = 50, seed: int = 0, **kw) -> None:
    """Run ``protocol(rank, world, **kw)`` on every rank under ``schedules`` random interleavings; raises ProtocolError."""
    for s in range(schedules):
        Sim(world, seed * 100003 + s).run([protocol(r, world, **kw) for r in range(world)])


# -- shared pieces ------------------------------------------------------------------------------------------------------------
def _signal_all(rank: int, world: int, slot: int, epoch: int) -> Iterable[tuple]:
    for p in range(world):
        yield ("signal", (rank + p) % world, slot, epoch)


def _wait_all(world: int, slot: int, epoch: int) -> Iterable[tuple]:
    for p in range(world):
        yield ("wait", slot, p, epoch)


def device_barrier(rank: int, world: int, slot: int, epoch: int) -> Iterable[tuple]:
    """``SymmWorld.device_barrier``: signal kernel, then wait kernel, on the rank's stream."""
    yield from _signal_all(rank, world, slot, epoch)
    yield from _wait_all(world, slot, epoch)


# -- the protocols ------------------------------------------------------------------------------------------------------------
def one_shot_all_reduce(rank: int, world: int, rounds: int = 6, buffers: int = 2):
    """``ar_add_rmsnorm_kernel`` / the one-shot form of the decode step: the rank's partial rows go into buffer
    ``epoch % buffers`` of its own workspace (stream order, before the kernel); the kernel signals the epoch, waits for every
    rank's signal and reads every rank's buffer. The kernels use two buffers; one is the broken form."""
    for e in range(1, rounds + 1):
        b = e % buffers
        yield ("write", ("partial", rank, b), e)
        yield from _signal_all(rank, world, 0, e)
        yield from _wait_all(world, 0, e)
        for p in range(world):
            yield ("read", ("partial", (rank + p) % world, b), e)


def two_shot_all_reduce(rank: int, world: int, rounds: int = 6, second_flag: bool = True, fixed_buffer: bool = True):
    """``ds_ar2_add_rmsnorm_kernel``: the producing GEMM writes the partial rows into a FIXED buffer of the rank's workspace;
    flag exchange 1; the owner of a row sums all ranks' partials and stores the result row into EVERY rank's ``out``; flag
    exchange 2 (the kernel ends only when every rank's rows have landed); the rank's next kernels read its ``out``.
    Without the second exchange neither the fixed partial buffer nor ``out`` is safe."""
    for e in range(1, rounds + 1):
        b = 0 if fixed_buffer else e % 2
        yield ("write", ("partial", rank, b), e)  # the GEMM before the reduction, same stream
        yield from _signal_all(rank, world, 0, e)
        yield from _wait_all(world, 0, e)
        for p in range(world):
            yield ("read", ("partial", (rank + p) % world, b), e)  # this rank's rows of every rank's partial
        for p in range(world):
            yield ("write", ("out", (rank + p) % world, "rows of", rank), e)  # its normalised rows into every rank's out
        if second_flag:
            yield from _signal_all(rank, world, 1, e)
            yield from _wait_all(world, 1, e)
        for owner in range(world):
            yield ("read", ("out", rank, "rows of", owner), e)  # the consumer kernels of this rank


def all_gather_push(rank: int, world: int, rounds: int = 6, leading_barrier: bool = True):
    """``SymmWorld.all_gather_logits`` / ``sharded_argmax``: every rank stores its shard into the ``full`` buffer of EVERY
    rank, signals, waits, and a later kernel of the rank (the sampler) reads its ``full``. One buffer, reused by every call:
    the call must start with a barrier, or a faster rank's next push lands while a slower rank still reads the last result."""
    sync_epoch = 0
    for e in range(1, rounds + 1):
        if leading_barrier:
            sync_epoch += 1
            yield from device_barrier(rank, world, 7, sync_epoch)
        for p in range(world):
            yield ("write", ("full", (rank + p) % world, "shard of", rank), e)
        yield from _signal_all(rank, world, 2, e)
        yield from _wait_all(world, 2, e)
        for src in range(world):
            yield ("read", ("full", rank, "shard of", src), e)


def staged_weight_pull(rank: int, world: int, buckets: int = 5, trailing_barrier: bool = True, src: int = 0):
    """``SymmTransport``: the sender copies a bucket into its staging buffer; barrier; every receiver pulls its blocks out of
    the sender's buffer; a second barrier hands the buffer back before the next bucket is staged."""
    e = 0
    for b in range(1, buckets + 1):
        if rank == src:
            yield ("write", ("staging", src), b)
        e += 1
        yield from device_barrier(rank, world, 3, e)
        if rank != src:
            yield ("read", ("staging", src), b)
        if trailing_barrier:
            e += 1
            yield from device_barrier(rank, world, 3, e)


def reduce_scatter_tiles(rank: int, world: int, rounds: int = 4, tiles_per_rank: int = 2, leading_barrier: bool = True):
    """GEMM -> reduce-scatter (``gemm_collective.cu`` MODE 1): a rank computes every output tile; a tile owned by a peer is
    pushed as a partial into the owner's staging slot for (tile, source rank) and a per-(tile, source) flag is released; the owner
    waits for the flags of its tile, adds the staged partials to its own and stores the tile. The staging slots are reused by
    the next call, which therefore starts with a barrier."""
    sync = 0
    for e in range(1, rounds + 1):
        if leading_barrier:
            sync += 1
            yield from device_barrier(rank, world, 7, sync)
        for owner in range(world):
            for t in range(tiles_per_rank):
                if owner != rank:
                    yield ("write", ("stage", owner, t, "from", rank), e)
                    yield ("signal", owner, 10 + t, e)
        for t in range(tiles_per_rank):
            for srcr in range(world):
                if srcr != rank:
                    yield ("wait", 10 + t, srcr, e)
                    yield ("read", ("stage", rank, t, "from", srcr), e)
            yield ("write", ("c", rank, t), e)


def record_exchange(rank: int, world: int, steps: int = 5, kinds: int = 1, buffers: int = 2):
    """The sampler's exchanges of the batched decode step (rejection-sampler records, top log-prob lists, the drafter's argmax
    keys): every rank pushes its records into buffer ``(counter + 1) % buffers`` of EVERY rank; one barrier that advances the
    device counter; a finish kernel of each rank reads buffer ``counter % buffers`` of its own memory. ``kinds`` exchanges with
    buffers of their own share the one counter per step (with an even number of them a kind meets the same buffer every step,
    ordered by the other kinds' barriers in between)."""
    ctr = 0
    for _ in range(steps):
        for k in range(kinds):
            b = (ctr + 1) % buffers
            for p in range(world):
                yield ("write", ("recs", k, (rank + p) % world, b, "from", rank), ctr + 1)
            ctr += 1
            yield from device_barrier(rank, world, 4, ctr)
            for srcr in range(world):
                yield ("read", ("recs", k, rank, ctr % buffers, "from", srcr), ctr)


def fused_optimizer_step(rank: int, world: int, steps: int = 4, final_barrier: bool = True):
    """``FusedShardedAdamW.step``: every rank's backward leaves its full gradient in its own bucket; barrier; a rank reduces ITS
    shard range out of every rank's bucket and stores its partial squared norm into every rank's norm table; barrier; it clips by
    the global norm, updates its shard and stores the new parameters into every rank's parameter bucket; barrier; the next
    forward reads the rank's own parameter bucket. Without the last barrier a rank may read shards that have not landed."""
    e = 0
    for s in range(1, steps + 1):
        if s > 1:
            for owner in range(world):
                yield ("read", ("params", rank, "shard of", owner), s - 1)  # forward / backward of this step
        yield ("write", ("grads", rank), s)
        e += 1
        yield from device_barrier(rank, world, 5, e)
        for p in range(world):
            yield ("read", ("grads", (rank + p) % world), s)
        for p in range(world):
            yield ("write", ("norms", (rank + p) % world, "of", rank), s)
        e += 1
        yield from device_barrier(rank, world, 5, e)
        for srcr in range(world):
            yield ("read", ("norms", rank, "of", srcr), s)
        for p in range(world):
            yield ("write", ("params", (rank + p) % world, "shard of", rank), s)
        if final_barrier:
            e += 1
            yield from device_barrier(rank, world, 5, e)


PROTOCOLS: dict[str, tuple[Callable[..., Generator], dict, dict]] = {
    # name: (program, arguments of the form the kernels use, arguments of a form that must be reported)
    "one_shot_all_reduce": (one_shot_all_reduce, {"buffers": 2}, {"buffers": 1}),
    "two_shot_all_reduce": (two_shot_all_reduce, {"second_flag": True, "fixed_buffer": True}, {"second_flag": False, "fixed_buffer": True}),
    "all_gather_push": (all_gather_push, {"leading_barrier": True}, {"leading_barrier": False}),
    "staged_weight_pull": (staged_weight_pull, {"trailing_barrier": True}, {"trailing_barrier": False}),
    "reduce_scatter_tiles": (reduce_scatter_tiles, {"leading_barrier": True}, {"leading_barrier": False}),
    "record_exchange": (record_exchange, {"kinds": 1, "buffers": 2}, {"kinds": 1, "buffers": 1}),
    "fused_optimizer_step": (fused_optimizer_step, {"final_barrier": True}, {"final_barrier": False}),
    "record_exchange x4": (record_exchange, {"kinds": 4, "buffers": 2}, {"kinds": 1, "buffers": 1}),
}


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="check the peer-memory flag protocols under random schedules")
    ap.add_argument("--world", type=int, nargs="+", default=[2, 4, 8])
    ap.add_argument("--schedules", type=int, default=200)
    args = ap.parse_args(argv)
    bad = 0
    for name, (prog, good, broken) in PROTOCOLS.items():
        for w in args.world:
            try:
                check(prog, w, args.schedules, **good)
                verdict = "ok"
            except ProtocolError as e:
                verdict, bad = f"FAILED: {e}", bad + 1
            try:
                check(prog, w, args.schedules, **broken)
                control = "NOT reported"
                bad += 1
            except ProtocolError:
                control = "reported"
            print(f"{name:24s} world {w}: {verdict}; broken form {broken}: {control}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())

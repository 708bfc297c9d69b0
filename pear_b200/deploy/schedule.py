"""Host-side instruction scheduler of the decode megakernel.

Builds, for one model and one SM count, the descriptor table and the per-CTA instruction lists the persistent kernel
walks (``pear_b200/ops/csrc/megakernel.cuh``). The counterpart of upstream
``pear/models/qwen3_5/deploy/blackwell/nvfp4/schedule.py`` (stream-K split of every GEMV over SMs, binary layouts
packed on the host) re-derived for 148 SMs: every GEMV's (row tile, k-stage) space is cut into contiguous, equal
per-CTA ranges whose start rotates from op to op so the remainders spread; ops are separated by grid barriers and the
weight producer warp streams through them.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

# opcodes / enums (megakernel.cuh)
OP_END, OP_GEMV, OP_BARRIER, OP_EMBED, OP_ZERO, OP_GDN, OP_ATTN, OP_ATTN_COMBINE = range(8)
OP_SAMPLE_PART, OP_SAMPLE_FIN, OP_DRAFT_IN, OP_ARGMAX_PART, OP_ARGMAX_FIN, OP_COPY, OP_QUANT = range(8, 15)
PRO_PLAIN, PRO_NORM, PRO_SWIGLU, PRO_GDN_NORM = range(4)
EPI_RED, EPI_STORE = range(2)
F_IN_PARITY, F_OUT_PARITY, F_OUT_OTHER_PARITY, F_DRAFT_ROWS = 1, 2, 4, 8

TILE_ROWS, STAGE_K, STAGE_BYTES, MAX_SEG_STAGES = 128, 256, 18432, 20

INSTR_DTYPE = np.dtype([(n, "<i4") for n in ("op", "desc", "a", "b", "c", "d", "e", "f")])
DESC_DTYPE = np.dtype(
    [(f"p{i}", "<u8") for i in range(8)] + [(f"i{i}", "<i4") for i in range(10)] + [(f"f{i}", "<f4") for i in range(4)]
    + [("pad", "<i4", (2,))]
)
assert INSTR_DTYPE.itemsize == 32 and DESC_DTYPE.itemsize == 128

STEPREC_INTS = 24  # T pos0 n_replay parity step mode n_out_total rows_draft tokens[8] n_acc aux[7]
STEPOUT_DTYPE = np.dtype([("step", "<i4"), ("n_out", "<i4"), ("n_accept", "<i4"), ("pos0", "<i4"),
                          ("tokens", "<i4", (8,)), ("logprobs", "<f4", (4,))])


@dataclass
class Program:
    """Descriptor table + per-CTA instruction lists under construction."""

    num_ctas: int
    lists: list[list[tuple]] = field(default_factory=list)
    descs: list[dict] = field(default_factory=list)
    rotate: int = 0
    gemv_stages: int = 0  # total weight stages streamed per launch (bytes = stages * STAGE_BYTES)
    expect: list[int] = field(default_factory=list)  # contributions per tile counter of the linked GEMVs

    def __post_init__(self) -> None:
        self.lists = [[] for _ in range(self.num_ctas)]

    # -- descriptors -------------------------------------------------------------------------------------------------
    def desc(self, **fields) -> int:
        self.descs.append(fields)
        return len(self.descs) - 1

    # -- instructions ------------------------------------------------------------------------------------------------
    def emit(self, cta: int, op: int, desc: int = 0, a: int = 0, b: int = 0, c: int = 0, d: int = 0) -> None:
        self.lists[cta].append((op, desc, a, b, c, d, 0, 0))

    def barrier(self) -> None:
        for cta in range(self.num_ctas):
            self.emit(cta, OP_BARRIER)

    def _next_rotation(self, items: int) -> int:
        r = self.rotate
        self.rotate = (self.rotate + items) % self.num_ctas
        return r

    def spread(self, op: int, desc: int, items: list[tuple]) -> None:
        """One instruction per item, dealt round-robin over the CTAs starting after the previous op's last CTA."""
        r = self._next_rotation(len(items))
        for i, it in enumerate(items):
            self.emit((r + i) % self.num_ctas, op, desc, *it)

    def ranged(self, op: int, desc: int, total: int, granule: int = 1) -> None:
        """Cut [0, total) into near-equal contiguous per-CTA ranges (multiples of ``granule``): instr a=start b=count."""
        units = (total + granule - 1) // granule
        n = min(self.num_ctas, units)
        r = self._next_rotation(n)
        for i in range(n):
            lo, hi = units * i // n, units * (i + 1) // n
            if hi > lo:
                self.emit((r + i) % self.num_ctas, op, desc, lo * granule, min(total, hi * granule) - lo * granule)

    def quant(self, desc: int, k: int) -> None:
        """Phase that builds the activation operand of GEMV ``desc``: one unit per 128 K elements, dealt over the CTAs."""
        self.spread(OP_QUANT, desc, [(u, 1) for u in range(k // 128)])

    def gemv(self, desc: int, rows: int, k: int, aligned: bool = False) -> None:
        """Stream-K split of a [rows x k] GEMV. ``aligned``: cuts only at tile boundaries (plain-store epilogues)."""
        tiles, ks = (rows + TILE_ROWS - 1) // TILE_ROWS, k // STAGE_K
        total = tiles * ks
        self.gemv_stages += total
        n = self.num_ctas
        r = self._next_rotation(total % n if not aligned else tiles % n)
        for i in range(n):
            cta = (r + i) % n
            if aligned:
                lo, hi = (tiles * i // n) * ks, (tiles * (i + 1) // n) * ks
            else:
                lo, hi = total * i // n, total * (i + 1) // n
            prev = None
            pos = lo
            whole = ks <= MAX_SEG_STAGES  # the whole activation row fits in shared memory: built once per CTA and op
            while pos < hi:
                tile, ks0 = divmod(pos, ks)
                cnt = min(ks - ks0, hi - pos, MAX_SEG_STAGES)
                if whole:
                    flags = 2 | (1 if pos == lo else 0)
                else:
                    flags = 0 if prev == (ks0, cnt) else 1
                self.emit(cta, OP_GEMV, desc, tile, ks0, cnt, flags)
                prev = (ks0, cnt)
                pos += cnt

    # -- finalisation ------------------------------------------------------------------------------------------------
    def finalize(self) -> tuple[np.ndarray, np.ndarray, int]:
        max_len = max(len(l) for l in self.lists) + 1
        instrs = np.zeros((self.num_ctas, max_len), dtype=INSTR_DTYPE)
        for c, l in enumerate(self.lists):
            for i, ins in enumerate(l):
                instrs[c, i] = ins
        descs = np.zeros(len(self.descs), dtype=DESC_DTYPE)
        for i, f in enumerate(self.descs):
            for k, v in f.items():
                descs[i][k] = v
        nbar = {sum(1 for ins in l if ins[0] == OP_BARRIER) for l in self.lists}
        assert len(nbar) == 1, "every CTA must pass the same number of grid barriers"
        return instrs, descs, max_len

    def stats(self) -> dict:
        per_cta = [sum(ins[4] for ins in l if ins[0] == OP_GEMV) for l in self.lists]
        return {
            "weight_bytes": self.gemv_stages * STAGE_BYTES,
            "stages_per_cta_min": min(per_cta), "stages_per_cta_max": max(per_cta),
            "barriers": sum(1 for ins in self.lists[0] if ins[0] == OP_BARRIER),
            "instrs_max": max(len(l) for l in self.lists),
        }

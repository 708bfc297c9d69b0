"""NVFP4: e2m1 codes in blocks of 16 with an e4m3 block scale and a power-of-two tensor scale.

Format as the upstream deploy path reads it (``pear/models/qwen3_5/deploy/blackwell/nvfp4/draft/quant.py:23-42``):
block scale = ``amax / 6 * global_scale`` clamped to 448 and rounded to e4m3, codes round to the nearest e2m1 value
(ties to the even code, saturating at 6), two codes per byte with the even index in the low nibble.
``dequant = code * block_scale / global_scale``.

:func:`pack_stages` lays a quantised matrix out in the decode megakernel's streaming order
(``pear_b200/ops/csrc/decode_megakernel.cu``: 18 KB stages of 128 rows x 256 K in mma-fragment order).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
BLOCK = 16
TILE_ROWS = 128
STAGE_K = 256
STAGE_CODE_BYTES = TILE_ROWS * STAGE_K // 2
STAGE_SCALE_BYTES = TILE_ROWS * STAGE_K // BLOCK
STAGE_BYTES = STAGE_CODE_BYTES + STAGE_SCALE_BYTES


@dataclass
class NVFP4Tensor:
    codes: torch.Tensor  # uint8 [N, K/2]
    scales: torch.Tensor  # uint8 view of e4m3 [N, K/16]
    global_scale: float  # power of two
    shape: tuple[int, int]

    def dequantize(self) -> torch.Tensor:
        return dequantize(self.codes, self.scales, self.global_scale)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()


def _e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code (0..7 magnitude | sign << 3) of ``x``; ties go to the even code; saturates at 6."""
    a = x.abs()
    # decision thresholds between consecutive magnitudes; a tie goes to the code with an even index
    code = torch.zeros_like(a, dtype=torch.uint8)
    bounds = [(0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False), (3.5, True), (5.0, False)]
    for i, (b, up_on_tie) in enumerate(bounds):
        code = torch.where((a >= b) if up_on_tie else (a > b), torch.full_like(code, i + 1), code)
    sign = (x < 0) & (code > 0)
    return code | (sign.to(torch.uint8) << 3)


def _e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    table = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=code.device)
    mag = table[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def choose_global_scale(amax: float) -> float:
    """Largest power of two keeping every block scale within e4m3's 448."""
    if amax <= 0.0 or not math.isfinite(amax):
        return 1.0
    return 2.0 ** math.floor(math.log2(448.0 * 6.0 / amax))


def quantize(w: torch.Tensor, global_scale: float | None = None) -> NVFP4Tensor:
    """Quantise ``w`` [N, K] (K a multiple of 16) to NVFP4."""
    n, k = w.shape
    if k % BLOCK:
        raise ValueError(f"K={k} is not a multiple of {BLOCK}")
    wf = w.float()
    blocks = wf.view(n, k // BLOCK, BLOCK)
    amax = blocks.abs().amax(-1)
    gs = global_scale if global_scale is not None else choose_global_scale(float(amax.max()))
    scale = (amax / 6.0 * gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    sf = scale.float()
    inv = torch.where(sf > 0, gs / sf, torch.zeros_like(sf))
    codes = _e2m1_encode(blocks * inv[..., None]).view(n, k)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return NVFP4Tensor(packed.contiguous(), scale.view(torch.uint8).contiguous(), gs, (n, k))


def dequantize(codes: torch.Tensor, scales: torch.Tensor, global_scale: float) -> torch.Tensor:
    n, half = codes.shape
    k = half * 2
    lo, hi = _e2m1_decode(codes & 0xF), _e2m1_decode(codes >> 4)
    vals = torch.stack([lo, hi], dim=-1).view(n, k)
    sf = scales.view(torch.float8_e4m3fn).float() / global_scale
    return (vals.view(n, k // BLOCK, BLOCK) * sf[..., None]).view(n, k)


def pack_stages(q: NVFP4Tensor) -> torch.Tensor:
    """Megakernel streaming layout: uint8 [tiles, kstages, STAGE_BYTES]; rows are zero-padded to a multiple of 128.

    A stage is the shared-memory image the tensor core reads in place. Codes: the K-major operand without swizzle, i.e.
    8-row x 16-byte core matrices, ``(chunk * 16 + row // 8) * 128 + (row % 8) * 16 + byte`` with ``chunk`` the 16-byte
    (32-element) K chunk 0..7. Scales: four 512-byte atoms, one per 64 K elements,
    ``16384 + j * 512 + (row % 32) * 16 + (row // 32) * 4 + block`` (the layout ``tcgen05.cp.32x128b.warpx4`` spreads
    over tensor memory for a 128-row block-scaled MMA).
    """
    n, k = q.shape
    if k % STAGE_K:
        raise ValueError(f"K={k} is not a multiple of {STAGE_K}")
    tiles, ks = (n + TILE_ROWS - 1) // TILE_ROWS, k // STAGE_K
    codes, scales = q.codes, q.scales
    if tiles * TILE_ROWS != n:
        pad = tiles * TILE_ROWS - n
        codes = torch.cat([codes, codes.new_zeros(pad, codes.shape[1])])
        scales = torch.cat([scales, scales.new_zeros(pad, scales.shape[1])])
    # rows -> (tile, row // 8, row % 8); code bytes -> (kstage, chunk, byte)
    c = codes.view(tiles, 16, 8, ks, 8, 16)
    #            0      1   2  3   4  5    -> (tile, ks, chunk, row // 8, row % 8, byte)
    c = c.permute(0, 3, 4, 1, 2, 5).reshape(tiles, ks, STAGE_CODE_BYTES)
    # rows -> (tile, row // 32, row % 32); scales -> (kstage, j, block)
    s = scales.view(tiles, 4, 32, ks, 4, 4)
    #             0     1  2   3   4  5    -> (tile, ks, j, row % 32, row // 32, block)
    s = s.permute(0, 3, 4, 2, 1, 5).reshape(tiles, ks, STAGE_SCALE_BYTES)
    return torch.cat([c, s], dim=-1).contiguous()


def unpack_stages(packed: torch.Tensor, n: int, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_stages` (tests)."""
    tiles, ks = packed.shape[0], packed.shape[1]
    c = packed[..., :STAGE_CODE_BYTES].reshape(tiles, ks, 8, 16, 8, 16)
    #   (tile, ks, chunk, row // 8, row % 8, byte) -> (tile, row // 8, row % 8, ks, chunk, byte)
    c = c.permute(0, 3, 4, 1, 2, 5).reshape(tiles * TILE_ROWS, k // 2)
    s = packed[..., STAGE_CODE_BYTES:].reshape(tiles, ks, 4, 32, 4, 4)
    #   (tile, ks, j, row % 32, row // 32, block) -> (tile, row // 32, row % 32, ks, j, block)
    s = s.permute(0, 4, 3, 1, 2, 5).reshape(tiles * TILE_ROWS, k // BLOCK)
    return c[:n].contiguous(), s[:n].contiguous()


def quantize_packed(w: torch.Tensor) -> tuple[torch.Tensor, float]:
    q = quantize(w)
    return pack_stages(q), q.global_scale

"""NVFP4 quantisation and the megakernel's stage layout, checked on CPU by emulating the kernel's fragment indexing."""

import numpy as np
import torch

from pear_b200.models import nvfp4


def test_quantize_roundtrip_error():
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    q = nvfp4.quantize(w)
    d = q.dequantize()
    # 4-bit blocks of 16 with e4m3 scales: relative error of a gaussian block stays below ~20 %
    assert (d - w).norm() / w.norm() < 0.2
    assert q.codes.shape == (64, 128) and q.scales.shape == (64, 16)
    # requantising an exactly representable matrix is the identity
    q2 = nvfp4.quantize(d, q.global_scale)
    assert torch.equal(q2.codes, q.codes) and torch.equal(q2.scales, q.scales)


def test_ties_round_to_even_code():
    x = torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, 7.0, 0.0, 0.1, 0.3, 2.4, 2.6]])
    codes = nvfp4._e2m1_encode(x)
    vals = nvfp4._e2m1_decode(codes)
    assert vals.tolist() == [[0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, 0.0, -1.0, 6.0, 0.0, 0.0, 0.5, 2.0, 3.0]]


def test_pack_unpack_roundtrip():
    torch.manual_seed(1)
    w = torch.randn(200, 512)
    q = nvfp4.quantize(w)
    packed = nvfp4.pack_stages(q)
    assert packed.shape == (2, 2, nvfp4.STAGE_BYTES)
    c, s = nvfp4.unpack_stages(packed, 200, 512)
    assert torch.equal(c, q.codes) and torch.equal(s, q.scales)


def test_stage_layout_matches_tensor_core_operand_addressing():
    """Emulates what the block-scaled MMA of decode_megakernel.cu reads: for the j-th K-64 step of a stage, element
    (row, k) sits at ``j*4096 + (k // 32) * LBO(2048) + (row // 8) * SBO(128) + (row % 8) * 16 + (k % 32) // 2`` (low
    nibble = even k), and its scale at ``16384 + j*512 + (row % 32) * 16 + (row // 32) * 4 + (k // 16)``."""
    torch.manual_seed(2)
    n, k = 128, 256
    w = torch.randn(n, k)
    q = nvfp4.quantize(w)
    stage = nvfp4.pack_stages(q)[0, 0].numpy()
    deq = q.dequantize().numpy() * q.global_scale  # code * e4m3 scale
    x = np.random.RandomState(0).randn(k).astype(np.float32)
    table = np.array(nvfp4.E2M1_VALUES, dtype=np.float32)

    def dec(nib):
        v = table[nib & 7]
        return -v if nib & 8 else v

    e4m3 = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    out = np.zeros(n, dtype=np.float64)
    for j in range(4):
        for row in range(n):
            for kk in range(64):
                byte = int(stage[j * 4096 + (kk // 32) * 2048 + (row // 8) * 128 + (row % 8) * 16 + (kk % 32) // 2])
                nib = (byte >> 4) if (kk & 1) else (byte & 15)
                sc = e4m3[stage[nvfp4.STAGE_CODE_BYTES + j * 512 + (row % 32) * 16 + (row // 32) * 4 + kk // 16]]
                out[row] += sc * dec(nib) * x[j * 64 + kk]
    ref = deq.astype(np.float64) @ x
    assert np.allclose(out, ref, rtol=1e-5, atol=1e-5)

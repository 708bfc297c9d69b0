"""tcgen05 variable-length attention forward against the fp32 PyTorch statement of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens_q, lens_k, hq=6, hkv=2, causal=True, fused=False, seed=0):
    from pear_b200.ops import attention as A

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=dev)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=dev)
    tq, tk = sum(lens_q), sum(lens_k)
    if fused:  # q, k, v as column slices of one projection output (row stride != heads * 256)
        assert tq == tk
        buf = torch.randn(tq, (hq + 2 * hkv) * 256, device=dev, generator=g).to(torch.bfloat16)
        q = buf[:, : hq * 256].unflatten(1, (hq, 256))
        k = buf[:, hq * 256 : (hq + hkv) * 256].unflatten(1, (hkv, 256))
        v = buf[:, (hq + hkv) * 256 :].unflatten(1, (hkv, 256))
    else:
        q = torch.randn(tq, hq, 256, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(tk, hkv, 256, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(tk, hkv, 256, device=dev, generator=g).to(torch.bfloat16)
    o, lse = A.attention_varlen_fwd(q, k, v, cu_q, cu_k, causal=causal)
    torch.cuda.synchronize()
    assert A.attention_status() == 0
    ro, rl = A.attention_varlen_reference(q, k, v, cu_q, cu_k, causal=causal)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - ro).abs().max().item() < 3e-2
    assert (lse - rl).abs().max().item() < 2e-3
    # relative check on the whole tensor: the error is rounding of P and O to bf16
    assert ((o.float() - ro).norm() / ro.norm()).item() < 1e-2


def test_one_sequence_with_a_ragged_tail():
    _case([300], [300])


def test_packed_sequences_of_unequal_length():
    _case([130, 77, 512, 1], [130, 77, 512, 1], hq=12, hkv=2)


def test_prefill_chunk_over_cached_keys():
    _case([128, 60], [700, 61])


def test_non_causal():
    _case([200], [333], causal=False)


def test_operands_sliced_from_a_fused_projection():
    _case([257, 640], [257, 640], hq=6, hkv=1, fused=True)

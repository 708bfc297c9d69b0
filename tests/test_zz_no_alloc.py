"""The no-allocation sampler entry point (``pear_fused_sample_static``, declared in ``ops/csrc/pear_no_alloc.h``) called
as the exported C symbol: same results as the regular entry point on two calls in a row, nothing allocated by the call,
sizes beyond the built-in workspace refused. (Named to be collected last: it must pass alone and after other tests.)"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, logits, noise, temperature, chunks, topk):
    rows, v = logits.shape
    dev = logits.device
    out = dict(tok=torch.empty(rows, dtype=torch.int32, device=dev), lp=torch.empty(rows, device=dev),
               tid=torch.empty(rows, topk, dtype=torch.int32, device=dev), tlp=torch.empty(rows, topk, device=dev),
               rank=torch.empty(rows, dtype=torch.int32, device=dev), nf=torch.empty(rows, dtype=torch.int32, device=dev))
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    before = torch.cuda.memory_allocated()
    code = lib.pear_fused_sample_static(p(logits), rows, v, logits.stride(0), ctypes.c_float(temperature), p(noise), chunks, topk,
                                        p(out["tok"]), p(out["lp"]), p(out["tid"]), p(out["tlp"]), p(out["rank"]), p(out["nf"]),
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert torch.cuda.memory_allocated() == before
    return code, out


def test_no_alloc_sampler_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import lib as kl, rollout_ops
    lib = kl.lib()
    lib.pear_fused_sample_static.restype = ctypes.c_int
    g = torch.Generator(device="cuda").manual_seed(11)
    for call in range(2):  # two calls in a row reuse the same built-in workspace
        logits = torch.randn(5, 50000, device="cuda", generator=g) * 2
        noise = torch.rand(5, 50000, device="cuda", generator=g)
        code, out = _call(lib, logits, noise, 0.8, 16, 32)
        assert code == 0
        torch.cuda.synchronize()
        tok, lp, tid, tlp, rank, nf = rollout_ops.fused_sample(logits, 0.8, noise, 32, chunks=16)
        assert torch.equal(out["tok"].long(), tok) and torch.equal(out["lp"], lp) and torch.equal(out["tid"].long(), tid)
        assert torch.equal(out["tlp"], tlp) and torch.equal(out["rank"].long(), rank) and torch.equal(out["nf"].long(), nf)
    # sizes beyond the built-in workspace, and bad arguments, are refused before anything is launched
    big = torch.zeros(65, 64, device="cuda")
    assert _call(lib, big, torch.rand(65, 64, device="cuda"), 1.0, 1, 4)[0] == -2
    many = torch.zeros(40, 64, device="cuda")
    assert _call(lib, many, torch.rand(40, 64, device="cuda"), 1.0, 32, 4)[0] == -2
    assert _call(lib, many, torch.rand(40, 64, device="cuda"), 1.0, 1, 33)[0] == -3
    assert _call(lib, many, torch.rand(40, 64, device="cuda"), 0.0, 1, 4)[0] == -3

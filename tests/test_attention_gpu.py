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


def test_one_sequence_of_8192_tokens():
    """The length of the profile (64 key tiles per query tile: many lazy rescales, the tile loop's phase bits wrap)."""
    _case([8192], [8192], hq=6, hkv=1)


def test_four_packed_sequences_of_8192_tokens():
    _case([8192] * 4, [8192] * 4, hq=6, hkv=1, seed=3)


def test_model_attention_without_gradients_runs_the_kernel():
    from pear_b200.ops import kernels as K
    from pear_b200.ops import lib as kl
    from pear_b200.ops import reference as ref

    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(400, 8, 256, device=dev, generator=g)
    k = torch.randn(400, 2, 256, device=dev, generator=g)
    v = torch.randn(400, 2, 256, device=dev, generator=g)
    bounds = [0, 150, 400]
    before = kl.LAUNCH_COUNT
    with torch.no_grad():
        o = K.causal_attention(q, k, v, bounds)
    assert kl.LAUNCH_COUNT == before + 1
    want = ref.causal_attention(q, k, v, bounds)
    assert o.dtype == torch.float32 and ((o - want).norm() / want.norm()).item() < 1e-2
    # with gradients: the same forward kernel, the backward by the FlashAttention-2 library kernel on its output and lse
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v)]
    w = torch.randn(400, 8, 256, device=dev, generator=g)
    before = kl.LAUNCH_COUNT
    (K.causal_attention(*leaves, bounds) * w).sum().backward()
    assert kl.LAUNCH_COUNT == before + 1
    leaves2 = [x.clone().requires_grad_(True) for x in (q, k, v)]
    (ref.causal_attention(*leaves2, bounds) * w).sum().backward()
    for a, b in zip(leaves, leaves2):
        assert ((a.grad - b.grad).norm() / b.grad.norm()).item() < 2e-2


def test_rollout_prefill_at_head_dim_256_goes_through_the_kernel():
    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.ops import lib as kl
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=1, head_dim=256, rotary_dim=64,
                       gdn_qk_heads=2, gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=0)
    prompts = [list(range(3, 300)), list(range(100, 117))]
    counts = {}
    for use in (True, False):
        model = HybridForCausalLM(cfg, with_mtp=False).init_weights(4)
        eng = RolloutEngine(model, EngineConfig(num_blocks=128, max_num_seqs=4), device="cuda")
        eng.runner.use_kernels = use
        before = kl.LAUNCH_COUNT
        reqs = eng.generate(prompts, SamplingParams(max_tokens=4, temperature=0.0))
        counts[use] = kl.LAUNCH_COUNT - before
        assert all(len(r.output) == 4 and all(0 <= t < cfg.vocab_size for t in r.output) for r in reqs)
    assert counts[True] > counts[False]

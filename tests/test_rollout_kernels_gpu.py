"""Stand-alone rollout kernels against plain PyTorch fp32 references of the same ops."""

import math

import pytest
import torch

from pear_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import rollout_ops
    return rollout_ops


def test_fused_sampler(ops):
    g = torch.Generator(device="cuda").manual_seed(0)
    for rows, v, k in ((4, 248320, 32), (3, 5000, 8), (1, 1024, 32)):
        logits = torch.randn(rows, v, device="cuda", generator=g) * 3
        u = torch.rand(rows, v, device="cuda", generator=g)
        tok, lp, tid, tlp, rank, nf = ops.fused_sample(logits, 0.7, u, k)
        rt, rlp, rid, rtlp, rrank, rnf = ref.sample_exponential_race(logits, 0.7, u, k)
        assert torch.equal(tok, rt) and torch.equal(rank, rrank) and torch.equal(nf, rnf)
        assert torch.allclose(lp, rlp, atol=1e-3) and torch.allclose(tlp, rtlp, atol=1e-3) and torch.equal(tid, rid)
    bad = torch.randn(2, 4096, device="cuda", generator=g)
    bad[0, 5], bad[1, 7], bad[1, 9] = float("nan"), float("inf"), float("-inf")
    nf = ops.fused_sample(bad, 1.0, torch.rand(2, 4096, device="cuda", generator=g), 4)[5]
    assert nf.tolist() == [1, 1]


def test_verify_greedy(ops):
    g = torch.Generator(device="cuda").manual_seed(1)
    r, n, v = 6, 3, 4096
    logits = torch.randn(r, n + 1, v, device="cuda", generator=g) * 2
    logp = torch.log_softmax(logits.float() / 0.9, -1)
    drafts = logits[:, :n].argmax(-1)  # greedy drafts of the same distribution: high acceptance
    drafts[1, 0] = 17  # an unlikely draft: rejected at row 0
    au = torch.rand(r, n, device="cuda", generator=g)
    u = torch.rand(r, n + 1, v, device="cuda", generator=g)
    tok, acc, lp = ops.verify_greedy(logits, drafts, 0.9, au, u)
    for i in range(r):
        a = 0
        while a < n and logp[i, a, drafts[i, a]] > math.log(max(float(au[i, a]), 1e-30)):
            a += 1
        assert int(acc[i]) == a
        assert tok[i, :a].tolist() == drafts[i, :a].tolist()
        z = logits[i, a].float() / 0.9
        key = z - torch.log(-torch.log(u[i, a].clamp(1e-20, 1 - 1e-7)))
        if a < n:
            key[drafts[i, a]] = float("-inf")
        assert int(tok[i, a]) == int(key.argmax()) and abs(float(lp[i, a]) - float(logp[i, a, tok[i, a]])) < 1e-3
        assert (tok[i, a + 1:] == -1).all()


def test_gdn_decode_step(ops):
    g = torch.Generator(device="cuda").manual_seed(2)
    B, Hk, Hv, D = 3, 4, 8, 128
    C = 2 * Hk * D + Hv * D
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    conv_w, A_log, dt_bias, norm_w = rn(C, 4) * 0.5, rn(Hv) * 0.1, rn(Hv) * 0.1, rn(D) * 0.1 + 1
    slots = torch.tensor([4, 0, 2], device="cuda")
    conv_state, state = rn(6, 3, C) * 0.5, rn(6, Hv, D, D) * 0.1
    cs_ref, st_ref = conv_state.clone(), state.clone()
    for step in range(3):
        x, z, a, b = rn(B, C), rn(B, Hv * D), rn(B, Hv), rn(B, Hv)
        out = ops.gdn_decode(x, z, a, b, conv_w, A_log, dt_bias, norm_w, conv_state, state, slots, Hk, Hv)
        for i in range(B):
            s = int(slots[i])
            y, fin = ref.causal_conv_silu(x[i:i + 1], conv_w, None, cs_ref[s][None])
            cs_ref[s] = fin[0]
            q = ref.l2norm(y[:, : Hk * D].view(1, Hk, D)) * D ** -0.5
            k = ref.l2norm(y[:, Hk * D: 2 * Hk * D].view(1, Hk, D))
            v = y[:, 2 * Hk * D:].view(1, Hv, D)
            gg, beta = ref.gdn_gates(a[i:i + 1], b[i:i + 1], A_log, dt_bias)
            o, st_ref[s] = ref.gdn_recurrent(q, k, v, gg, beta, st_ref[s])
            want = ref.gated_rms_norm(o[0], z[i].view(Hv, D), norm_w).reshape(-1)
            assert torch.allclose(out[i], want, atol=2e-4, rtol=2e-3), (out[i] - want).abs().max()
        assert torch.allclose(conv_state, cs_ref) and torch.allclose(state, st_ref, atol=1e-4, rtol=1e-3)


def test_paged_attention(ops):
    g = torch.Generator(device="cuda").manual_seed(3)
    Hq, Hkv, D, nblocks = 12, 2, 256, 64
    kc = (torch.randn(nblocks, 16, Hkv, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nblocks, 16, Hkv, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    lens = [37, 160, 1, 203]
    perm = torch.randperm(nblocks, device="cuda", generator=g)
    table = torch.zeros(len(lens), 16, dtype=torch.int32, device="cuda")
    off = 0
    for i, n in enumerate(lens):
        nb = (n + 15) // 16
        table[i, :nb] = perm[off: off + nb]
        off += nb
    q = torch.randn(len(lens), Hq, D, device="cuda", generator=g)
    out = ops.paged_attention(q, kc, vc, table, torch.tensor(lens, device="cuda"), D ** -0.5)
    for i, n in enumerate(lens):
        nb = (n + 15) // 16
        k = kc[table[i, :nb].long()].reshape(-1, Hkv, D)[:n]
        v = vc[table[i, :nb].long()].reshape(-1, Hkv, D)[:n]
        want = ref.attention_with_cache(q[i:i + 1], k, v, n - 1, D ** -0.5)[0]
        assert torch.allclose(out[i], want, atol=2e-3, rtol=2e-3), (out[i] - want).abs().max()


def test_embed_merge_and_kv_block_copy(ops):
    g = torch.Generator(device="cuda").manual_seed(4)
    table = torch.randn(1000, 512, device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 1000, (33,), device="cuda", generator=g)
    emb = torch.randn(33, 512, device="cuda", generator=g)
    mask = torch.rand(33, device="cuda", generator=g) < 0.3
    out = ops.embed_merge(ids, table, emb, mask)
    want = torch.where(mask[:, None], emb, table[ids].float())
    assert torch.equal(out, want)
    assert torch.equal(ops.embed_merge(ids, table), table[ids].float())
    cache = torch.randn(40, 16, 4, 64, device="cuda", generator=g).to(torch.bfloat16)
    staging = torch.zeros(8, 16, 4, 64, dtype=torch.bfloat16, device="cuda")
    bid = torch.tensor([3, 39, 0, 17, 5], device="cuda")
    ops.kv_blocks_copy(cache, staging, bid, True)
    assert torch.equal(staging[:5], cache[bid])
    cache2 = torch.zeros_like(cache)
    ops.kv_blocks_copy(cache2, staging, bid, False)
    others = torch.ones(40, dtype=torch.bool, device="cuda")
    others[bid] = False
    assert torch.equal(cache2[bid], cache[bid]) and not cache2[others].any()


def test_rollout_sampler_uses_the_fused_kernel_on_gpu(ops):
    from pear_b200.ops import lib as kl
    from pear_b200.rollout import sampler
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(3, 9000, device="cuda", generator=g)
    noise = torch.rand(3, 9000, device="cuda", generator=g)
    before = kl.LAUNCH_COUNT
    out = sampler.sample(logits, 0.8, 1.0, -1, topk_logprobs=8, noise=noise)
    assert kl.LAUNCH_COUNT == before + 2
    want = sampler.sample(logits.cpu(), 0.8, 1.0, -1, topk_logprobs=8, noise=noise.cpu())
    assert torch.equal(out.tokens.cpu(), want.tokens) and torch.allclose(out.logprobs.cpu(), want.logprobs, atol=1e-3)
    assert torch.equal(out.topk_ids.cpu(), want.topk_ids) and torch.equal(out.ranks.cpu(), want.ranks)
    # top-p rows: the nucleus kernel, then the fused sampler
    before = kl.LAUNCH_COUNT
    sampler.sample(logits, 0.8, 0.9, -1, noise=noise)
    assert kl.LAUNCH_COUNT == before + 3
    # top-k rows take the general path
    before = kl.LAUNCH_COUNT
    sampler.sample(logits, 0.8, 1.0, 5, noise=noise)
    assert kl.LAUNCH_COUNT == before


def test_fused_head_forward(ops):
    g = torch.Generator(device="cuda").manual_seed(6)
    t, h, v, j = 300, 512, 40000, 5
    hidden = torch.randn(t, h, device="cuda", generator=g)
    w = torch.randn(v, h, device="cuda", generator=g) * 0.05
    ids = torch.randint(0, v, (t, j), device="cuda", generator=g)
    lp, ent = ops.logprob_entropy_fused(hidden, w, ids, 0.9, row_chunk=128, vocab_chunk=8192)
    logits = hidden.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().t() / 0.9
    logp = torch.log_softmax(logits, -1)
    assert torch.allclose(lp, logp.gather(1, ids), atol=2e-3, rtol=1e-3)
    assert torch.allclose(ent, -(logp.exp() * logp).sum(-1), atol=2e-3, rtol=1e-3)


def test_gdn_front_end(ops):
    g = torch.Generator(device="cuda").manual_seed(7)
    hk, hv, d = 2, 4, 128
    c = 2 * hk * d + hv * d
    cu = [0, 5, 6, 40]
    x = torch.randn(cu[-1], c, device="cuda", generator=g)
    w = torch.randn(c, 4, device="cuda", generator=g) * 0.5
    y = ops.gdn_front(x, w, cu, 2 * hk * d)
    want, _ = ref.causal_conv_silu(x, w, cu)
    q = ref.l2norm(want[:, : hk * d].view(-1, hk, d)).reshape(-1, hk * d) * d ** -0.5
    k = ref.l2norm(want[:, hk * d: 2 * hk * d].view(-1, hk, d)).reshape(-1, hk * d)
    want = torch.cat([q, k, want[:, 2 * hk * d:]], dim=1)
    assert torch.allclose(y, want, atol=1e-5, rtol=1e-4), (y - want).abs().max()


def test_rollout_engine_decodes_through_the_kernels(ops):
    """The engine's decode steps on a GPU use the paged-attention and GDN-decode kernels; tokens equal the PyTorch path."""
    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.ops import lib as kl
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=8, num_kv_heads=2, head_dim=128, rotary_dim=64,
                       gdn_qk_heads=2, gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=0)
    prompts = [list(range(3, 40)), list(range(100, 117)), [5, 6, 7]]
    outs = {}
    for use in (True, False):
        model = HybridForCausalLM(cfg, with_mtp=False).init_weights(4)
        eng = RolloutEngine(model, EngineConfig(num_blocks=128, max_num_seqs=4), device="cuda")
        eng.runner.use_kernels = use
        before = kl.LAUNCH_COUNT
        reqs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
        outs[use] = ([r.output for r in reqs], kl.LAUNCH_COUNT - before)
    assert outs[True][0] == outs[False][0]
    assert outs[True][1] > outs[False][1] + 50  # the decode steps launched the attention and GDN kernels


def test_exact_max_top_p_kernel(ops):
    """The nucleus kernel against the definition (sort by probability, keep the shortest prefix whose mass reaches p) and
    against the bisection statement of rollout/sampler.py, on rows with a dominant token, a flat tail and ties."""
    import torch
    from pear_b200.rollout import sampler as S

    torch.manual_seed(0)
    rows, V, temp = 6, 248320, 0.8
    logits = torch.randn(rows, V, device="cuda") * 2.0
    logits[0, 123] = 40.0                      # one token holds (almost) everything: the nucleus is that token
    logits[1] = 0.0                            # a flat row: every token is tied with the pivot and kept
    logits[2, :4] = torch.tensor([9.0, 9.0, 9.0, 1.0], device="cuda")  # ties at the pivot
    top_p = torch.tensor([0.9, 0.5, 0.6, 0.95, 1.0, 0.2], device="cuda")
    x = logits.clone()
    ops.top_p_mask_(x, top_p, temp)
    torch.cuda.synchronize()
    kept = torch.isfinite(x)
    assert torch.equal(x[kept], logits[kept])                      # kept tokens are untouched
    assert kept[4].all()                                           # top_p = 1: the row is left alone
    assert kept[0].sum() == 1 and kept[0, 123] and kept[1].all()
    p = torch.softmax(logits.double() / temp, -1)
    for r in range(rows):
        if float(top_p[r]) >= 1.0:
            continue
        mass = float(p[r][kept[r]].sum())
        assert mass >= float(top_p[r]) - 1e-6, (r, mass)
        # minimal up to ties and the bisection's resolution: dropping every token at the smallest kept probability (and the
        # ones within 2^-18 of the largest probability of it) falls below p
        pivot = float(p[r][kept[r]].min())
        res = float(p[r].max()) * 2.0 ** -17
        assert float(p[r][p[r] > pivot + res].sum()) < float(top_p[r]) + 1e-6, r
        assert not (p[r][~kept[r]] > pivot + res).any()              # nothing above the pivot was dropped
    want = S.top_p_mask_exact_max(logits / temp, top_p)
    differ = (want != kept)
    # the two bisections add in different orders: they may part on tokens within the last bisection step of the pivot only
    assert int(differ.sum()) <= 8, int(differ.sum())


def test_sampler_with_top_p_runs_the_kernels(ops):
    import torch
    from pear_b200.ops import lib as kl
    from pear_b200.rollout import sampler as S

    torch.manual_seed(1)
    logits = torch.randn(4, 4096, device="cuda") * 3
    before = kl.LAUNCH_COUNT
    out = S.sample(logits, 0.7, 0.3, generator=torch.Generator(device="cuda").manual_seed(5))
    assert kl.LAUNCH_COUNT > before  # top-p kernel + fused sampler, not the torch statements
    keep = S.top_p_mask_exact_max(logits / 0.7, torch.full((4,), 0.3, device="cuda"))
    assert all(bool(keep[i, int(out.tokens[i])]) for i in range(4))  # every sampled token lies inside its row's nucleus
    lp = torch.log_softmax((logits / 0.7).masked_fill(~keep, float("-inf")), -1)
    got = out.logprobs.reshape(-1)
    assert all(abs(float(got[i]) - float(lp[i, int(out.tokens[i])])) < 2e-3 for i in range(4))

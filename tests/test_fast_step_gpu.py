"""The batched GPU-resident rollout step: every new kernel against a plain PyTorch fp32 statement of the same op, then the
whole step (graph replay included) against the incremental fp32 oracle of the model."""

import math

import pytest
import torch

from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import DenseCache, HybridForCausalLM, forward_cached
from pear_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import decode_ops
    return decode_ops


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g) * scale


@pytest.mark.parametrize("m,n,k,ns", [(128, 5120, 6144, 3), (4, 1000, 512, 1), (300, 520, 1096, 2), (64, 384, 256, 4), (32, 12288, 1024, 1)])
def test_stream_gemm_planes(K, m, n, k, ns):
    x = _rand(m, k, scale=0.5, seed=1).to(torch.bfloat16)
    w = _rand(n, k, scale=0.1, seed=2).to(torch.bfloat16)
    out = torch.full((ns, m, n + 4), float("nan"), device="cuda")
    K.stream_gemm(x, w, out, ns, 0)
    torch.cuda.synchronize()
    K.check_status()
    got = out[:, :, :n].sum(0)
    want = x.float() @ w.float().t()
    assert torch.isnan(out[:, :, n:]).all()  # nothing written outside the N columns
    assert (got - want).abs().max() <= 2e-3 * want.abs().max() + 1e-4


def test_stream_gemm_bf16_and_swiglu(K):
    m, f, k = 200, 1000, 768
    x = _rand(m, k, scale=0.5, seed=3).to(torch.bfloat16)
    w = _rand(2 * f, k, scale=0.1, seed=4).to(torch.bfloat16)
    out = torch.zeros(m, 2 * f, dtype=torch.bfloat16, device="cuda")
    want = x.float() @ w.float().t()
    K.stream_gemm(x[:120], w, out[:120], 1, 1)
    assert (out[:120].float() - want[:120]).abs().max() <= 1e-2 * want.abs().max()
    out.zero_()
    K.stream_gemm(x, w, out, 1, 1)
    assert (out.float() - want).abs().max() <= 1e-2 * want.abs().max()
    act = torch.zeros(m, f, dtype=torch.bfloat16, device="cuda")
    K.stream_gemm(x, w, act, 1, 2, up_row0=f, n=f)
    torch.cuda.synchronize()
    K.check_status()
    want_act = torch.nn.functional.silu(want[:, :f]) * want[:, f:]
    assert (act.float() - want_act).abs().max() <= 1.5e-2 * want_act.abs().max()


def _paged_setup(batch, t, hq, hkv, d, ctx_list, seed=0, gated=True):
    """Random q/k/v projection rows and a paged cache already holding `ctx` tokens per sequence."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    bs = 16
    max_blocks = (max(ctx_list) + t + bs - 1) // bs + 1
    pages = batch * max_blocks + 1
    kc = torch.zeros(pages, bs, hkv, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    table = torch.zeros(batch, max_blocks, dtype=torch.int32, device="cuda")
    perm = torch.randperm(pages - 1, generator=torch.Generator().manual_seed(seed)) + 1
    dense_k, dense_v = [], []
    for b in range(batch):
        table[b] = perm[b * max_blocks:(b + 1) * max_blocks].int().cuda()
        k = (torch.randn(ctx_list[b], hkv, d, device="cuda", generator=g)).to(torch.bfloat16)
        v = (torch.randn(ctx_list[b], hkv, d, device="cuda", generator=g)).to(torch.bfloat16)
        for p in range(ctx_list[b]):
            kc[table[b, p // bs], p % bs] = k[p]
            vc[table[b, p // bs], p % bs] = v[p]
        dense_k.append(k)
        dense_v.append(v)
    qw = (2 if gated else 1) * hq * d
    qkv = torch.randn(batch * t, qw + 2 * hkv * d, device="cuda", generator=g)
    return kc, vc, table, qkv, dense_k, dense_v


@pytest.mark.parametrize("d,hq,hkv,t,rot,gated", [(256, 12, 2, 4, 64, True), (256, 6, 1, 1, 64, True), (64, 4, 2, 3, 32, True), (128, 8, 8, 2, 64, False)])
def test_attn_prep_and_paged_attention(K, d, hq, hkv, t, rot, gated):
    batch = 3
    ctx_list = [130, 17, 300]
    kc, vc, table, qkv, dense_k, dense_v = _paged_setup(batch, t, hq, hkv, d, ctx_list, seed=5, gated=gated)
    ctx = torch.tensor(ctx_list, dtype=torch.int32, device="cuda")
    rope_off = torch.tensor([0, 3, 0], dtype=torch.int32, device="cuda")
    qn = _rand(d, scale=0.1, seed=6)
    kn = _rand(d, scale=0.1, seed=7)
    theta = 1e6
    inv_freq = (theta ** (-torch.arange(rot // 2, dtype=torch.float64) * 2.0 / rot)).cuda()
    q_out = torch.zeros(batch * t, hq, d, dtype=torch.bfloat16, device="cuda")
    K.attn_prep(qkv, qn, kn, inv_freq, rot, ctx, rope_off, table, batch * t, t, hq, hkv, d, gated, 1e-6, q_out, kc, vc)
    out = torch.zeros(batch * t, hq * d, dtype=torch.bfloat16, device="cuda")
    K.paged_attention(q_out, kc, vc, table, ctx, batch, t, hq, hkv, d, d ** -0.5, qkv, gated, out)
    out_simt = torch.zeros_like(out)
    K.paged_attention(q_out, kc, vc, table, ctx, batch, t, hq, hkv, d, d ** -0.5, qkv, gated, out_simt, tensor_core=False)
    torch.cuda.synchronize()
    K.check_status()
    # the plain statement
    qs = 2 * d if gated else d
    group = hq // hkv
    for b in range(batch):
        rows = qkv[b * t:(b + 1) * t]
        qg = rows[:, : hq * qs].view(t, hq, qs)
        q, gate = qg[..., :d], (qg[..., d:] if gated else None)
        k = rows[:, hq * qs: hq * qs + hkv * d].view(t, hkv, d)
        v = rows[:, hq * qs + hkv * d:].view(t, hkv, d)
        pos = torch.arange(ctx_list[b], ctx_list[b] + t, device="cuda") + int(rope_off[b])
        cos, sin = ref.mrope_cos_sin(pos, rot, theta, (rot // 2 - 2 * (rot // 6), rot // 6, rot // 6))
        qr = ref.apply_rope(ref.rms_norm(q, qn, 1e-6), cos, sin)
        kr = ref.apply_rope(ref.rms_norm(k, kn, 1e-6), cos, sin)
        assert (q_out[b * t:(b + 1) * t].float() - qr).abs().max() < 0.03
        kk = torch.cat([dense_k[b].float(), kr.to(torch.bfloat16).float()], 0)
        vv = torch.cat([dense_v[b].float(), v.to(torch.bfloat16).float()], 0)
        # what the kernels wrote into the pages
        for j in range(t):
            p = ctx_list[b] + j
            assert torch.equal(kc[table[b, p // 16], p % 16], kr[j].to(torch.bfloat16)) or (kc[table[b, p // 16], p % 16].float() - kr[j]).abs().max() < 0.03
            assert torch.equal(vc[table[b, p // 16], p % 16], v[j].to(torch.bfloat16))
        qb = q_out[b * t:(b + 1) * t].float()
        for j in range(t):
            n = ctx_list[b] + j + 1
            for h in range(hq):
                s = (kk[:n, h // group] @ qb[j, h]) * d ** -0.5
                o = torch.softmax(s, 0) @ vv[:n, h // group]
                if gated:
                    o = o * torch.sigmoid(gate[j, h])
                for got in (out, out_simt):
                    g_ = got[b * t + j, h * d:(h + 1) * d].float()
                    assert (g_ - o).abs().max() < 0.03, (b, j, h, float((g_ - o).abs().max()))


def test_gdn_verify_replay(K):
    """Three steps with different accepted counts against the token recurrence run only over the accepted rows."""
    hk, hv, D, T = 2, 4, 128, 4
    C = 2 * hk * D + hv * D
    B, slots = 3, 5
    g = torch.Generator(device="cuda").manual_seed(11)
    conv_w = torch.randn(C, 4, device="cuda", generator=g) * 0.3
    a_log = torch.log(torch.rand(hv, device="cuda", generator=g) * 4 + 1)
    dt_bias = torch.randn(hv, device="cuda", generator=g) * 0.1
    norm_w = torch.rand(D, device="cuda", generator=g) + 0.5
    state = torch.randn(slots, hv, D, D, device="cuda", generator=g) * 0.1
    conv_rec = torch.zeros(slots, 2, 3 + T, C, device="cuda")
    ab_rec = torch.zeros(slots, 2, T, 2 * hv, device="cuda")
    slot_ids = torch.tensor([3, 0, 4], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([5, -1, 9], dtype=torch.int32, device="cuda")  # the middle batch slot is empty
    parity = torch.zeros(B, dtype=torch.int32, device="cuda")
    ncommit = torch.zeros(B, dtype=torch.int32, device="cuda")
    win0 = torch.randn(slots, 3, C, device="cuda", generator=g)
    conv_rec[:, 0, :3] = win0
    # oracle state per active sequence
    o_state = {b: state[int(slot_ids[b])].clone() for b in (0, 2)}
    o_win = {b: win0[int(slot_ids[b])].clone() for b in (0, 2)}
    ld = C + hv * D + 2 * hv
    accepted_plan = [[2, 4], [1, 3], [4, 1]]  # rows committed after each step, per active sequence
    state_before = state.clone()
    for step in range(3):
        proj = torch.randn(B * T, ld, device="cuda", generator=g)
        out = torch.zeros(B * T, hv * D, dtype=torch.bfloat16, device="cuda")
        K.gdn_verify(proj, conv_w, a_log, dt_bias, norm_w, state, conv_rec, ab_rec, slot_ids, ctx, parity, ncommit, B, T, T, hk, hv, 1e-6, 1e-6, out)
        torch.cuda.synchronize()
        assert torch.equal(state[int(slot_ids[1])], state_before[int(slot_ids[1])])  # empty slot untouched
        for n, b in enumerate((0, 2)):
            rows = proj[b * T:(b + 1) * T]
            mixed, z = rows[:, :C], rows[:, C:C + hv * D].view(T, hv, D)
            bb, aa = rows[:, C + hv * D:C + hv * D + hv], rows[:, C + hv * D + hv:]
            u, _ = ref.causal_conv_silu(mixed, conv_w, [0, T], o_win[b][None])
            q = ref.l2norm(u[:, :hk * D].view(T, hk, D)) * D ** -0.5
            k = ref.l2norm(u[:, hk * D:2 * hk * D].view(T, hk, D))
            v = u[:, 2 * hk * D:].view(T, hv, D)
            gg, beta = ref.gdn_gates(aa, bb, a_log, dt_bias)
            o, _ = ref.gdn_recurrent(q, k, v, gg, beta, o_state[b])
            y = ref.gated_rms_norm(o, z, norm_w, 1e-6).reshape(T, hv * D)
            got = out[b * T:(b + 1) * T].float()
            assert (got - y).abs().max() < 0.02 * max(1.0, float(y.abs().max())), (step, b)
            acc = accepted_plan[step][n]
            _, o_state[b] = ref.gdn_recurrent(q[:acc], k[:acc], v[:acc], gg[:acc], beta[:acc], o_state[b])
            o_win[b] = torch.cat([o_win[b], mixed[:acc]], 0)[-3:]
            ncommit[b] = acc
            parity[b] ^= 1
            ctx[b] += acc
    # flush: replay the last accepted rows, state equals the oracle's
    K.gdn_verify(None, conv_w, a_log, dt_bias, norm_w, state, conv_rec, ab_rec, slot_ids, ctx, parity, ncommit, B, 0, T, hk, hv, 1e-6, 1e-6, None)
    torch.cuda.synchronize()
    for b in (0, 2):
        s = int(slot_ids[b])
        assert (state[s] - o_state[b]).abs().max() < 2e-4 * max(1.0, float(o_state[b].abs().max()))
        assert torch.allclose(conv_rec[s, int(parity[b]) ^ 1, :3], o_win[b])


def test_sharded_verify_sampler(K):
    """Two emulated vocabulary shards on one GPU (two chunk launches into one record buffer) against torch on the same noise."""
    B, T, V, world, chunks = 5, 4, 4096, 2, 3
    seed, temp = 1234, 0.8
    g = torch.Generator(device="cuda").manual_seed(21)
    logits = torch.randn(B * T, V, device="cuda", generator=g) * 3
    i32 = dict(dtype=torch.int32, device="cuda")
    tok_in = torch.randint(0, V, (B * T,), device="cuda", generator=g).int()
    lp_all = torch.log_softmax(logits / temp, -1)
    for b in range(B):  # greedy drafts of the same distribution: most are accepted
        for t in range(T - 1):
            tok_in[b * T + t + 1] = int(logits[b * T + t].argmax())
    tok_in[1 * T + 1] = 77  # an unlikely draft: rejected at row 0
    ctx = torch.tensor([10, 20, -1, 40, 50], **i32)
    step_ctr = torch.full((1,), 7, **i32)
    Vs = V // world
    recs = torch.zeros(world * B * T * chunks * K.rec_bytes(), dtype=torch.uint8, device="cuda")
    ptrs = K._ptr_array([recs.data_ptr()])
    tok0 = tok_in.clone()
    for r in range(world):
        shard = logits[:, r * Vs:(r + 1) * Vs].contiguous()
        # rank r of a 2-rank world writing into a single-rank pointer table: emulate by offsetting through `rank`
        from pear_b200.ops import lib as _lib
        import ctypes
        _lib.check(_lib.lib().pear_ds_verify_chunks(_lib.ptr(shard), shard.stride(0), Vs, r * Vs, ctypes.c_float(temp), _lib.ptr(tok_in), _lib.ptr(ctx), B, T,
                                                    chunks, ctypes.c_uint(seed), _lib.ptr(step_ctr), K._ptr_array([recs.data_ptr()] * 2), r, 1,
                                                    _lib.ptr(None), ctypes.c_size_t(0), _lib.stream()), "chunks")
    ncommit, parity = torch.zeros(B, **i32), torch.zeros(B, **i32)
    out_tok, out_lp = torch.zeros(B, T, **i32), torch.zeros(B, T, device="cuda")
    n_acc, nonf, sel, mtp_tok, mtp_ctx = torch.zeros(B, **i32), torch.zeros(B, **i32), torch.zeros(B, **i32), torch.zeros(B * T, **i32), torch.zeros(T, B, **i32)
    K.verify_finish(recs, 0, None, world, chunks, B, T, seed, step_ctr, tok_in, ctx, ncommit, parity, out_tok, out_lp, n_acc, nonf, sel, mtp_tok, mtp_ctx)
    torch.cuda.synchronize()
    assert int(step_ctr) == 8
    u = K.philox_uniform(B * T, V, seed, 7)
    au = K.accept_uniform(B * T, seed, 7)
    old = [10, 20, -1, 40, 50]
    for b in range(B):
        if old[b] < 0:
            assert int(n_acc[b]) == 0 and (out_tok[b] == -1).all()
            continue
        a = 0
        while a < T - 1 and float(lp_all[b * T + a, tok0[b * T + a + 1]]) > math.log(max(float(au[b * T + a]), 1e-30)):
            a += 1
        assert int(n_acc[b]) == a, (b, a, int(n_acc[b]))
        assert out_tok[b, :a].tolist() == tok0[b * T + 1:b * T + 1 + a].tolist()
        key = logits[b * T + a] / temp - torch.log(-torch.log(u[b * T + a]))
        if a < T - 1:
            key[tok0[b * T + a + 1]] = float("-inf")
        assert int(out_tok[b, a]) == int(key.argmax())
        assert abs(float(out_lp[b, a]) - float(lp_all[b * T + a, out_tok[b, a]])) < 2e-3
        assert (out_tok[b, a + 1:] == -1).all()
        assert int(ctx[b]) == old[b] + a + 1 and int(ncommit[b]) == a + 1 and int(parity[b]) == 1 and int(sel[b]) == b * T + a
        assert int(tok_in[b * T]) == int(out_tok[b, a])
        assert int(mtp_ctx[0, b]) == old[b] and int(mtp_ctx[1, b]) == old[b] + a + 1


def _small_cfg(mtp=1):
    return HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256, gdn_qk_heads=2,
                        gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=mtp, init_std=0.05)


def _load_from_oracle(dec, model, cfg, b, slot, cache: DenseCache, table, last_token):
    """Copy one sequence's dense oracle cache into the paged caches / state slots and put it into batch slot b."""
    n = cache.length
    for li in cfg.attention_layers:
        for p in range(n):
            dec.k_cache[li][table[p // 16], p % 16] = cache.k[li][p].to(torch.bfloat16)
            dec.v_cache[li][table[p // 16], p % 16] = cache.v[li][p].to(torch.bfloat16)
    conv = {}
    for li in cfg.gdn_layers:
        dec.rec_state[li][slot] = cache.state[li]
        conv[li] = cache.conv[li]
    dec.assign(b, slot, n, table, last_token, conv)


@pytest.mark.parametrize("n_draft,graph", [(0, False), (3, True)])
def test_fast_decoder_matches_oracle(K, n_draft, graph):
    from pear_b200.ops import api
    monkey = api.FORCE_REFERENCE
    api.FORCE_REFERENCE = True  # the oracle is the plain PyTorch statement even on CUDA tensors
    try:
        _run_fast_decoder_case(K, n_draft, graph)
    finally:
        api.FORCE_REFERENCE = monkey


def _run_fast_decoder_case(K, n_draft, graph):
    from pear_b200.rollout.fast_step import FastDecoder

    cfg = _small_cfg()
    torch.manual_seed(0)
    oracle = HybridForCausalLM(cfg).init_weights(3)
    with torch.no_grad():
        for p in oracle.parameters():  # bf16-representable weights: the two models hold the same numbers
            p.copy_(p.to(torch.bfloat16).float())
    oracle = oracle.cuda().eval()
    fast_model = HybridForCausalLM(cfg)
    fast_model.load_state_dict(oracle.state_dict())
    fast_model = fast_model.cuda().eval()
    for name, p in fast_model.named_parameters():
        if p.dim() >= 2 and "conv1d" not in name:
            p.data = p.data.to(torch.bfloat16)
    B, T, pages, slots = 3, 1 + n_draft, 64, 6
    kc = {li: torch.zeros(pages, 16, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device="cuda") for li in cfg.attention_layers}
    vc = {li: torch.zeros_like(kc[li]) for li in cfg.attention_layers}
    rs = {li: torch.zeros(slots, cfg.gdn_v_heads, 128, 128, device="cuda") for li in cfg.gdn_layers}
    mk = [torch.zeros(pages, 16, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device="cuda")]
    mv = [torch.zeros_like(mk[0])]
    dec = FastDecoder(fast_model, kc, vc, rs, mk, mv, slots, B, n_draft, 8, temperature=0.7, seed=5, use_graph=graph)
    dec.debug_logits = torch.zeros_like(dec.logits)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(n)).cuda() for n in (37, 20)]
    caches, last, seqs = [], [], []
    for i, pr in enumerate(prompts):
        c = DenseCache(cfg)
        with torch.no_grad():
            forward_cached(oracle, pr[:-1], c)
        caches.append(c)
        last.append(int(pr[-1]))
        seqs.append(pr.tolist())
    tables = [list(range(1 + 8 * i, 9 + 8 * i)) for i in range(2)]
    _load_from_oracle(dec, oracle, cfg, 0, 4, caches[0], tables[0], last[0])
    _load_from_oracle(dec, oracle, cfg, 2, 1, caches[1], tables[1], last[1])  # batch slot 1 stays empty
    for step in range(6):
        tok_in = dec.tok_in.clone()
        dec.step()
        res = dec.results()
        dec.check()
        for i, b in enumerate((0, 2)):
            rows = tok_in[b * T:(b + 1) * T].long()
            acc = int(res.accepted[b])
            # the oracle runs the same input rows on a copy of the committed cache
            trial = caches[i].clone()
            with torch.no_grad():
                hid = forward_cached(oracle, rows, trial)
                want = oracle.logits(hid)
            got = dec.debug_logits[b * T:(b + 1) * T, :cfg.vocab_size]
            err = float((got - want).abs().max())
            assert err < 0.06 * max(1.0, float(want.abs().max())), (step, b, err)
            new = [int(x) for x in res.tokens[b, :acc + 1]]
            assert all(x >= 0 for x in new) and (res.tokens[b, acc + 1:] == -1).all()
            assert new[:acc] == rows[1:1 + acc].tolist()
            # commit: the accepted rows enter the oracle cache
            with torch.no_grad():
                forward_cached(oracle, rows[:acc + 1], caches[i])
            seqs[i] += new
            assert int(dec.ctx[b]) == caches[i].length
        assert int(res.accepted[1]) == 0 and (res.tokens[1] == -1).all()
    if graph:
        assert dec.graph is not None
    # leaving the batch: the recurrent state equals the oracle's
    conv = dec.release(0)
    torch.cuda.synchronize()
    for li in cfg.gdn_layers:
        assert (rs[li][4] - caches[0].state[li]).abs().max() < 3e-2 * max(1.0, float(caches[0].state[li].abs().max()))
        assert (conv[li] - caches[0].conv[li]).abs().max() < 0.05


def test_paged_attention_shared_prefix_items(K):
    """Sequences whose first 256 tokens live in the same pages: the item form (stacked rows over the shared keys, partial
    results merged) against the one-CTA-per-sequence form and the SIMT statement."""
    batch, t, hq, hkv, d = 5, 4, 12, 2, 256
    ctx_list = [300, 257, 410, 130, 290]  # sequence 3 shares nothing; the others share 256 tokens
    g = torch.Generator(device="cuda").manual_seed(31)
    pages = 200
    kc = torch.randn(pages, 16, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn(pages, 16, hkv, d, device="cuda", generator=g).to(torch.bfloat16)
    table = torch.zeros(batch, 32, dtype=torch.int32, device="cuda")
    shared = torch.arange(1, 17, dtype=torch.int32)
    nxt = 20
    for b in range(batch):
        own = torch.arange(nxt, nxt + 32, dtype=torch.int32)
        nxt += 32
        if b != 3:
            own[:16] = shared
        table[b] = own.cuda()
    ctx = torch.tensor(ctx_list, dtype=torch.int32, device="cuda")
    q = (torch.randn(batch * t, hq, d, device="cuda", generator=g)).to(torch.bfloat16)
    gate = torch.randn(batch * t, 2 * hq * d + 2 * hkv * d, device="cuda", generator=g)
    outs = []
    nparts, splits = 3, 2
    rows = [[1, 256 if b != 3 else 0, -1, 0, 1 + (splits if b != 3 else 0), nparts, 0, 0, b] + [0] * 15 for b in range(batch)]
    for sp in range(splits):
        rows.append([4, sp * 128, (sp + 1) * 128, 1 + sp, 0, 0, 0, 0, 0, 1, 2, 4] + [0] * 12)
    rows.append([0] * 24)  # an empty item
    items = torch.tensor(rows, dtype=torch.int32, device="cuda")
    part_o = torch.full((nparts, batch * t, hq, d), float("nan"), device="cuda")
    part_ml = torch.full((nparts, batch * t, hq, 2), float("nan"), device="cuda")
    for mode in ("items", "direct", "simt"):
        out = torch.zeros(batch * t, hq * d, dtype=torch.bfloat16, device="cuda")
        if mode == "items":
            K.paged_attention(q, kc, vc, table, ctx, batch, t, hq, hkv, d, d ** -0.5, gate, True, out, True, items, nparts, part_o, part_ml)
        else:
            K.paged_attention(q, kc, vc, table, ctx, batch, t, hq, hkv, d, d ** -0.5, gate, True, out, mode == "direct")
        outs.append(out.float())
    torch.cuda.synchronize()
    K.check_status()
    assert (outs[0] - outs[2]).abs().max() < 0.03 and (outs[1] - outs[2]).abs().max() < 0.03


def test_topk_logprob_kernels(K):
    """The 32 largest log-probs per row over two emulated vocabulary shards (two chunk launches into one list buffer) against
    torch.topk of log_softmax; a row with fewer than 32 finite tokens, a flat row (ties at the threshold) and an empty slot."""
    import ctypes

    from pear_b200.ops import lib as _lib

    B, T, V, world, chunks, temp = 4, 2, 8192, 2, 2, 0.7
    g = torch.Generator(device="cuda").manual_seed(31)
    logits = torch.randn(B * T, V, device="cuda", generator=g) * 3
    logits[2, 40:] = float("-inf")            # 40 finite tokens
    logits[3] = 1.5                            # flat: every token ties
    i32 = dict(dtype=torch.int32, device="cuda")
    ctx = torch.tensor([10, 20, -1, 40], **i32)  # the third sequence's slot is empty
    tok_in = torch.zeros(B * T, **i32)
    step_ctr = torch.zeros(1, **i32)
    Vs = V // world
    rows = B * T
    recs = torch.zeros(world * rows * chunks * K.rec_bytes(), dtype=torch.uint8, device="cuda")
    tops = torch.zeros(world * rows * chunks * K.top_bytes(), dtype=torch.uint8, device="cuda")
    for r in range(world):
        shard = logits[:, r * Vs:(r + 1) * Vs].contiguous()
        _lib.check(_lib.lib().pear_ds_verify_chunks(_lib.ptr(shard), shard.stride(0), Vs, r * Vs, ctypes.c_float(temp), _lib.ptr(tok_in), _lib.ptr(ctx), B, T,
                                                    chunks, ctypes.c_uint(1), _lib.ptr(step_ctr), K._ptr_array([recs.data_ptr()] * 2), r, 1,
                                                    _lib.ptr(None), ctypes.c_size_t(0), _lib.stream()), "chunks")
        _lib.check(_lib.lib().pear_ds_topk_chunks(_lib.ptr(shard), shard.stride(0), Vs, r * Vs, ctypes.c_float(temp), _lib.ptr(ctx), B, T, chunks,
                                                  K._ptr_array([tops.data_ptr()] * 2), r, 1, _lib.ptr(None), ctypes.c_size_t(0), _lib.stream()), "topk")
    out_id = torch.full((rows, 32), -7, **i32)
    out_lp = torch.zeros(rows, 32, device="cuda")
    K.topk_finish(tops, 0, recs, 0, None, world, chunks, B, T, ctx, out_id, out_lp)
    torch.cuda.synchronize()
    lp = torch.log_softmax(logits.float() / temp, -1)
    for row in range(rows):
        if int(ctx[row // T]) < 0:
            assert (out_id[row] == -7).all()  # untouched
            continue
        want_lp, want_id = lp[row].topk(32)
        if row == 3:  # all equal: any 32 distinct tokens, each at log(1 / V)
            assert len(set(out_id[row].tolist())) == 32 and (out_id[row] >= 0).all()
            assert torch.allclose(out_lp[row], want_lp, atol=1e-4)
            continue
        n = 32 if row != 2 else 32  # row 2 has 40 finite tokens: still 32 results
        assert torch.equal(out_id[row, :n].long(), want_id[:n]), row
        assert torch.allclose(out_lp[row, :n], want_lp[:n], atol=2e-4), row
    # fewer than 32 finite tokens in the whole row: the rest are tokens at -inf (as torch.topk would list them)
    logits[0, 5:] = float("-inf")
    for r in range(world):
        shard = logits[:, r * Vs:(r + 1) * Vs].contiguous()
        _lib.check(_lib.lib().pear_ds_verify_chunks(_lib.ptr(shard), shard.stride(0), Vs, r * Vs, ctypes.c_float(temp), _lib.ptr(tok_in), _lib.ptr(ctx), B, T,
                                                    chunks, ctypes.c_uint(1), _lib.ptr(step_ctr), K._ptr_array([recs.data_ptr()] * 2), r, 1,
                                                    _lib.ptr(None), ctypes.c_size_t(0), _lib.stream()), "chunks")
        _lib.check(_lib.lib().pear_ds_topk_chunks(_lib.ptr(shard), shard.stride(0), Vs, r * Vs, ctypes.c_float(temp), _lib.ptr(ctx), B, T, chunks,
                                                  K._ptr_array([tops.data_ptr()] * 2), r, 1, _lib.ptr(None), ctypes.c_size_t(0), _lib.stream()), "topk")
    K.topk_finish(tops, 0, recs, 0, None, world, chunks, B, T, ctx, out_id, out_lp)
    torch.cuda.synchronize()
    K.check_status()
    assert out_id[0, :5].tolist() == torch.log_softmax(logits[0] / temp, -1).topk(5).indices.tolist()
    assert torch.isinf(out_lp[0, 5:]).all() and len(set(out_id[0].tolist())) == 32 and (out_id[0] >= 0).all()

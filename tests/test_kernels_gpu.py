"""Elementwise / norm / rope kernels and the tcgen05 GEMM against the plain fp32 torch statements (forward + backward)."""

import pytest
import torch

from pear_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _grads(fn, inputs, gout_seed=0):
    ins = [i.clone().requires_grad_(True) if i.is_floating_point() else i for i in inputs]
    out = fn(*ins)
    outs = out if isinstance(out, tuple) else (out,)
    g = torch.Generator(device=outs[0].device).manual_seed(gout_seed)
    loss = sum((o * torch.randn(o.shape, device=o.device, generator=g)).sum() for o in outs)
    loss.backward()
    return outs, [i.grad for i in ins if i.is_floating_point()]


def _cmp(a, b, tol=2e-5):
    for x, y in zip(a, b):
        scale = y.abs().max().item() + 1e-6
        assert (x.float() - y.float()).abs().max().item() <= tol * scale + 1e-6


@pytest.mark.parametrize("rows,dim,one_plus", [(37, 5120, True), (300, 256, True), (129, 128, False)])
def test_rms_norm(rows, dim, one_plus):
    from pear_b200.ops import kernels as K

    torch.manual_seed(0)
    x = torch.randn(rows, dim, device="cuda") * 3
    w = torch.randn(dim, device="cuda") * 0.2
    o1, g1 = _grads(lambda a, b: K.rms_norm(a, b, 1e-6, one_plus), [x, w])
    o2, g2 = _grads(lambda a, b: ref.rms_norm(a, b, 1e-6, one_plus), [x, w])
    _cmp(o1, o2)
    _cmp(g1, g2, 1e-4)


def test_add_rms_norm():
    from pear_b200.ops import kernels as K

    torch.manual_seed(1)
    x, r = torch.randn(65, 5120, device="cuda"), torch.randn(65, 5120, device="cuda") * 4
    w = torch.randn(5120, device="cuda") * 0.1
    o1, g1 = _grads(lambda a, b, c: K.add_rms_norm(a, b, c, 1e-6), [x, r, w])
    o2, g2 = _grads(lambda a, b, c: ref.add_rms_norm(a, b, c, 1e-6), [x, r, w])
    _cmp(o1, o2)
    _cmp(g1, g2, 1e-4)


def test_gated_rms_norm_swiglu_gate_rope():
    from pear_b200.ops import kernels as K

    torch.manual_seed(2)
    o, z = torch.randn(50, 48, 128, device="cuda"), torch.randn(50, 48, 128, device="cuda")
    w = torch.rand(128, device="cuda") + 0.5
    _o1, _g1 = _grads(lambda a, b, c: K.gated_rms_norm(a, b, c, 1e-6), [o, z, w])
    _o2, _g2 = _grads(lambda a, b, c: ref.gated_rms_norm(a, b, c, 1e-6), [o, z, w])
    _cmp(_o1, _o2); _cmp(_g1, _g2, 1e-4)
    g, u = torch.randn(33, 17408, device="cuda"), torch.randn(33, 17408, device="cuda")
    a1, b1 = _grads(K.swiglu, [g, u]); a2, b2 = _grads(ref.swiglu, [g, u])
    _cmp(a1, a2); _cmp(b1, b2)
    a1, b1 = _grads(K.sigmoid_gate, [g, u]); a2, b2 = _grads(ref.sigmoid_gate, [g, u])
    _cmp(a1, a2); _cmp(b1, b2)
    x = torch.randn(77, 24, 256, device="cuda")
    pos = torch.stack([torch.arange(77), torch.arange(77) // 2, torch.arange(77) // 3]).cuda()
    cos, sin = ref.mrope_cos_sin(pos, 64, 1e7, (11, 11, 10))
    a1, b1 = _grads(lambda t: K.apply_rope(t, cos, sin), [x]); a2, b2 = _grads(lambda t: ref.apply_rope(t, cos, sin), [x])
    _cmp(a1, a2); _cmp(b1, b2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 200), (4096, 5120, 5120), (77, 100, 136), (1024, 34816, 5120)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05(m, n, k, out_dtype):
    from pear_b200.ops import gemm

    torch.manual_seed(3)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(n, k, device="cuda") * 0.5).bfloat16()
    c = gemm.gemm_nt(a, b, out_dtype)
    torch.cuda.synchronize()
    assert gemm.gemm_status() == 0
    refc = a.float() @ b.float().t()
    err = (c.float() - refc).abs().max().item()
    tol = (2e-5 if out_dtype == torch.float32 else 8e-3) * refc.abs().max().item() + 1e-4
    assert err <= tol, f"max err {err} tol {tol}"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (304, 520, 200), (4096, 5120, 5120), (80, 104, 136), (1024, 128, 776)])
def test_gemm_backward_forms(m, n, k):
    """The MN-major operand forms against the fp32 statement: C = A[M,K] B[K,N] (dX = dY W) and C = A[K,M]^T B[K,N] (dW = dY^T X),
    ragged M, N and K (the reduction's tail rows come from the TMA's zero fill)."""
    from pear_b200.ops import gemm, lib as kl

    torch.manual_seed(5)
    a = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(k, n, device="cuda") * 0.5).bfloat16()
    before = kl.LAUNCH_COUNT
    c = gemm.gemm_nn(a, b)
    at = a.t().contiguous()  # stored [K, M]
    c2 = gemm.gemm_tn(at, b)
    torch.cuda.synchronize()
    assert gemm.gemm_status() == 0 and kl.LAUNCH_COUNT == before + 2  # the kernel ran both, not the fallback
    refc = a.float() @ b.float()
    tol = 2e-5 * refc.abs().max().item() + 1e-4
    assert (c - refc).abs().max().item() <= tol
    assert (c2 - refc).abs().max().item() <= tol
    # operands that are column slices of wider matrices (row stride != width)
    wide = (torch.randn(k, n + 64, device="cuda") * 0.5).bfloat16()
    c3 = gemm.gemm_nn(a, wide[:, 32:32 + n] if n % 8 == 0 and 32 * 2 % 16 == 0 else wide[:, :n])
    ref3 = a.float() @ (wide[:, 32:32 + n] if n % 8 == 0 else wide[:, :n]).float()
    assert (c3 - ref3).abs().max().item() <= 2e-5 * ref3.abs().max().item() + 1e-4


def test_linear_bf16_autograd():
    from pear_b200.ops import gemm

    torch.manual_seed(4)
    x = torch.randn(200, 512, device="cuda", requires_grad=True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    from pear_b200.ops import lib as kl

    before = kl.LAUNCH_COUNT
    y = gemm.linear_bf16(x, w)
    y.square().sum().backward()
    assert kl.LAUNCH_COUNT == before + 3  # forward, input gradient and weight gradient: three launches of the own kernel
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = xr.bfloat16().float() @ wr.t()
    yr.square().sum().backward()
    assert (y - yr).abs().max() <= 1e-3 * yr.abs().max()
    assert (x.grad - xr.grad).abs().max() <= 2e-2 * xr.grad.abs().max()
    assert (w.grad.float() - wr.grad).abs().max() <= 2e-2 * wr.grad.abs().max()


def test_split_bf16_gemm_is_close_to_fp32():
    """The head's logits GEMM: three bf16 products in one tcgen05 GEMM over 3K against an fp64 product."""
    from pear_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn(300, 512, device="cuda", generator=g)
    b = torch.randn(1000, 512, device="cuda", generator=g)
    want = (a.double() @ b.double().t())
    got = gemm.matmul_split3(a, b)
    plain = gemm.gemm_nt(a.to(torch.bfloat16), b.to(torch.bfloat16))
    err = ((got.double() - want).norm() / want.norm()).item()
    err_bf16 = ((plain.double() - want).norm() / want.norm()).item()
    assert err < 2e-5 and err < err_bf16 / 50, (err, err_bf16)


def test_chunked_head_on_gpu_matches_the_dense_statement():
    from pear_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(1)
    h = (torch.randn(200, 256, device="cuda", generator=g) * 0.5).requires_grad_(True)
    w = (torch.randn(1024, 256, device="cuda", generator=g) * 0.1).requires_grad_(True)
    ids = torch.randint(0, 1024, (200, 1), device="cuda", generator=g)
    lp, ent = ref.logprob_entropy(h, w, ids, temperature=0.7, chunk=64)
    (lp.sum() + 0.1 * ent.sum()).backward()
    gh, gw = h.grad.clone(), w.grad.clone()
    h.grad = w.grad = None
    lp2, ent2 = ref.logprob_entropy_dense(h.double(), w.double(), ids, temperature=0.7)
    (lp2.sum() + 0.1 * ent2.sum()).backward()
    assert (lp - lp2).abs().max().item() < 1e-4 and (ent - ent2).abs().max().item() < 1e-4
    assert ((gh - h.grad).norm() / h.grad.norm()).item() < 2e-2  # bf16 operands in the gradient products
    assert ((gw - w.grad).norm() / w.grad.norm()).item() < 2e-2


def test_gdn_front_end_backward_matches_autograd_of_the_torch_statement():
    from pear_b200.ops import rollout_ops

    g = torch.Generator(device="cuda").manual_seed(2)
    hk, hv, d = 2, 4, 128
    c = (2 * hk + hv) * d
    bounds = [0, 37, 38, 150]
    x = torch.randn(150, c, device="cuda", generator=g).requires_grad_(True)
    w = (torch.randn(c, 4, device="cuda", generator=g) * 0.5).requires_grad_(True)
    dy = torch.randn(150, c, device="cuda", generator=g)
    y = rollout_ops.gdn_front_autograd(x, w, bounds, 2 * hk * d, 1e-6)
    y.backward(dy)
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    u, _ = ref.causal_conv_silu(x, w, bounds, None)
    kd = hk * d
    q = ref.l2norm(u[:, :kd].reshape(150, hk, d), 1e-6) * d ** -0.5
    k = ref.l2norm(u[:, kd:2 * kd].reshape(150, hk, d), 1e-6)
    want = torch.cat([q.reshape(150, kd), k.reshape(150, kd), u[:, 2 * kd:]], dim=1)
    assert (y - want).abs().max().item() < 1e-5
    want.backward(dy)
    assert (gx - x.grad).abs().max().item() < 1e-4 * max(1.0, x.grad.abs().max().item())
    assert (gw - w.grad).abs().max().item() < 1e-3 * max(1.0, w.grad.abs().max().item())


def test_gdn_chunk_loop_kernel_matches_the_torch_loop_and_the_recurrence():
    from pear_b200.ops import kernels as K
    from pear_b200.ops import lib as kl

    g = torch.Generator(device="cuda").manual_seed(4)
    t, hk, hv, d = 333, 2, 4, 128  # 333 tokens: five full chunks and a padded tail
    q = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g)) * d ** -0.5
    k = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g))
    v = torch.randn(t, hv, d, device="cuda", generator=g)
    gate = -torch.rand(t, hv, device="cuda", generator=g) * 0.2
    beta = torch.rand(t, hv, device="cuda", generator=g)
    s0 = torch.randn(hv, d, d, device="cuda", generator=g) * 0.1
    before = kl.LAUNCH_COUNT
    with torch.no_grad():
        o, s = K.gdn_scan(q, k, v, gate, beta, s0)
    assert kl.LAUNCH_COUNT == before + 1
    o_ref, s_ref = ref.gdn_chunked(q, k, v, gate, beta, s0)
    assert (o - o_ref).abs().max().item() < 1e-4 and (s - s_ref).abs().max().item() < 1e-4
    o_rec, s_rec = ref.gdn_recurrent(q, k, v, gate, beta, s0)
    assert (o - o_rec).abs().max().item() < 2e-3 and (s - s_rec).abs().max().item() < 2e-3
    # with gradients: the same kernel run in reverse gives the state gradients; compare with autograd of the torch loop
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, gate, beta, s0)]
    w_o = torch.randn(t, hv, d, device="cuda", generator=g)
    w_s = torch.randn(hv, d, d, device="cuda", generator=g)
    before = kl.LAUNCH_COUNT
    o1, s1 = K.gdn_scan(*leaves)
    ((o1 * w_o).sum() + (s1 * w_s).sum()).backward()
    assert kl.LAUNCH_COUNT == before + 2  # forward loop + reversed loop
    got = [x.grad.clone() for x in leaves]
    leaves2 = [x.clone().requires_grad_(True) for x in (q, k, v, gate, beta, s0)]
    o2, s2 = ref.gdn_chunked(*leaves2)
    ((o2 * w_o).sum() + (s2 * w_s).sum()).backward()
    for name, a_, b_ in zip(("q", "k", "v", "g", "beta", "s0"), got, [x.grad for x in leaves2]):
        assert ((a_ - b_).norm() / (b_.norm() + 1e-12)).item() < 1e-4, name


def test_fused_adamw_kernel_matches_torch_adamw():
    from pear_b200.ops import lib as kl
    from pear_b200.train.fused_adamw import FusedAdamW

    def run(opt_cls, grad_dtype, **kw):
        g = torch.Generator(device="cuda").manual_seed(0)
        ps = [torch.nn.Parameter(torch.randn(1000, 37, device="cuda", generator=g)), torch.nn.Parameter(torch.randn(13, device="cuda", generator=g))]
        opt = opt_cls(ps, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, **kw)
        for _ in range(3):
            for x in ps:
                gr = torch.randn(x.shape, device="cuda", generator=g).to(grad_dtype)
                x.grad = gr if opt_cls is FusedAdamW else gr.float() * 0.5
            if opt_cls is FusedAdamW:
                opt.step(grad_scale=0.5)
            else:
                opt.step()
        return [x.detach().clone() for x in ps]

    for gd in (torch.float32,):  # torch keeps a parameter's gradient in the parameter's dtype
        before = kl.LAUNCH_COUNT
        a = run(FusedAdamW, gd)
        assert kl.LAUNCH_COUNT == before + 6
        b = run(torch.optim.AdamW, gd, foreach=False, fused=False)
        for x, y in zip(a, b):
            assert torch.allclose(x, y, atol=1e-6, rtol=1e-5), (x - y).abs().max()

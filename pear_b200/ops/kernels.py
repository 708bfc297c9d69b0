"""Autograd bindings of the sm_100a kernels in ``csrc/`` (library loaded by :mod:`pear_b200.ops.lib`).

Each op is a :class:`torch.autograd.Function` whose forward and backward launch the hand-written kernels on the current
stream. What still runs a library kernel is named where it happens: the backward GEMM forms of ``ops/gemm.py`` (cuBLAS),
the attention backward of ``ops/attention.py`` (FlashAttention-2), the chunk-local operands of the delta-rule scan (torch).
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import reference as ref
from .lib import check, count_launch, lib, on_device, ptr, stream

DT_F32, DT_BF16 = 0, 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _f32c(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


# ---------------------------------------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, one_plus, residual):
        shape = x.shape
        dim = shape[-1]
        on_device(x)
        xc = x.contiguous()
        if xc.dtype not in (torch.float32, torch.bfloat16):
            xc = xc.float()
        rows = xc.numel() // dim
        w = _f32c(weight)
        y = torch.empty(shape, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        res_in = _f32c(residual) if residual is not None else None
        res_out = torch.empty(shape, dtype=torch.float32, device=x.device) if residual is not None else None
        check(lib().pear_rms_norm_fwd(ptr(xc), _dt(xc), ptr(res_in), ptr(w), ptr(y), DT_F32, ptr(res_out), ptr(rstd),
                                      rows, dim, ctypes.c_float(eps), int(one_plus), stream()), "rms_norm_fwd")
        count_launch()
        normed_in = res_out if residual is not None else (xc if xc.dtype == torch.float32 else xc.float())
        ctx.save_for_backward(normed_in, w, rstd)
        ctx.one_plus, ctx.has_res, ctx.wdtype, ctx.xdtype = one_plus, residual is not None, weight.dtype, x.dtype
        if residual is not None:
            return y, res_out
        return y

    @staticmethod
    def backward(ctx, dy, dres=None):
        r, w, rstd = ctx.saved_tensors
        dim = r.shape[-1]
        rows = r.numel() // dim
        dyc = _f32c(dy) if dy is not None else torch.zeros_like(r)
        dresc = _f32c(dres) if (ctx.has_res and dres is not None) else None
        dx = torch.empty_like(r)
        dw = torch.zeros(dim, dtype=torch.float32, device=r.device)
        check(lib().pear_rms_norm_bwd(ptr(dyc), ptr(r), ptr(w), ptr(rstd), ptr(dresc), ptr(dx), ptr(dw), rows, dim,
                                      int(ctx.one_plus), stream()), "rms_norm_bwd")
        count_launch()
        dxo = dx.to(ctx.xdtype)
        return dxo, dw.to(ctx.wdtype), None, None, (dx if ctx.has_res else None)


def rms_norm(x, weight, eps=1e-6, one_plus=True):
    return _RMSNorm.apply(x, weight, eps, one_plus, None)


def add_rms_norm(x, residual, weight, eps=1e-6):
    return _RMSNorm.apply(x, weight, eps, True, residual)


# ---------------------------------------------------------------------------------------------------------------------
class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, z, weight, eps):
        oc, zc, w = _f32c(o), _f32c(z), _f32c(weight)
        dim = oc.shape[-1]
        rows = oc.numel() // dim
        y = torch.empty_like(oc)
        rstd = torch.empty(rows, dtype=torch.float32, device=o.device)
        check(lib().pear_gated_rms_norm_fwd(ptr(oc), ptr(zc), ptr(w), ptr(y), DT_F32, ptr(rstd), rows, dim,
                                            ctypes.c_float(eps), stream()), "gated_rms_norm_fwd")
        count_launch()
        ctx.save_for_backward(oc, zc, w, rstd)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        oc, zc, w, rstd = ctx.saved_tensors
        dim = oc.shape[-1]
        rows = oc.numel() // dim
        d_o, d_z = torch.empty_like(oc), torch.empty_like(zc)
        dw = torch.zeros(dim, dtype=torch.float32, device=oc.device)
        check(lib().pear_gated_rms_norm_bwd(ptr(_f32c(dy)), ptr(oc), ptr(zc), ptr(w), ptr(rstd), ptr(d_o), ptr(d_z), ptr(dw),
                                            rows, dim, stream()), "gated_rms_norm_bwd")
        count_launch()
        return d_o, d_z, dw.to(ctx.wdtype), None


def gated_rms_norm(o, z, weight, eps=1e-6):
    return _GatedRMSNorm.apply(o, z, weight, eps)


# ---------------------------------------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        g, u = _f32c(gate), _f32c(up)
        y = torch.empty_like(g)
        check(lib().pear_swiglu_fwd(ptr(g), ptr(u), ptr(y), DT_F32, ctypes.c_longlong(g.numel()), stream()), "swiglu_fwd")
        count_launch()
        ctx.save_for_backward(g, u)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dg, du = torch.empty_like(g), torch.empty_like(u)
        check(lib().pear_swiglu_bwd(ptr(_f32c(dy)), ptr(g), ptr(u), ptr(dg), ptr(du), ctypes.c_longlong(g.numel()), stream()),
              "swiglu_bwd")
        count_launch()
        return dg, du


def swiglu(gate, up):
    return _SwiGLU.apply(gate, up)


class _SigmoidGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate):
        xc, g = _f32c(x), _f32c(gate)
        y = torch.empty_like(xc)
        check(lib().pear_sigmoid_gate_fwd(ptr(xc), ptr(g), ptr(y), DT_F32, ctypes.c_longlong(xc.numel()), stream()), "gate_fwd")
        count_launch()
        ctx.save_for_backward(xc, g)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, g = ctx.saved_tensors
        dx, dg = torch.empty_like(xc), torch.empty_like(g)
        check(lib().pear_sigmoid_gate_bwd(ptr(_f32c(dy)), ptr(xc), ptr(g), ptr(dx), ptr(dg), ctypes.c_longlong(xc.numel()),
                                          stream()), "gate_bwd")
        count_launch()
        return dx, dg


def sigmoid_gate(x, gate):
    return _SigmoidGate.apply(x, gate)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        xc, c, s = _f32c(x), _f32c(cos), _f32c(sin)
        t, h, d = xc.shape
        y = torch.empty_like(xc)
        check(lib().pear_rope(ptr(xc), ptr(c), ptr(s), ptr(y), t, h, d, c.shape[-1], ctypes.c_float(1.0), stream()), "rope")
        count_launch()
        ctx.save_for_backward(c, s)
        return y

    @staticmethod
    def backward(ctx, dy):
        c, s = ctx.saved_tensors
        dyc = _f32c(dy)
        t, h, d = dyc.shape
        dx = torch.empty_like(dyc)
        check(lib().pear_rope(ptr(dyc), ptr(c), ptr(s), ptr(dx), t, h, d, c.shape[-1], ctypes.c_float(-1.0), stream()), "rope_bwd")
        count_launch()
        return dx, None, None


def apply_rope(x, cos, sin):
    return _Rope.apply(x, cos, sin)


# ---------------------------------------------------------------------------------------------------------------------
# GEMM: tcgen05 kernel when the shape qualifies, cuBLAS otherwise
# ---------------------------------------------------------------------------------------------------------------------
def linear_bf16(x: torch.Tensor, weight: torch.Tensor, output_unused: bool = False) -> torch.Tensor:
    from . import gemm

    return gemm.linear_bf16(x, weight, output_unused)


# ---------------------------------------------------------------------------------------------------------------------
# ops still on library kernels
# ---------------------------------------------------------------------------------------------------------------------
_CU_CACHE: dict = {}


def _cu_tensor(bounds: tuple, device) -> torch.Tensor:
    """Sequence boundaries as an int32 device tensor; the same boundaries recur for every layer and pass of a batch."""
    key = (bounds, str(device))
    t = _CU_CACHE.get(key)
    if t is None:
        if len(_CU_CACHE) >= 32:
            _CU_CACHE.pop(next(iter(_CU_CACHE)))
        host = torch.tensor(bounds, dtype=torch.int32)
        t = (host.pin_memory() if torch.cuda.is_available() else host).to(device, non_blocking=True)
        _CU_CACHE[key] = t
    return t


USE_TCGEN05_ATTENTION = True  # forward passes without gradients on a GPU, head dimension 256


def causal_attention(q, k, v, cu_seqlens, scale=None):
    """Packed causal attention; fp32 [T, Hq, D]. On a GPU at head dimension 256 the forward is the tcgen05 kernel of
    ``ops/attention.py`` on bf16 operands; with gradients the backward is the FlashAttention-2 library kernel fed with
    that forward's output and log-sum-exp (torch SDPA when the package is missing)."""
    if USE_TCGEN05_ATTENTION and q.is_cuda and q.shape[-1] == 256:
        from . import attention as A

        bounds = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
        cu = _cu_tensor(tuple(bounds), q.device)
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            if A.flash_attn_backward_available():  # own forward, library backward on its output and log-sum-exp
                longest = max(e - s for s, e in zip(bounds[:-1], bounds[1:]))
                return A.attention_varlen(q, k, v, cu, cu, longest, longest, True, scale).float()
            return ref.causal_attention(q, k, v, cu_seqlens, scale)
        record = A._RETAIN["mode"] == "record" and A.flash_attn_backward_available()
        res = A.attention_varlen_fwd(q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous(),
                                     v.to(torch.bfloat16).contiguous(), cu, cu, causal=True, scale=scale, return_lse=record)
        if record:  # first pass of a checkpointed layer: keep output and log-sum-exp for the recompute pass
            A._RETAIN["store"].append(res)
            return res[0].float()
        return res.float()
    return ref.causal_attention(q, k, v, cu_seqlens, scale)


def prefill_attention(q, k_all, v_all, scale=None):
    """One sequence's chunk of queries (its last positions) over all its keys so far: q [Tq, Hq, 256], k_all / v_all
    [Tk, Hkv, 256] -> fp32 [Tq, Hq, 256], through the tcgen05 kernel."""
    from . import attention as A

    cu_q = torch.tensor([0, q.shape[0]], dtype=torch.int32, device=q.device)
    cu_k = torch.tensor([0, k_all.shape[0]], dtype=torch.int32, device=q.device)
    o = A.attention_varlen_fwd(q.to(torch.bfloat16).contiguous(), k_all.to(torch.bfloat16).contiguous(),
                               v_all.to(torch.bfloat16).contiguous(), cu_q, cu_k, causal=True, scale=scale, return_lse=False)
    return o.float()


def causal_conv_silu(x, weight, bounds, init_state=None):
    return ref.causal_conv_silu(x, weight, bounds, init_state)


USE_SCAN_KERNEL = True  # the chunk-by-chunk loop of the delta-rule scan as one kernel launch on a GPU


def _chunk_loop(W, U, Qe, A, Kt, gamma, S0, E=None, want_o=True, want_hist=False, want_vp=False):
    """One launch of ``gdn_chunk_loop_kernel`` over [H, n, 64, *] operands; returns (O, S_out, S_hist, VP)."""
    hv, n, _, vd = U.shape
    dev = U.device
    c = lambda x: None if x is None else x.contiguous().float()
    W, U, Qe, A, Kt, gamma, S0, E = (c(x) for x in (W, U, Qe, A, Kt, gamma, S0, E))
    if not U.is_cuda:  # the kernel's statement in torch (CPU tests of the backward derivation)
        s = S0 if S0 is not None else U.new_zeros(hv, vd, W.shape[-1])
        outs, hists, vps = [], [], []
        for i in range(n):
            hists.append(s)
            vpi = U[:, i] - torch.einsum("hik,hvk->hiv", W[:, i], s)
            outs.append(torch.einsum("hik,hvk->hiv", Qe[:, i], s) + torch.einsum("hij,hjv->hiv", A[:, i], vpi))
            vps.append(vpi)
            s = s * gamma[:, i][:, None, None] + torch.einsum("hiv,hik->hvk", vpi, Kt[:, i])
            if E is not None:
                s = s + E[:, i]
        return (torch.stack(outs, 1) if want_o else None, s, torch.stack(hists, 1) if want_hist else None,
                torch.stack(vps, 1) if want_vp else None)
    o = torch.empty(hv, n, 64, vd, dtype=torch.float32, device=dev) if want_o else None
    s_out = torch.empty(hv, vd, 128, dtype=torch.float32, device=dev)
    hist = torch.empty(hv, n, vd, 128, dtype=torch.float32, device=dev) if want_hist else None
    vp = torch.empty(hv, n, 64, vd, dtype=torch.float32, device=dev) if want_vp else None
    check(lib().pear_gdn_chunk_loop(ptr(W), ptr(U), ptr(Qe), ptr(A), ptr(Kt), ptr(gamma), ptr(S0), ptr(E), ptr(o), ptr(s_out), ptr(hist),
                                    ptr(vp), hv, n, vd, stream()), "gdn_chunk_loop")
    count_launch()
    return o, s_out, hist, vp


class _ScanLoop(torch.autograd.Function):
    """``v' = U - W S^T; o = Qe S^T + A v'; S <- gamma S + v'^T Kt`` over the chunks of one sequence.

    Backward: with dS the gradient of the state after a chunk, ``dv' = A^T dO + Kt dS^T`` and
    ``dS_before = gamma dS + dO^T Qe - dv'^T W``: the same recurrence as the forward with W and Kt swapped,
    ``U' = -A^T dO`` and the additive term ``dO^T Qe``, run over the chunks in reverse by the same kernel; every other
    gradient is a batched product over all chunks at once of the saved states, v', dS and dv'."""

    @staticmethod
    def forward(ctx, W, U, Qe, A, Kt, gamma, S0):
        need = any(ctx.needs_input_grad)
        o, s_out, hist, vp = _chunk_loop(W, U, Qe, A, Kt, gamma, S0, want_hist=need, want_vp=need)
        if need:
            ctx.save_for_backward(W, Qe, A, Kt, gamma, hist, vp)
        ctx.has_s0 = S0 is not None
        return o, s_out

    @staticmethod
    def backward(ctx, dO, dS_out):
        W, Qe, A, Kt, gamma, hist, vp = ctx.saved_tensors
        dO = dO.contiguous().float()
        up = -torch.einsum("hnij,hniv->hnjv", A.float(), dO)
        e = torch.einsum("hniv,hnik->hnvk", dO, Qe.float())
        f = lambda x: x.flip(1)
        _, ds0, dhist_r, vp_r = _chunk_loop(f(Kt), f(up), f(Kt), f(A), f(W), f(gamma), dS_out, E=f(e), want_o=False, want_hist=True,
                                            want_vp=True)
        ds_next = f(dhist_r)      # gradient of the state AFTER chunk c
        dvp = -f(vp_r)
        dA = torch.einsum("hniv,hnjv->hnij", dO, vp)
        dQe = torch.einsum("hniv,hnvk->hnik", dO, hist)
        dKt = torch.einsum("hnjv,hnvk->hnjk", vp, ds_next)
        dW = -torch.einsum("hnjv,hnvk->hnjk", dvp, hist)
        dgamma = (ds_next * hist).sum((-1, -2))
        return dW, dvp, dQe, dA, dKt, dgamma, (ds0 if ctx.has_s0 else None)


def gdn_scan(q, k, v, g, beta, state=None):
    """Chunked delta-rule scan of one sequence. On a GPU the chunk-by-chunk loop (64 dependent steps of small products
    for 4096 tokens) is ONE launch of ``gdn_chunk_loop_kernel``, and its backward one more launch of the same kernel
    plus batched products; the chunk-local operands stay batched torch statements under autograd."""
    if (USE_SCAN_KERNEL and q.is_cuda and q.shape[2] == 128 and v.shape[2] % 32 == 0 and ref.GDN_CHUNK == 64 and q.shape[0] > 0):
        op = ref.gdn_chunk_operands(q, k, v, g, beta)
        hv, vd, n, t = v.shape[1], v.shape[2], op["n"], op["t"]
        s0 = state.float() if state is not None else None
        o, s_out = _ScanLoop.apply(op["W"], op["U"], op["Qe"], op["A"], op["Kt"], op["gamma"], s0)
        return o.permute(1, 2, 0, 3).reshape(n * 64, hv, vd)[:t], s_out
    return ref.gdn_chunked(q, k, v, g, beta, state)


def logprob_entropy(hidden, weight, ids, temperature=1.0, chunk=4096):
    return ref.logprob_entropy(hidden, weight, ids, temperature, chunk)

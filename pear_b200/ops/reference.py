"""Plain PyTorch fp32 statements of every hot op: the oracle each CUDA kernel is tested against, and the CPU path.

Math follows the upstream model family: (1+w) RMSNorm in fp32 with one rounding (``pear/models/qwen3_5/trainer/
rms_norm.py:140-143``), interleaved M-RoPE with NeoX pairing (``rollout/attention.py:27-71``), the gated delta rule
recurrence (``rollout/blackwell/gdn/kernels.py:131-181``), gated RMSNorm with a plain weight
(``gdn/kernels.py:275-278``), and the fp32 head's log-probs and entropy (``trainer/head.py:26-28, 77-78``).
All functions are differentiable through autograd unless stated otherwise.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

GDN_CHUNK = 64


# ---------------------------------------------------------------------------------------------------------------------
# norms and activations
# ---------------------------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, one_plus: bool = True) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * (1 + w)`` in fp32; returns fp32."""
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float()
    return xf * rstd * ((1.0 + w) if one_plus else w)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Residual add on the fp32 stream, then (1+w) RMSNorm. Returns ``(normed fp32, new residual fp32)``."""
    r = residual.float() + x.float()
    return rms_norm(r, weight, eps), r


def gated_rms_norm(o: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Per (token, head): ``o * rsqrt(mean(o^2) + eps) * w * silu(z)``; o, z: [..., D], weight: [D]."""
    of = o.float()
    rstd = torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    return of * rstd * weight.float() * F.silu(z.float())


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate.float()) * up.float()


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """Attention output gate ``x * sigmoid(gate)`` in fp32 (``trainer/attention.py:42-44``)."""
    return x.float() * torch.sigmoid(gate.float())


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)


# ---------------------------------------------------------------------------------------------------------------------
# interleaved M-RoPE
# ---------------------------------------------------------------------------------------------------------------------
def mrope_axis_of_frequency(rotary_dim: int, sections: tuple[int, int, int]) -> torch.Tensor:
    """Which of the (T, H, W) position rows frequency ``i`` reads: H if ``i % 3 == 1 and i < 3 * sections[1]``,
    W if ``i % 3 == 2 and i < 3 * sections[2]``, else T."""
    half = rotary_dim // 2
    i = torch.arange(half)
    axis = torch.zeros(half, dtype=torch.long)
    axis[(i % 3 == 1) & (i < 3 * sections[1])] = 1
    axis[(i % 3 == 2) & (i < 3 * sections[2])] = 2
    return axis


def mrope_cos_sin(position_ids: torch.Tensor, rotary_dim: int, theta: float, sections: tuple[int, int, int]):
    """``position_ids``: [3, T] (or [T] for text, broadcast to the three axes). Returns fp32 cos, sin of [T, rotary_dim/2]."""
    if position_ids.dim() == 1:
        position_ids = position_ids.unsqueeze(0).expand(3, -1)
    half = rotary_dim // 2
    inv_freq = theta ** (-torch.arange(half, dtype=torch.float64, device=position_ids.device) * 2.0 / rotary_dim)
    axis = mrope_axis_of_frequency(rotary_dim, sections).to(position_ids.device)
    pos = position_ids.to(torch.float64)[axis, :].transpose(0, 1)  # [T, half]: per frequency its axis' position
    ang = pos * inv_freq
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate the first ``2 * cos.shape[-1]`` channels of x [T, H, D], pairing channel i with i + rotary_dim/2."""
    half = cos.shape[-1]
    xf = x.float()
    x1, x2, rest = xf[..., :half], xf[..., half : 2 * half], xf[..., 2 * half :]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


# ---------------------------------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------------------------------
def seq_bounds(cu_seqlens) -> list[tuple[int, int]]:
    cs = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    return [(cs[i], cs[i + 1]) for i in range(len(cs) - 1)]


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens, scale: float | None = None):
    """Packed causal GQA attention. q: [T, Hq, D], k, v: [T, Hkv, D]; returns fp32 [T, Hq, D]."""
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    outs = []
    for s, e in seq_bounds(cu_seqlens):
        qs = q[s:e].float().transpose(0, 1).unsqueeze(0)
        ks = k[s:e].float().transpose(0, 1).unsqueeze(0)
        vs = v[s:e].float().transpose(0, 1).unsqueeze(0)
        o = F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=scale, enable_gqa=True)
        outs.append(o.squeeze(0).transpose(0, 1))
    out = torch.cat(outs, dim=0) if outs else out
    return out


def attention_with_cache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, q_start: int, scale: float):
    """q: [Tq, Hq, D] at absolute positions q_start..; k_cache, v_cache: [Tk, Hkv, D] positions 0..Tk-1 (Tk = q_start+Tq)."""
    tq, tk = q.shape[0], k_cache.shape[0]
    group = q.shape[1] // k_cache.shape[1]
    kk = k_cache.float().repeat_interleave(group, dim=1)
    vv = v_cache.float().repeat_interleave(group, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    qpos = torch.arange(q_start, q_start + tq, device=q.device)[:, None]
    kpos = torch.arange(tk, device=q.device)[None, :]
    s = s.masked_fill(kpos > qpos, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vv)


# ---------------------------------------------------------------------------------------------------------------------
# gated delta net
# ---------------------------------------------------------------------------------------------------------------------
def causal_conv_silu(x: torch.Tensor, weight: torch.Tensor, cu_seqlens=None, init_state: torch.Tensor | None = None):
    """Depthwise causal conv (no bias) + SiLU over packed sequences; never reads across a sequence boundary.

    x: [T, C]; weight: [C, W]; init_state: [num_seqs, W-1, C] rows preceding each sequence (zeros when None).
    ``u_t = silu(sum_j w[c, j] * x[t - (W-1) + j, c])``. Returns (y fp32 [T, C], final_state [num_seqs, W-1, C]).
    """
    t, c = x.shape
    w = weight.shape[1]
    bounds = seq_bounds(cu_seqlens) if cu_seqlens is not None else [(0, t)]
    ys, finals = [], []
    xf, wf = x.float(), weight.float()
    for i, (s, e) in enumerate(bounds):
        head = init_state[i].float() if init_state is not None else xf.new_zeros(w - 1, c)
        ext = torch.cat([head, xf[s:e]], dim=0)  # [L + W-1, C]
        acc = sum(ext[j : j + (e - s)] * wf[:, j] for j in range(w))
        ys.append(F.silu(acc))
        finals.append(ext[ext.shape[0] - (w - 1) :])
    return torch.cat(ys, dim=0), torch.stack(finals, dim=0)


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (log decay, <= 0) and ``beta = sigmoid(b)``; fp32."""
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float(), threshold=20.0)
    return g, torch.sigmoid(b.float())


def gdn_recurrent(q, k, v, g, beta, state: torch.Tensor | None = None):
    """Token-by-token gated delta rule for ONE sequence.

    q, k: [T, Hk, K] (already L2-normalised, q scaled by K^-0.5); v: [T, Hv, V]; g, beta: [T, Hv];
    state: [Hv, V, K] fp32. ``S <- S exp(g); u = (v - S k) beta; S <- S + u k^T; o = S q``.
    """
    t, hk, kd = q.shape
    hv, vd = v.shape[1], v.shape[2]
    rep = hv // hk
    qf = q.float().repeat_interleave(rep, dim=1)
    kf = k.float().repeat_interleave(rep, dim=1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    s = state.float().clone() if state is not None else qf.new_zeros(hv, vd, kd)
    outs = []
    for i in range(t):
        s = s * torch.exp(gf[i])[:, None, None]
        u = (vf[i] - torch.einsum("hvk,hk->hv", s, kf[i])) * bf[i][:, None]
        s = s + u[:, :, None] * kf[i][:, None, :]
        outs.append(torch.einsum("hvk,hk->hv", s, qf[i]))
    return torch.stack(outs, dim=0) if outs else vf.new_zeros(0, hv, vd), s


def gdn_chunk_operands(q, k, v, g, beta, chunk: int = GDN_CHUNK):
    """The chunk-local operands of the chunked (WY) form, computed for all chunks in parallel: per chunk with in-chunk
    cumulative log decay G: ``L_ij = beta_i (k_i.k_j) exp(G_i - G_j)`` for i > j, ``T = (I + L)^-1``,
    ``W = T (beta k e^G)``, ``U = T (beta v)``, ``Qe = q e^G``, ``A = tril((q k^T) * e^(G_i - G_j))``,
    ``Kt = k e^(G_C - G)``, ``gamma = e^(G_C)``. All fp32, shapes [Hv, n, C, *] (gamma [Hv, n])."""
    t, hk, kd = q.shape
    hv, vd = v.shape[1], v.shape[2]
    rep = hv // hk
    pad = (-t) % chunk
    n = (t + pad) // chunk

    def prep(x):
        x = x.float()
        if pad:
            x = torch.cat([x, x.new_zeros((pad,) + x.shape[1:])], dim=0)
        return x

    # q and k stay at their own head count: the value heads of a group share them, so the products over the key
    # dimension are taken once per q/k head and every per-value-head factor is applied by broadcasting
    qf, kf = prep(q), prep(k)  # [Tp, Hk, K]
    vf, gf, bf = prep(v), prep(g), prep(beta)  # padding: g = 0, beta = 0, k = 0 -> no state change
    qc = qf.view(n, chunk, hk, kd).permute(2, 0, 1, 3)  # [Hk, n, C, K]
    kc = kf.view(n, chunk, hk, kd).permute(2, 0, 1, 3)
    vc = vf.view(n, chunk, hv, vd).permute(2, 0, 1, 3)  # [Hv, n, C, V]
    gc = gf.view(n, chunk, hv).permute(2, 0, 1)
    bc = bf.view(n, chunk, hv).permute(2, 0, 1)
    G = gc.cumsum(-1)  # [Hv, n, C]
    diff = G[..., :, None] - G[..., None, :]  # G_i - G_j
    idx = torch.arange(chunk, device=q.device)
    lower_strict = (idx[:, None] > idx[None, :])
    lower = (idx[:, None] >= idx[None, :])
    decay = torch.exp(diff.masked_fill(~lower, 0.0)) * lower  # exp only where i >= j

    def per_value_head(x_hk, scale_hv):
        """x_hk [Hk, n, C, D] times a per-value-head factor [Hv, n, C] -> [Hv, n, C, D] without a repeated copy of x."""
        return (x_hk[:, None] * scale_hv.reshape(hk, rep, n, chunk, 1)).reshape(hv, n, chunk, x_hk.shape[-1])

    def spread(m_hk):
        """[Hk, n, C, C] -> a [Hv, n, C, C] view-like expansion (small: C x C per chunk)."""
        return m_hk[:, None].expand(hk, rep, n, chunk, chunk).reshape(hv, n, chunk, chunk)

    kk = spread(torch.einsum("hnik,hnjk->hnij", kc, kc))
    L = bc[..., :, None] * kk * decay * lower_strict
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    eG = torch.exp(G)
    rhs = torch.cat([per_value_head(kc, bc * eG), bc[..., None] * vc], dim=-1)  # [Hv, n, C, K+V]
    WU = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
    W, U = WU[..., :kd], WU[..., kd:]
    qk = spread(torch.einsum("hnik,hnjk->hnij", qc, kc)) * decay
    G_last = G[..., -1]
    k_tail = per_value_head(kc, torch.exp(G_last[..., None] - G))  # k e^(G_C - G)
    Qe = per_value_head(qc, eG)
    return {"W": W, "U": U, "Qe": Qe, "A": qk, "Kt": k_tail, "gamma": torch.exp(G_last), "n": n, "t": t}


def gdn_chunked(q, k, v, g, beta, state: torch.Tensor | None = None, chunk: int = GDN_CHUNK):
    """Chunked (WY) form of :func:`gdn_recurrent` for ONE sequence; same shapes, same result up to rounding.

    With the operands of :func:`gdn_chunk_operands`, chunk by chunk: ``v' = U - W S0^T``,
    ``o = Qe S0^T + A v'``, ``S1 = gamma S0 + v'^T Kt``.
    """
    hv, vd, kd = v.shape[1], v.shape[2], q.shape[2]
    op = gdn_chunk_operands(q, k, v, g, beta, chunk)
    n, t = op["n"], op["t"]
    s = state.float() if state is not None else q.new_zeros(hv, vd, kd, dtype=torch.float32)
    outs = []
    for c in range(n):
        v_new = op["U"][:, c] - torch.einsum("hik,hvk->hiv", op["W"][:, c], s)
        o = torch.einsum("hik,hvk->hiv", op["Qe"][:, c], s) + torch.einsum("hij,hjv->hiv", op["A"][:, c], v_new)
        s = s * op["gamma"][:, c][:, None, None] + torch.einsum("hiv,hik->hvk", v_new, op["Kt"][:, c])
        outs.append(o)
    o = torch.stack(outs, dim=1).permute(1, 2, 0, 3).reshape(n * chunk, hv, vd)[:t]
    return o, s


def gdn_span_summary(k, g, beta, chunk: int = GDN_CHUNK):
    """Transition of a token span on an incoming state: ``S_out = S_in M + H`` with M: [Hv, K, K] (right-multiplied on
    the K axis) and H the span's final state from a zero start. Returns M only (H comes from the scan itself).

    Used by context parallelism: each rank publishes (H, M) of its slice and the ranks fold ``X <- X M + H`` left to
    right (upstream ``trainer/blackwell/delta_rule.py:51-89``).
    """
    t, hk, kd = k.shape
    hv = g.shape[1]
    rep = hv // hk
    kf = k.float().repeat_interleave(rep, dim=1)
    m = torch.eye(kd, device=k.device, dtype=torch.float32).expand(hv, kd, kd).clone()
    gf, bf = g.float(), beta.float()
    for i in range(t):
        # S <- a S - b (a S k) k^T  = S (a (I - b k k^T))
        a = torch.exp(gf[i])[:, None, None]
        kk = kf[i][:, :, None] * kf[i][:, None, :]
        step = a * (torch.eye(kd, device=k.device) - bf[i][:, None, None] * kk)
        m = torch.bmm(m, step)
    return m


# ---------------------------------------------------------------------------------------------------------------------
# head: log-probs at ids, entropy, without keeping logits
# ---------------------------------------------------------------------------------------------------------------------
class _LogProbEntropy(torch.autograd.Function):
    """Rows are processed in chunks; only lse per row is saved, logits are recomputed per chunk in backward."""

    @staticmethod
    def _kernels(hidden, weight):
        """On a GPU the three GEMMs of the head run on the tcgen05 kernel: logits with split operands (close to fp32),
        the two gradient products with bf16 operands and fp32 accumulation."""
        if not hidden.is_cuda or weight.shape[1] % 8:
            return None
        from . import gemm, lib

        return gemm if lib.available() else None

    @staticmethod
    def forward(ctx, hidden, weight, ids, inv_temperature, chunk):
        n = hidden.shape[0]
        lp = torch.empty(ids.shape, dtype=torch.float32, device=hidden.device)
        ent = torch.empty(n, dtype=torch.float32, device=hidden.device)
        lse = torch.empty(n, dtype=torch.float32, device=hidden.device)
        g = _LogProbEntropy._kernels(hidden, weight)
        wf = weight.float() if g is None else None
        ws = g.split_operand(weight, "b") if g is not None else None
        for s in range(0, n, chunk):
            e = min(s + chunk, n)
            logits = (hidden[s:e].float() @ wf.t()) if g is None else g.matmul_split3(hidden[s:e], weight, ws)
            logits = logits.mul_(inv_temperature)
            l = torch.logsumexp(logits, dim=-1)
            logp = logits.sub_(l[:, None])
            lp[s:e] = logp.gather(-1, ids[s:e])
            ent[s:e] = -(logp.exp() * logp).sum(-1)
            lse[s:e] = l
        ctx.save_for_backward(hidden, weight, ids, lse, ent)
        ctx.inv_temperature, ctx.chunk = inv_temperature, chunk
        return lp, ent

    @staticmethod
    def backward(ctx, g_lp, g_ent):
        hidden, weight, ids, lse, ent = ctx.saved_tensors
        n = hidden.shape[0]
        g = _LogProbEntropy._kernels(hidden, weight)
        wf = weight.float() if g is None else None
        g_hidden = torch.zeros(hidden.shape, dtype=torch.float32, device=hidden.device)
        g_weight = torch.zeros(weight.shape, dtype=torch.float32, device=hidden.device)
        if g is not None:
            ws = g.split_operand(weight, "b")
            wt = weight.to(torch.bfloat16).t().contiguous()  # [K, V]: the contraction of d @ W runs over V
        for s in range(0, n, ctx.chunk):
            e = min(s + ctx.chunk, n)
            hf = hidden[s:e].float()
            logits = (hf @ wf.t()) if g is None else g.matmul_split3(hf, weight, ws)
            logp = logits.mul_(ctx.inv_temperature).sub_(lse[s:e, None])
            p = logp.exp()
            glp = g_lp[s:e].float()
            d = -p * glp.sum(-1, keepdim=True)
            d.scatter_add_(-1, ids[s:e], glp)
            if g_ent is not None:
                d = d - g_ent[s:e, None].float() * p * (logp + ent[s:e, None])
            d = d * ctx.inv_temperature
            if g is None or (e - s) % 8:
                g_hidden[s:e] = d @ (wf if wf is not None else weight.float())
                g_weight += d.t() @ hf
            else:
                db = d.to(torch.bfloat16)
                g.gemm_nt(db, wt, torch.float32, out=g_hidden[s:e])
                g_weight += g.gemm_nt(db.t().contiguous(), hf.to(torch.bfloat16).t().contiguous(), torch.float32)
        return g_hidden.to(hidden.dtype), g_weight.to(weight.dtype), None, None, None


def logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor, temperature: float = 1.0,
                    chunk: int = 4096):
    """``log_softmax(hidden @ weight^T / T)`` gathered at ``ids`` [N, k] and the entropy per row, in fp32.

    Returns (log_probs [N, k], entropy [N]). Logits exist only one ``chunk`` of rows at a time.
    """
    return _LogProbEntropy.apply(hidden, weight, ids.long(), 1.0 / temperature, chunk)


def logprob_entropy_dense(hidden, weight, ids, temperature: float = 1.0):
    """Unfused statement of :func:`logprob_entropy` (materialises all logits); test oracle."""
    logits = hidden.float() @ weight.float().t() / temperature
    logp = torch.log_softmax(logits, dim=-1)
    return logp.gather(-1, ids.long()), -(logp.exp() * logp).sum(-1)


# ---------------------------------------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------------------------------------
def sample_exponential_race(logits: torch.Tensor, temperature: float, noise_u: torch.Tensor, topk: int = 32):
    """Temperature-only sampling ``argmax(logits / T - log(-log u))`` with the top-k processed log-probs.

    Returns (token [N], logprob of token [N], topk ids [N, k], topk log-probs [N, k], rank of token [N],
    count of non-finite logits [N]). The statement of upstream ``rollout/blackwell/csrc/sampler.cu``.
    """
    z = logits.float() / temperature
    nonfinite = (~torch.isfinite(z) & ~(z == float("-inf"))).sum(-1)
    logp = torch.log_softmax(z, dim=-1)
    gumbel = -torch.log(-torch.log(noise_u.clamp(1e-20, 1.0 - 1e-7)))
    tok = torch.argmax(z + gumbel, dim=-1)
    tok_lp = logp.gather(-1, tok[:, None]).squeeze(-1)
    top_lp, top_id = torch.topk(logp, min(topk, logp.shape[-1]), dim=-1)
    rank = (logp >= tok_lp[:, None]).sum(-1)
    return tok, tok_lp, top_id, top_lp, rank, nonfinite


def softmax_entropy_from_logits(logits: torch.Tensor) -> torch.Tensor:
    logp = torch.log_softmax(logits.float(), dim=-1)
    return -(logp.exp() * logp).sum(-1)


def log_of(x: float) -> float:
    return math.log(x)

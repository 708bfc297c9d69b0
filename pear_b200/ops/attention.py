"""Variable-length causal attention forward on the tcgen05 tensor cores (``csrc/attn_tcgen05.cu``).

``attention_varlen_fwd`` takes packed rows ``q [Tq, Hq, 256]``, ``k, v [Tk, Hkv, 256]`` (bf16, any row stride that is a
multiple of 8 elements, heads contiguous) and the int32 row offsets of the sequences. In every sequence the queries are
the last positions of the keys (``len_k >= len_q``: plain causal self-attention when equal, a prefill chunk over cached
keys when longer). Returns ``o [Tq, Hq, 256]`` bf16 and the log-sum-exp ``[Hq, Tq]`` fp32.

``attention_varlen_reference`` is the plain fp32 PyTorch statement of the same op that the tests compare against.
(Upstream: FlashAttention-4 forward in pear/models/qwen3_5/trainer/blackwell/ulysses_attention.py:144 and the context
FMHA of the rollout engine.)

``python -m pear_b200.ops.attention T [--seqs B] [--heads 24] [--kv-heads 4] [--iters N]`` times the kernel with CUDA
events and prints one JSON line.
"""

from __future__ import annotations

import math

import torch

from . import lib as _lib

HEAD_DIM = 256
_status: dict = {}


def _status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def attention_status(device=None) -> int:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status_word(dev).item())


def _row_stride(x: torch.Tensor) -> int:
    if x.dim() != 3 or x.shape[2] != HEAD_DIM or x.stride(2) != 1 or x.stride(1) != HEAD_DIM:
        raise ValueError("expected [rows, heads, 256] with contiguous heads")
    return x.stride(0)


def attention_varlen_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor,
                         causal: bool = True, scale: float | None = None, return_lse: bool = True):
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("attention_varlen_fwd takes bf16 operands")
    tq, hq, _ = q.shape
    tk, hkv, _ = k.shape
    batch = cu_q.numel() - 1
    if cu_q.dtype != torch.int32 or cu_k.dtype != torch.int32 or cu_k.numel() != cu_q.numel():
        raise TypeError("cu_q / cu_k: int32 tensors of batch + 1 row offsets")
    out = torch.empty(tq, hq, HEAD_DIM, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(hq, tq, dtype=torch.float32, device=q.device) if return_lse else None
    scale = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
    import ctypes

    _lib.check(_lib.lib().pear_attn_varlen_fwd_hd256(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(cu_q), _lib.ptr(cu_k), batch, tq, tk, hq, hkv,
        _row_stride(q), _row_stride(k), _row_stride(v), out.stride(0), ctypes.c_float(scale), 1 if causal else 0,
        _lib.ptr(_status_word(q.device)), _lib.stream()), "attn_varlen_fwd")
    _lib.count_launch()
    return (out, lse) if return_lse else out


# Retained attention outputs of a checkpointed layer (upstream verl patch 0026): the graph-free first pass RECORDS the
# output and log-sum-exp of every attention call of the layer, the recompute pass of the backward REPLAYS them instead of
# running the forward kernel again (q, k, v are recomputed by the projections either way).
_RETAIN: dict = {"mode": None, "store": None}


class retain_attention:
    """``with retain_attention("record", box)`` / ``with retain_attention("replay", box)``; ``box`` is a list owned by
    the caller (one per checkpointed layer call)."""

    def __init__(self, mode: str, box: list):
        self.mode, self.box = mode, box

    def __enter__(self):
        self.prev = dict(_RETAIN)
        _RETAIN["mode"], _RETAIN["store"] = self.mode, self.box
        return self.box

    def __exit__(self, *exc):
        _RETAIN.update(self.prev)


class _AttnVarlen(torch.autograd.Function):
    """Forward on the tcgen05 kernel; backward through the FlashAttention-2 library kernel of the ``flash_attn`` package,
    fed with this forward's output and log-sum-exp (no own backward kernel yet)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, causal, scale):
        qb, kb, vb = (x.to(torch.bfloat16).contiguous() for x in (q, k, v))
        if _RETAIN["mode"] == "replay" and _RETAIN["store"]:
            o, lse = _RETAIN["store"].pop(0)
        else:
            o, lse = attention_varlen_fwd(qb, kb, vb, cu_q, cu_k, causal=causal, scale=scale)
        ctx.save_for_backward(qb, kb, vb, o, lse, cu_q, cu_k)
        ctx.args = (max_q, max_k, causal, scale, q.dtype, k.dtype, v.dtype)
        return o

    @staticmethod
    def backward(ctx, do):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        qb, kb, vb, o, lse, cu_q, cu_k = ctx.saved_tensors
        max_q, max_k, causal, scale, dq_t, dk_t, dv_t = ctx.args
        dq, dk, dv = torch.empty_like(qb), torch.empty_like(kb), torch.empty_like(vb)
        _flash_attn_varlen_backward(do.to(torch.bfloat16).contiguous(), qb, kb, vb, o, lse, dq, dk, dv, cu_q, cu_k, max_q, max_k, 0.0,
                                    scale, causal, -1, -1, 0.0, None, False)
        return dq.to(dq_t), dk.to(dk_t), dv.to(dv_t), None, None, None, None, None, None


def flash_attn_backward_available() -> bool:
    try:
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward  # noqa: F401

        return True
    except Exception:
        return False


def attention_varlen(q, k, v, cu_q, cu_k, max_q: int, max_k: int, causal: bool = True, scale: float | None = None) -> torch.Tensor:
    """Differentiable packed attention, head dimension 256: bf16 output [Tq, Hq, 256]."""
    scale = 1.0 / math.sqrt(HEAD_DIM) if scale is None else float(scale)
    return _AttnVarlen.apply(q, k, v, cu_q, cu_k, int(max_q), int(max_k), bool(causal), scale)


def attention_varlen_reference(q, k, v, cu_q, cu_k, causal: bool = True, scale: float | None = None):
    """fp32 PyTorch oracle: per sequence, per head, masked softmax(q k^T * scale) v; returns (o fp32, lse fp32 [Hq, Tq])."""
    tq, hq, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    o = torch.zeros(tq, hq, d, dtype=torch.float32, device=q.device)
    lse = torch.zeros(hq, tq, dtype=torch.float32, device=q.device)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(len(cq) - 1):
        qs = q[cq[b]:cq[b + 1]].float().transpose(0, 1)  # [Hq, lq, d]
        ks = k[ck[b]:ck[b + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[ck[b]:ck[b + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        lq, lk = qs.shape[1], ks.shape[1]
        s = torch.einsum("hid,hjd->hij", qs, ks) * scale
        if causal:
            i = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
            j = torch.arange(lk, device=q.device)[None, :]
            s = s.masked_fill(j > i, float("-inf"))
        lse[:, cq[b]:cq[b + 1]] = torch.logsumexp(s, dim=-1)
        o[cq[b]:cq[b + 1]] = torch.einsum("hij,hjd->hid", torch.softmax(s, dim=-1), vs).transpose(0, 1)
    return o, lse


def _main() -> None:
    import argparse
    import json

    ap = argparse.ArgumentParser()
    ap.add_argument("tokens", type=int)
    ap.add_argument("--seqs", type=int, default=1)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--compare", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    per = a.tokens // a.seqs
    cu = torch.arange(0, a.seqs + 1, dtype=torch.int32, device=dev) * per
    t = per * a.seqs
    q = torch.randn(t, a.heads, HEAD_DIM, device=dev, dtype=torch.bfloat16)
    k = torch.randn(t, a.kv_heads, HEAD_DIM, device=dev, dtype=torch.bfloat16)
    v = torch.randn(t, a.kv_heads, HEAD_DIM, device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        o, lse = attention_varlen_fwd(q, k, v, cu, cu)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        attention_varlen_fwd(q, k, v, cu, cu)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    flops = 4.0 * a.heads * HEAD_DIM * a.seqs * per * (per + 1) / 2
    rec = {"op": "attn_varlen_fwd_hd256", "tokens": t, "seqs": a.seqs, "heads": a.heads, "kv_heads": a.kv_heads, "ms": round(ms, 4),
           "tflops_causal": round(flops / ms / 1e9, 1), "status": attention_status()}
    if a.compare:  # the library call this kernel replaces: torch SDPA on the same bf16 operands, one call per sequence
        import torch.nn.functional as F

        def lib_call():
            for b in range(a.seqs):
                sl = slice(b * per, (b + 1) * per)
                F.scaled_dot_product_attention(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None], v[sl].transpose(0, 1)[None],
                                               is_causal=True, enable_gqa=True)

        for _ in range(3):
            lib_call()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.iters):
            lib_call()
        e1.record()
        torch.cuda.synchronize()
        rec["sdpa_ms"] = round(e0.elapsed_time(e1) / a.iters, 4)
    if a.check:
        ro, rl = attention_varlen_reference(q, k, v, cu, cu)
        rec["max_abs_err_o"] = float((o.float() - ro).abs().max())
        rec["max_abs_err_lse"] = float((lse - rl).abs().max())
    print(json.dumps(rec))


if __name__ == "__main__":
    _main()

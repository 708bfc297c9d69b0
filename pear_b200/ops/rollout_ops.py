"""Python bindings of the stand-alone rollout kernels (``csrc/rollout_kernels.cu``): fused sampler, rejection sampler of
greedy drafts, GDN decode step, split-KV paged attention, embedding merge, paged-KV block gather/scatter."""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import lib as _lib

_f = ctypes.c_float


def fused_sample(logits: torch.Tensor, temperature: float, noise_u: torch.Tensor, topk: int = 32, chunks: int = 0):
    """Returns (token, logprob, topk ids, topk log-probs, rank, nonfinite count) per row; see ``reference.sample_exponential_race``."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and noise_u.is_contiguous()
    rows, v = logits.shape
    if chunks <= 0:
        chunks = max(1, min(64, (2 * 148 + rows - 1) // rows))
    dev = logits.device
    ws = torch.empty(_lib.lib().pear_sample_workspace_bytes(rows, chunks), dtype=torch.uint8, device=dev)
    tok = torch.empty(rows, dtype=torch.int32, device=dev)
    lp = torch.empty(rows, dtype=torch.float32, device=dev)
    tid = torch.empty(rows, topk, dtype=torch.int32, device=dev)
    tlp = torch.empty(rows, topk, dtype=torch.float32, device=dev)
    rank = torch.empty(rows, dtype=torch.int32, device=dev)
    nf = torch.empty(rows, dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().pear_fused_sample(_lib.ptr(logits), rows, v, logits.stride(0), _f(temperature), _lib.ptr(noise_u), chunks, topk,
                                            _lib.ptr(ws), _lib.ptr(tok), _lib.ptr(lp), _lib.ptr(tid), _lib.ptr(tlp), _lib.ptr(rank), _lib.ptr(nf),
                                            _lib.stream()), "fused_sample")
    _lib.count_launch(2)
    return tok.long(), lp, tid.long(), tlp, rank.long(), nf.long()


def verify_greedy(logits: torch.Tensor, drafts: torch.Tensor, temperature: float, accept_u: torch.Tensor, noise_u: torch.Tensor):
    """logits [requests, n_draft + 1, V]; drafts [requests, n_draft]. Returns (tokens [requests, n_draft + 1] with -1 after the
    stop, accepted count per request, log-probs)."""
    r, rows, v = logits.shape
    n = rows - 1
    logits = logits.contiguous()
    dev = logits.device
    out = torch.empty(r, rows, dtype=torch.int32, device=dev)
    acc = torch.empty(r, dtype=torch.int32, device=dev)
    lp = torch.zeros(r, rows, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().pear_verify_greedy(_lib.ptr(logits), r, n, v, v, _f(temperature), _lib.ptr(drafts.int().contiguous()),
                                             _lib.ptr(accept_u.contiguous()), _lib.ptr(noise_u.contiguous()), _lib.ptr(out), _lib.ptr(acc),
                                             _lib.ptr(lp), _lib.stream()), "verify_greedy")
    _lib.count_launch(1)
    return out.long(), acc.long(), lp


def gdn_decode(x, z, a, b, conv_w, A_log, dt_bias, norm_w, conv_state, state, slots, hk: int, hv: int, l2_eps=1e-6, rms_eps=1e-6):
    """One decode token per sequence; updates ``conv_state`` [slots, 3, C] and ``state`` [slots, Hv, 128, 128] in place."""
    batch = x.shape[0]
    _lib.on_device(x)
    _lib.expect(torch.float32, x=x, z=z, a=a, b=b, conv_w=conv_w, A_log=A_log, dt_bias=dt_bias, norm_w=norm_w, conv_state=conv_state, state=state)
    out = torch.empty(batch, hv * 128, dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().pear_gdn_decode(_lib.ptr(x), _lib.ptr(z), _lib.ptr(a), _lib.ptr(b), _lib.ptr(conv_w), _lib.ptr(A_log), _lib.ptr(dt_bias),
                                          _lib.ptr(norm_w), _lib.ptr(conv_state), _lib.ptr(state), _lib.ptr(slots.int()), _lib.ptr(out), batch, hk, hv,
                                          _f(l2_eps), _f(rms_eps), _lib.stream()), "gdn_decode")
    _lib.count_launch(2)
    return out


def paged_attention(q, k_cache, v_cache, block_table, ctx_len, scale: float, nsplit: int = 0):
    """q [rows, Hq, D] fp32; caches [blocks, 16, Hkv, D] bf16; block_table [rows, max_blocks] int32; ctx_len [rows] int32."""
    rows, hq, d = q.shape
    hkv = k_cache.shape[2]
    q = q.contiguous()
    _lib.expect(torch.float32, q=q)
    _lib.expect(torch.bfloat16, k_cache=k_cache, v_cache=v_cache)
    if nsplit <= 0:
        nsplit = max(1, min(32, (2 * 148) // max(1, rows * hkv)))
    dev = q.device
    part_o = torch.empty(rows * hq * nsplit * d, dtype=torch.float32, device=dev)
    part_ml = torch.empty(rows * hq * nsplit * 2, dtype=torch.float32, device=dev)
    out = torch.empty(rows, hq, d, dtype=torch.float32, device=dev)
    _lib.check(_lib.lib().pear_paged_attention(_lib.ptr(q.contiguous()), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(block_table.int().contiguous()),
                                               block_table.shape[1], _lib.ptr(ctx_len.int().contiguous()), rows, hq, hkv, d, _f(scale), nsplit,
                                               _lib.ptr(part_o), _lib.ptr(part_ml), _lib.ptr(out), _lib.stream()), "paged_attention")
    _lib.count_launch(2)
    return out


def top_p_mask_(logits: torch.Tensor, top_p: torch.Tensor, temperature: float = 1.0, iters: int = 18) -> torch.Tensor:
    """In place: every token outside the row's nucleus (smallest set of tokens of softmax(logits / temperature) whose mass
    reaches ``top_p[row]``; ties with the pivot are kept) becomes -inf. ``logits`` fp32 [rows, V] with unit inner stride."""
    _lib.on_device(logits)
    _lib.expect(torch.float32, False, logits=logits)
    _lib.expect(torch.float32, top_p=top_p)
    assert logits.dim() == 2 and logits.stride(1) == 1 and top_p.numel() == logits.shape[0]
    import ctypes

    _lib.check(_lib.lib().pear_top_p_mask(_lib.ptr(logits), ctypes.c_longlong(logits.stride(0)), logits.shape[0], logits.shape[1], _f(temperature),
                                          _lib.ptr(top_p), iters, _lib.stream()), "top_p_mask")
    _lib.count_launch(1)
    return logits


def embed_merge(ids: torch.Tensor, table: torch.Tensor, embeds: Optional[torch.Tensor] = None, mask: Optional[torch.Tensor] = None):
    t, (v, h) = ids.shape[0], table.shape
    _lib.on_device(table)
    _lib.expect(torch.bfloat16, table=table)
    out = torch.empty(t, h, dtype=torch.float32, device=ids.device)
    m = mask.to(torch.uint8).contiguous() if mask is not None else None
    _lib.check(_lib.lib().pear_embed_merge(_lib.ptr(ids.int().contiguous()), _lib.ptr(table), _lib.ptr(embeds.float().contiguous() if embeds is not None else None),
                                           _lib.ptr(m), _lib.ptr(out), t, h, v, _lib.stream()), "embed_merge")
    _lib.count_launch(1)
    return out


def kv_blocks_copy(cache: torch.Tensor, staging: torch.Tensor, block_ids: torch.Tensor, to_staging: bool) -> None:
    """cache [blocks, ...] and staging [n, ...] with equal per-block byte size (a multiple of 16)."""
    n = block_ids.numel()
    bb = cache[0].numel() * cache.element_size()
    assert staging[0].numel() * staging.element_size() == bb and staging.shape[0] >= n
    _lib.check(_lib.lib().pear_kv_blocks_copy(_lib.ptr(cache), _lib.ptr(staging), _lib.ptr(block_ids.int().contiguous()), n, bb, 1 if to_staging else 0,
                                              _lib.stream()), "kv_blocks_copy")
    _lib.count_launch(1)


def logprob_entropy_fused(hidden: torch.Tensor, weight: torch.Tensor, ids: torch.Tensor, temperature: float = 1.0,
                          row_chunk: int = 1024, vocab_chunk: int = 16384):
    """Forward of the fused head: log-probs at ``ids`` [T, J] and the entropy per row, with the logits produced chunk by
    chunk by the tcgen05 GEMM ([row_chunk, vocab_chunk] fp32, sized to stay in L2) and folded into running softmax
    statistics; the full [T, V] logits never exist. ``hidden`` [T, H], ``weight`` [V, H] (cast to bf16 operands)."""
    from .gemm import gemm_nt

    t, h = hidden.shape
    v = weight.shape[0]
    j = ids.shape[1]
    dev = hidden.device
    hb = hidden.to(torch.bfloat16).contiguous()
    wb = weight.to(torch.bfloat16).contiguous()
    ids32 = ids.int().contiguous()
    lp = torch.empty(t, j, dtype=torch.float32, device=dev)
    ent = torch.empty(t, dtype=torch.float32, device=dev)
    lib = _lib.lib()
    buf = torch.empty(min(row_chunk, t), min(vocab_chunk, v), dtype=torch.float32, device=dev)
    for r0 in range(0, t, row_chunk):
        r1 = min(t, r0 + row_chunk)
        n = r1 - r0
        run = torch.zeros(n, 4, dtype=torch.float32, device=dev)
        run[:, 0] = -3.4028234663852886e38
        idz = torch.zeros(n, j, dtype=torch.float32, device=dev)
        for v0 in range(0, v, vocab_chunk):
            v1 = min(v, v0 + vocab_chunk)
            out = buf[:n, : v1 - v0]
            gemm_nt(hb[r0:r1], wb[v0:v1], torch.float32, out=out)
            _lib.check(lib.pear_head_stats_update(_lib.ptr(out), n, out.stride(0), v1 - v0, v0, _f(temperature), _lib.ptr(run),
                                                  _lib.ptr(ids32[r0:r1]), j, _lib.ptr(idz), _lib.stream()), "head_stats_update")
            _lib.count_launch(2)
        _lib.check(lib.pear_head_stats_finish(_lib.ptr(run), _lib.ptr(idz), j, _lib.ptr(lp[r0:r1]), _lib.ptr(ent[r0:r1]), n, _lib.stream()),
                   "head_stats_finish")
        _lib.count_launch(1)
    return lp, ent


_STARTS_CACHE: dict = {}


def _seq_starts(cu_seqlens, t: int, device) -> torch.Tensor:
    """First row of its sequence for every packed row, on the device. The same boundaries come back for every layer and
    pass of a micro-batch, so the last few results are kept (a host-to-device copy from pageable memory would otherwise
    drain the stream each time)."""
    key = (tuple(cu_seqlens), t, str(device))
    hit = _STARTS_CACHE.get(key)
    if hit is not None:
        return hit
    b = torch.tensor(list(cu_seqlens[:-1]), dtype=torch.int64)
    lens = torch.tensor([e - s for s, e in zip(cu_seqlens[:-1], cu_seqlens[1:])], dtype=torch.int64)
    starts = torch.repeat_interleave(b, lens).to(torch.int32)
    if starts.numel() != t:
        raise ValueError("sequence boundaries do not cover the rows")
    if torch.cuda.is_available():
        starts = starts.pin_memory()
    out = starts.to(device, non_blocking=True)
    if len(_STARTS_CACHE) >= 16:
        _STARTS_CACHE.pop(next(iter(_STARTS_CACHE)))
    _STARTS_CACHE[key] = out
    return out


class _GdnFront(torch.autograd.Function):
    """Forward and backward of the GDN front end on the kernels of ``csrc/train_kernels.cu``."""

    @staticmethod
    def forward(ctx, x, conv_w, starts, qk_channels, eps):
        xc, wc = x.contiguous(), conv_w.float().contiguous()
        t, c = xc.shape
        y = torch.empty_like(xc)
        _lib.check(_lib.lib().pear_gdn_front(_lib.ptr(xc), _lib.ptr(wc), _lib.ptr(starts), _lib.ptr(y), t, c, qk_channels, _f(eps), _lib.stream()),
                   "gdn_front")
        _lib.count_launch(1)
        ctx.save_for_backward(xc, wc, starts)
        ctx.qk_channels, ctx.eps, ctx.w_dtype = qk_channels, eps, conv_w.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, wc, starts = ctx.saved_tensors
        t, c = xc.shape
        dyc = dy.contiguous().float()
        dacc, dx = torch.empty_like(xc), torch.empty_like(xc)
        dw = torch.zeros_like(wc)
        _lib.check(_lib.lib().pear_gdn_front_bwd(_lib.ptr(xc), _lib.ptr(wc), _lib.ptr(starts), _lib.ptr(dyc), _lib.ptr(dacc), _lib.ptr(dx), _lib.ptr(dw),
                                                 t, c, ctx.qk_channels, _f(ctx.eps), _lib.stream()), "gdn_front_bwd")
        _lib.count_launch(2)
        return dx, dw.to(ctx.w_dtype), None, None, None


def gdn_front_autograd(x: torch.Tensor, conv_w: torch.Tensor, cu_seqlens, qk_channels: int, eps: float = 1e-6) -> torch.Tensor:
    """:func:`gdn_front` with a backward (the trainer's path): x [T, C] fp32, conv_w [C, 4]."""
    return _GdnFront.apply(x, conv_w, _seq_starts(list(cu_seqlens), x.shape[0], x.device), qk_channels, eps)


def gdn_front(x: torch.Tensor, conv_w: torch.Tensor, cu_seqlens: list[int], qk_channels: int, eps: float = 1e-6) -> torch.Tensor:
    """conv(4) + SiLU over packed sequences, q / k heads L2-normalised (q scaled by 128^-0.5). x [T, C] fp32."""
    t, c = x.shape
    starts = _seq_starts(list(cu_seqlens), t, x.device)
    y = torch.empty_like(x)
    _lib.check(_lib.lib().pear_gdn_front(_lib.ptr(x.contiguous()), _lib.ptr(conv_w.float().contiguous()), _lib.ptr(starts), _lib.ptr(y), t, c,
                                         qk_channels, _f(eps), _lib.stream()), "gdn_front")
    _lib.count_launch(1)
    return y

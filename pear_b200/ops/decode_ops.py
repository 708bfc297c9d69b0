"""Python bindings of the batched rollout-step kernels: the weight-streaming GEMM (``csrc/stream_gemm.cu``), the tensor-core
paged verify attention (``csrc/paged_attn_tc.cu``) and the step kernels of ``csrc/decode_step.cu``.

Every function launches on the current stream with the pointers of the tensors it is given and allocates nothing unless
``out`` is omitted, so a sequence of these calls over fixed buffers can be captured into a CUDA graph.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import lib as _lib

_f, _ll, _sz, _u = ctypes.c_float, ctypes.c_longlong, ctypes.c_size_t, ctypes.c_uint
_status: dict = {}
_sms: dict = {}


def status_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
        _sms[key] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _status[key]


def num_sms(device=None) -> int:
    status_word(device)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return _sms[dev.index if dev.index is not None else torch.cuda.current_device()]


def check_status(device=None) -> None:
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise RuntimeError(f"a bounded device-side wait of the rollout step gave up (status {code})")


def pick_splits(m: int, n: int, k: int, sms: int = 148, max_splits: int = 8) -> int:
    """K splits of the streaming GEMM. Work items (weight tiles x token blocks x splits) run one per SM at a time, so the
    split count is the largest that still fits ONE round of the SMs: measured in a replayed graph at 128 tokens on
    5120 x 17408, 3 splits (120 items) take 37.5 us, 4 splits (160 items: a second round for 12 of them) 52.9 us, 7 splits
    (280 items, two nearly full rounds) 38.4 us; every split is also one more fp32 plane for the consumer to add."""
    bt = 32 if m <= 32 else 64 if m <= 64 else 128 if m <= 128 else 256
    items = ((n + 127) // 128) * ((m + bt - 1) // bt)
    kblocks = (k + 63) // 64
    return max(1, min(max_splits, sms // max(items, 1), kblocks // 4))


def stream_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, nsplit: int = 1, epi: int = 0, up_row0: int = 0, n: Optional[int] = None) -> torch.Tensor:
    """``x`` [M, K] bf16, ``w`` [N, K] bf16. epi 0: ``out`` fp32 [nsplit, M, ldo] planes; epi 1: ``out`` bf16 [M, ldo];
    epi 2 (SwiGLU): ``w`` = [gate rows | up rows], ``n`` gate rows, up rows from ``up_row0``; ``out`` bf16 [M, ldo]."""
    m, k = x.shape
    n = w.shape[0] if n is None else n
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    if epi == 0:
        assert out.dtype == torch.float32
        ldo = out.stride(-2)
        split_stride = out.stride(0) if out.dim() == 3 else 0
        assert out.dim() == 3 or nsplit == 1
    else:
        assert out.dtype == torch.bfloat16 and nsplit == 1
        ldo, split_stride = out.stride(0), 0
    _lib.check(_lib.lib().pear_stream_gemm_bf16(_lib.ptr(x), _lib.ptr(w), _lib.ptr(out), m, n, k, x.stride(0), w.stride(0), ldo, _ll(split_stride),
                                                nsplit, epi, up_row0, _lib.ptr(status_word(x.device)), num_sms(x.device), _lib.stream()), "stream_gemm")
    _lib.count_launch()
    return out


def philox_uniform(rows: int, v: int, seed: int, step: int, device="cuda") -> torch.Tensor:
    out = torch.empty(rows, v, dtype=torch.float32, device=device)
    _lib.check(_lib.lib().pear_ds_philox_uniform(_lib.ptr(out), rows, v, _u(seed), _u(step), _lib.stream()), "philox_uniform")
    return out


def accept_uniform(rows: int, seed: int, step: int, device="cuda") -> torch.Tensor:
    out = torch.empty(rows, dtype=torch.float32, device=device)
    _lib.check(_lib.lib().pear_ds_accept_uniform(_lib.ptr(out), rows, _u(seed), _u(step), _lib.stream()), "accept_uniform")
    return out


def add_rmsnorm(parts: Optional[torch.Tensor], nsplit: int, residual: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                mode: int = 0, one_plus: bool = True, rows: Optional[int] = None) -> torch.Tensor:
    """residual (+)= sum of the first ``nsplit`` planes of ``parts`` [S, M, ld]; ``out`` bf16 = RMSNorm(residual)."""
    rows = residual.shape[0] if rows is None else rows
    h = residual.shape[1]
    _lib.expect(torch.float32, False, parts=parts, residual=residual, weight=weight)
    _lib.expect(torch.bfloat16, False, out=out)
    ss, ldp = (parts.stride(0), parts.stride(1)) if parts is not None else (0, 0)
    _lib.check(_lib.lib().pear_ds_add_rmsnorm(_lib.ptr(parts), nsplit, _ll(ss), ldp, _lib.ptr(residual), mode, _lib.ptr(weight), _lib.ptr(out), rows, h,
                                              _f(eps), 1 if one_plus else 0, _lib.stream()), "ds_add_rmsnorm")
    _lib.count_launch()
    return out


def reduce_parts_bf16(parts: torch.Tensor, nsplit: int, out: torch.Tensor, rows: int, h: int, buf_elems: int = 0,
                      epoch_ctr: Optional[torch.Tensor] = None) -> None:
    _lib.check(_lib.lib().pear_ds_reduce_parts_bf16(_lib.ptr(parts), nsplit, _ll(parts.stride(0)), parts.stride(1), _lib.ptr(out), _sz(buf_elems),
                                                    _lib.ptr(epoch_ctr), rows, h, _lib.stream()), "ds_reduce_parts_bf16")
    _lib.count_launch()


def attn_prep(qkv: torch.Tensor, qn_w, kn_w, inv_freq: torch.Tensor, rot: int, ctx, rope_off, block_table, rows: int, t: int, hq: int, hkv: int, d: int,
              gated: bool, eps: float, q_out, kc, vc) -> None:
    _lib.expect(torch.float32, False, qkv=qkv, qn_w=qn_w, kn_w=kn_w)
    _lib.expect(torch.float64, inv_freq=inv_freq)
    _lib.expect(torch.bfloat16, False, q_out=q_out, kc=kc, vc=vc)
    _lib.expect(torch.int32, False, ctx=ctx, rope_off=rope_off, block_table=block_table)
    _lib.check(_lib.lib().pear_ds_attn_prep(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(qn_w), _lib.ptr(kn_w), _lib.ptr(inv_freq), rot, _lib.ptr(ctx),
                                            _lib.ptr(rope_off), _lib.ptr(block_table), block_table.stride(0), rows, t, hq, hkv, d, 1 if gated else 0,
                                            _f(eps), _lib.ptr(q_out), _lib.ptr(kc), _lib.ptr(vc), _lib.stream()), "ds_attn_prep")
    _lib.count_launch()


PA_ITEM_INTS, PA_ITEM_SEQS = 24, 16  # layout of one work item of the tensor-core paged attention (csrc/paged_attn_tc.cu: PaItem)


def tc_attention_ok(d: int, hq: int, hkv: int, t: int) -> bool:
    return d == 256 and (hq // hkv) * t <= 128


def paged_attention(q, kc, vc, block_table, ctx, batch: int, t: int, hq: int, hkv: int, d: int, scale: float, gate_src, gated: bool, out,
                    tensor_core: Optional[bool] = None, items: Optional[torch.Tensor] = None, nparts: int = 0, part_o=None, part_ml=None) -> None:
    """Verify / decode attention over the paged cache (row (b, t) sees keys 0 .. ctx[b] + t), sigmoid gate fused.
    Head dimension 256 with ``group * t <= 128`` runs on the tcgen05 kernel, other shapes on the SIMT kernel. ``items``
    (int32 [n, 24]): the work table of the tensor-core kernel (sequences that share pages stacked in one CTA); the partial
    results go through ``part_o`` [nparts, batch * t, hq, 256] and ``part_ml`` [nparts, batch * t, hq, 2]."""
    use_tc = tc_attention_ok(d, hq, hkv, t) if tensor_core is None else tensor_core
    gate_ld = gate_src.stride(0) if gated else 0
    if use_tc:
        _lib.check(_lib.lib().pear_paged_attn_tc_hd256(_lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _ll(kc.shape[0]), _lib.ptr(block_table),
                                                       block_table.stride(0), _lib.ptr(ctx), batch, t, hq, hkv, _f(scale),
                                                       _lib.ptr(gate_src) if gated else _lib.ptr(None), gate_ld, 1 if gated else 0, _lib.ptr(out),
                                                       _lib.ptr(status_word(q.device)), _lib.ptr(items), items.shape[0] if items is not None else 0,
                                                       nparts, _lib.ptr(part_o), _lib.ptr(part_ml), _lib.stream()), "paged_attn_tc")
        if items is not None:
            _lib.count_launch()
    else:
        _lib.check(_lib.lib().pear_ds_paged_attn_simt(_lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(block_table), block_table.stride(0),
                                                      _lib.ptr(ctx), batch * t, t, hq, hkv, d, _f(scale), _lib.ptr(gate_src) if gated else _lib.ptr(None),
                                                      gate_ld, 1 if gated else 0, _lib.ptr(out), _lib.stream()), "paged_attn_simt")
    _lib.count_launch()


_gdn_scratch: dict = {}


def gdn_scratch(device, batch: int, hk: int, hv: int) -> torch.Tensor:
    """Scratch of the GDN verify pair of kernels (what the front-end kernel hands to the state kernel), one per device,
    grown on demand (never while a graph is being captured: size it with the largest batch first)."""
    fn = _lib.lib().pear_ds_gdn_scratch_bytes
    fn.restype = ctypes.c_longlong
    need = int(fn(batch, hk, hv))
    buf = _gdn_scratch.get(device)
    if buf is None or buf.numel() < need:
        assert not torch.cuda.is_current_stream_capturing(), "the GDN scratch cannot grow inside a graph capture"
        buf = torch.empty(need, dtype=torch.uint8, device=device)
        _gdn_scratch[device] = buf
    return buf


def gdn_verify(proj, conv_w, a_log, dt_bias, norm_w, state, conv_rec, ab_rec, slots, ctx, parity, ncommit, batch: int, t: int, tmax: int, hk: int,
               hv: int, l2_eps: float, rms_eps: float, out) -> None:
    scratch = gdn_scratch(state.device, batch, hk, hv)
    _lib.expect(torch.float32, False, proj=proj)
    _lib.expect(torch.float32, conv_w=conv_w, a_log=a_log, dt_bias=dt_bias, norm_w=norm_w, state=state, conv_rec=conv_rec, ab_rec=ab_rec)
    _lib.expect(torch.int32, slots=slots, ctx=ctx, parity=parity, ncommit=ncommit)
    _lib.expect(torch.bfloat16, out=out)
    _lib.check(_lib.lib().pear_ds_gdn_verify(_lib.ptr(proj), proj.stride(0) if proj is not None else 0, _lib.ptr(conv_w), _lib.ptr(a_log),
                                             _lib.ptr(dt_bias), _lib.ptr(norm_w), _lib.ptr(state), state.shape[0], _lib.ptr(conv_rec), _lib.ptr(ab_rec), _lib.ptr(slots),
                                             _lib.ptr(ctx), _lib.ptr(parity), _lib.ptr(ncommit), batch, t, tmax, hk, hv, _f(l2_eps), _f(rms_eps),
                                             _lib.ptr(out), _lib.ptr(scratch), _lib.ptr(status_word(state.device)), _lib.stream()), "ds_gdn_verify")
    _lib.count_launch(2)


def rec_bytes() -> int:
    return int(_lib.lib().pear_ds_rec_bytes())


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs) if ptrs is not None else None


def verify_chunks(logits, vs: int, v0: int, temperature: float, tok_in, ctx, batch: int, t: int, chunks: int, seed: int, step_ctr, recs_ptrs,
                  rank: int, world: int, epoch_ctr, rec_buf_elems: int) -> None:
    _lib.expect(torch.float32, False, logits=logits)
    _lib.expect(torch.int32, False, tok_in=tok_in, ctx=ctx)
    _lib.check(_lib.lib().pear_ds_verify_chunks(_lib.ptr(logits), logits.stride(0), vs, v0, _f(temperature), _lib.ptr(tok_in), _lib.ptr(ctx), batch, t,
                                                chunks, _u(seed), _lib.ptr(step_ctr), recs_ptrs, rank, world, _lib.ptr(epoch_ctr), _sz(rec_buf_elems),
                                                _lib.stream()), "ds_verify_chunks")
    _lib.count_launch()


def verify_finish(my_recs, rec_buf_elems: int, epoch_ctr, world: int, chunks: int, batch: int, t: int, seed: int, step_ctr, tok_in, ctx, ncommit, parity,
                  out_tok, out_lp, n_accept, nonfinite, sel_row, mtp_tok, mtp_ctx) -> None:
    _lib.check(_lib.lib().pear_ds_verify_finish(_lib.ptr(my_recs), _sz(rec_buf_elems), _lib.ptr(epoch_ctr), world, chunks, batch, t, _u(seed),
                                                _lib.ptr(step_ctr), _lib.ptr(tok_in), _lib.ptr(ctx), _lib.ptr(ncommit), _lib.ptr(parity), _lib.ptr(out_tok),
                                                _lib.ptr(out_lp), _lib.ptr(n_accept), _lib.ptr(nonfinite), _lib.ptr(sel_row), _lib.ptr(mtp_tok),
                                                _lib.ptr(mtp_ctx), _lib.stream()), "ds_verify_finish")
    _lib.count_launch(2)


TOPK = 32  # log-probs per row the top-k kernels produce


def top_bytes() -> int:
    return int(_lib.lib().pear_ds_top_bytes())


def topk_chunks(logits, vs: int, v0: int, temperature: float, ctx, batch: int, t: int, chunks: int, tops_ptrs, rank: int, world: int, epoch_ctr,
                buf_elems: int) -> None:
    """Per (row, chunk of this rank's vocabulary shard): the 32 largest scaled logits with their token ids, stored to every
    rank's list buffer (same slots and epochs as the sampler's records)."""
    _lib.expect(torch.float32, False, logits=logits)
    _lib.expect(torch.int32, False, ctx=ctx)
    _lib.check(_lib.lib().pear_ds_topk_chunks(_lib.ptr(logits), logits.stride(0), vs, v0, _f(temperature), _lib.ptr(ctx), batch, t, chunks, tops_ptrs,
                                              rank, world, _lib.ptr(epoch_ctr), _sz(buf_elems), _lib.stream()), "ds_topk_chunks")
    _lib.count_launch()


def topk_finish(my_tops, top_buf_elems: int, my_recs, rec_buf_elems: int, epoch_ctr, world: int, chunks: int, batch: int, t: int, ctx, out_id,
                out_lp) -> None:
    """Merge the lists of all ranks and chunks into ``out_id`` int32 / ``out_lp`` fp32 [rows, 32] (log-probs of the step's
    temperature-scaled distribution, descending; -1 / -inf padding)."""
    _lib.expect(torch.int32, out_id=out_id, ctx=ctx)
    _lib.expect(torch.float32, out_lp=out_lp)
    _lib.check(_lib.lib().pear_ds_topk_finish(_lib.ptr(my_tops), _sz(top_buf_elems), _lib.ptr(my_recs), _sz(rec_buf_elems), _lib.ptr(epoch_ctr), world,
                                              chunks, batch, t, _lib.ptr(ctx), _lib.ptr(out_id), _lib.ptr(out_lp), _lib.stream()), "ds_topk_finish")
    _lib.count_launch()


def mtp_input(tokens, table, hidden, sel, we, wh, rows: int, h: int, eps: float, out) -> None:
    _lib.expect(torch.bfloat16, table=table, out=out)
    _lib.expect(torch.float32, False, hidden=hidden, we=we, wh=wh)
    _lib.expect(torch.int32, False, tokens=tokens, sel=sel)
    _lib.check(_lib.lib().pear_ds_mtp_input(_lib.ptr(tokens), _lib.ptr(table), table.shape[0], _lib.ptr(hidden), _lib.ptr(sel), _lib.ptr(we), _lib.ptr(wh),
                                            rows, h, _f(eps), _lib.ptr(out), _lib.stream()), "ds_mtp_input")
    _lib.count_launch()


def gather_rows(src: torch.Tensor, sel: torch.Tensor, dst: torch.Tensor, rows: int) -> None:
    """dst[i] = src[sel[i]] for contiguous rows whose byte size is a multiple of 16."""
    words = src.shape[1] * src.element_size() // 4
    _lib.check(_lib.lib().pear_ds_gather_rows(_lib.ptr(src), _lib.ptr(sel), _lib.ptr(dst), rows, words, _lib.stream()), "ds_gather_rows")
    _lib.count_launch()


def argmax_chunks(logits, vs: int, v0: int, rows: int, chunks: int, keys_ptrs, rank: int, world: int, epoch_ctr, buf_elems: int) -> None:
    _lib.expect(torch.float32, False, logits=logits)
    _lib.check(_lib.lib().pear_ds_argmax_chunks(_lib.ptr(logits), logits.stride(0), vs, v0, rows, chunks, keys_ptrs, rank, world, _lib.ptr(epoch_ctr),
                                                _sz(buf_elems), _lib.stream()), "ds_argmax_chunks")
    _lib.count_launch()


def argmax_finish(my_keys, buf_elems: int, epoch_ctr, world: int, chunks: int, rows: int, dst, dst_stride: int, dst_off: int, tok_out) -> None:
    _lib.check(_lib.lib().pear_ds_argmax_finish(_lib.ptr(my_keys), _sz(buf_elems), _lib.ptr(epoch_ctr), world, chunks, rows, _lib.ptr(dst), dst_stride,
                                                dst_off, _lib.ptr(tok_out), _lib.stream()), "ds_argmax_finish")
    _lib.count_launch()


def symm_barrier(flag_ptrs, rank: int, world: int, slot: int, ctr, budget: int, status) -> None:
    _lib.check(_lib.lib().pear_ds_symm_barrier(flag_ptrs, rank, world, slot, _lib.ptr(ctr), _u(budget), _lib.ptr(status), _lib.stream()), "ds_symm_barrier")
    _lib.count_launch()


def ar_add_rmsnorm(partial_ptrs, flag_ptrs, rank: int, world: int, slot: int, ctr, ticket, residual, mode: int, weight, out, rows: int, h: int,
                   buf_elems: int, eps: float, budget: int, status, num_ctas: int) -> None:
    _lib.check(_lib.lib().pear_ds_ar_add_rmsnorm(partial_ptrs, flag_ptrs, rank, world, slot, _lib.ptr(ctr), _lib.ptr(ticket), _lib.ptr(residual), mode,
                                                 _lib.ptr(weight), _lib.ptr(out), rows, h, _sz(buf_elems), _f(eps), _u(budget), _lib.ptr(status), num_ctas,
                                                 _lib.stream()), "ds_ar_add_rmsnorm")
    _lib.count_launch()


def ar2_add_rmsnorm(partial_ptrs, flag_ptrs, out_ptrs, residual_ptrs, rank: int, world: int, slot: int, ctr, ticket, mode: int, bcast_residual: bool,
                    weight, rows: int, h: int, buf_elems: int, eps: float, budget: int, status, num_ctas: int, fixed_buf: int = -1,
                    mc_partials: int = 0, mc_outs: int = 0, mc_residuals: int = 0) -> None:
    """Two-shot all-reduce + add + RMSNorm over symmetric ``out`` / ``residual`` buffers (row t is reduced by rank t % world).
    ``mc_*``: multicast (NVLS) addresses of the same buffers; when given the sum and the broadcast go through the switch."""
    _lib.check(_lib.lib().pear_ds_ar2_add_rmsnorm(partial_ptrs, flag_ptrs, out_ptrs, residual_ptrs, rank, world, slot, _lib.ptr(ctr), _lib.ptr(ticket), mode,
                                                  1 if bcast_residual else 0, _lib.ptr(weight), rows, h, _sz(buf_elems), fixed_buf, _f(eps), _u(budget),
                                                  _lib.ptr(status), num_ctas, ctypes.c_void_p(mc_partials), ctypes.c_void_p(mc_outs),
                                                  ctypes.c_void_p(mc_residuals), _lib.stream()), "ds_ar2_add_rmsnorm")
    _lib.count_launch()

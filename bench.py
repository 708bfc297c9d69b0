#!/usr/bin/env python
"""Headline benchmark: rollout decode tokens/s of the 27B-shape hybrid model in bf16, tensor-parallel over the N GPUs.

    python bench.py --gpus N --steps K --warmup W        # N > 1: launched by torch.distributed.run, one rank per GPU

Workload (weak scaling, 32 sequences per GPU; at N = 8 it is the 256-sequence TP = 8 rollout configuration): every
sequence has a 6144-token prefix shared by all sequences (the same KV pages in every block table: a prefix-cache hit)
plus a 2048-token suffix of its own, 16-token KV pages, temperature 1.0, MTP speculative decoding with 3 draft tokens.
One step = one speculative verify step of ALL sequences (4 rows each) through the batched GPU-resident rollout step
(`pear_b200/rollout/fast_step.py`): weight-streaming tcgen05 GEMMs, tcgen05 paged attention, the GDN replay core, the
fused NVSwitch all-reduce + add + RMSNorm, the sharded rejection sampler and the MTP drafter, replayed as one CUDA graph.
Weights are random-init; the caches hold synthetic values of the shapes a prefill would leave (prefill is not part of
the metric). Every step streams this rank's whole weight shard (54 GB / N) plus KV pages and recurrent states, all far
larger than the 126 MB L2, so no L2 flush is needed between steps.

Secondary keys of the same JSON line: `nvfp4_bs1` (N = 1 only): NVFP4 batch-1 decode tok/s on the persistent decode
megakernel, the configuration upstream publishes 921 tok/s for on one GB300 (README.md:52).
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

BASELINE_TOK_S = 921.0  # upstream README.md:52, 1 x GB300, NVFP4 batch-1 decode with the DFlash-2 draft


def reference_arm() -> None:
    """The reference's own paths for these metrics are its patched vLLM + verl rollout stack and its sm_103a decode
    megakernel. The reference package itself installs offline (pure Python, into baseline/_ref); what decides is whether
    its stack can start here."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "pear")):
        why = "baseline/_ref is missing: python -m pip install --no-index --no-build-isolation --target baseline/_ref <reference> was not run"
    else:
        sys.path.insert(0, ref)
        try:
            import importlib

            import pear  # noqa: F401  the reference's own package, unmodified

            missing = [m for m in ("verl", "lmcache") if importlib.util.find_spec(m) is None]
            why = ("the reference's rollout engine is vLLM 0.34 (V2 runner) + verl at a pinned commit with 53 patches + LMCache; "
                   f"`{'`, `'.join(missing) or 'verl'}` cannot be installed offline (3rdparty/verl/scripts/checkout_verl.sh clones from GitHub) and the "
                   "installed vllm is not the patched version its plug-in registers against; its decode megakernel needs compute capability 10.3")
        except Exception as e:  # noqa: BLE001
            why = f"reference import failed: {type(e).__name__}: {e}"
    print(json.dumps({"impl": "reference", "unavailable": why}))


def reference_kernels_arm(args) -> None:
    """``--impl reference --kernels``: the sm_100 kernels the reference itself ships for its Blackwell rollout backend
    (``pear/models/qwen3_5/rollout/blackwell/csrc``: weight-streaming GEMM, tcgen05 verify attention, fused sampler, output
    gate), JIT-built unmodified from ``baseline/_ref`` by the reference's own loader and timed on one GPU at the 27B shapes,
    next to this repository's kernel for the same op on the same operands. Its peer-memory ops (fused all-reduce, logits
    gather, draft argmax exchange) are not run: their device-side polls have no limit. CUDA events, L2 flushed between
    iterations. Prints one JSON line."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "baseline", "_ref")
    out = {"impl": "reference", "mode": "kernels"}
    if not os.path.isdir(os.path.join(ref, "pear")):
        out["unavailable"] = "baseline/_ref is missing"
        print(json.dumps(out))
        return
    sys.path.insert(0, ref)
    import torch

    try:
        from pear.models.qwen3_5.rollout.blackwell.extension import BlackwellExtension

        t0 = time.time()
        try:
            BlackwellExtension.load()
        except RuntimeError as e:
            # the installed package carries the .cu sources but not the host-only cuBLASLt wrappers (*.cpp), so the loader's
            # last step (fake registration of `lt_mm` for traced graphs) fails AFTER the kernels were built and loaded; the
            # ops timed here do not depend on it
            if not hasattr(torch.ops.pear_rollout_blackwell, "sg_partials"):
                raise
            out["loader_note"] = f"register_fakes failed after the build ({str(e)[:120]}); the CUDA ops are loaded"
        out["build_s"] = round(time.time() - t0, 1)
    except Exception as e:  # noqa: BLE001
        out["unavailable"] = f"the reference's extension did not build / load here: {type(e).__name__}: {str(e)[-600:]}"
        print(json.dumps(out))
        return
    ref_ops = torch.ops.pear_rollout_blackwell
    from pear_b200.ops import decode_ops as K

    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters=10, warmup=3) -> float:
        """One launch at a time on an idle GPU with L2 flushed: includes the host's launch path (microseconds)."""
        for _ in range(warmup):
            fn()
        total = 0.0
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / iters * 1e3  # microseconds

    def timed_stream(fns, reps=4, iters=5) -> float:
        """The launches of ``fns`` (one per operand copy, together larger than L2) captured back to back in a CUDA graph and
        replayed: device time per launch as inside a decode step, no host launch path (microseconds)."""
        for fn in fns:
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for fn in fns:
                fn()
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps):
                    for fn in fns:
                        fn()
        torch.cuda.synchronize()
        graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (iters * reps * len(fns)) * 1e3

    def bf(*shape, scale=0.05):
        return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)

    rows = []

    class guarded:  # one failing op must not lose the others' numbers
        def __init__(self, what):
            self.what = what

        def __enter__(self):
            return self

        def __exit__(self, et, ev, tb):
            if et is not None:
                rows.append({"op": self.what, "error": f"{et.__name__}: {str(ev)[:300]}"})
                torch.cuda.synchronize()
            return True

    M = 128
    x5120 = bf(M, 5120, scale=0.5)
    for name, n, k, splits in (("o_proj 5120x6144", 5120, 6144, 3), ("down_proj 5120x17408", 5120, 17408, 3), ("in_proj 16384x5120", 16384, 5120, 1)):
      with guarded(f"stream GEMM {name}"):
        copies = (300 << 20) // (n * k * 2) + 2  # weight copies cycled through: together well past L2
        x, ws = bf(M, k, scale=0.5), [bf(n, k) for _ in range(copies)]
        w = ws[0]
        mine = torch.zeros(8, M, n, device="cuda")
        ns = 1 if splits == 1 else K.pick_splits(M, n, k)  # the step runs its column-parallel GEMMs unsplit
        t_ref = timed(lambda: ref_ops.sg_partials(x, w, splits))
        t_own = timed(lambda: K.stream_gemm(x, w, mine, ns, 0))
        err = float((mine[:ns].sum(0) - ref_ops.sg_partials(x, w, splits).sum(0)).abs().max())
        row = {"op": f"stream GEMM fp32 partials, {M} tokens, {name}", "reference_us": round(t_ref, 1), "own_us": round(t_own, 1),
               "reference_splits": splits, "own_splits": ns, "max_abs_diff": err}
        with guarded(f"stream GEMM {name}, graph replay"):
            s_ref = timed_stream([(lambda w_=w_: ref_ops.sg_partials(x, w_, splits)) for w_ in ws])
            s_own = timed_stream([(lambda w_=w_: K.stream_gemm(x, w_, mine, ns, 0)) for w_ in ws])
            s_own3 = timed_stream([(lambda w_=w_: K.stream_gemm(x, w_, mine, splits, 0)) for w_ in ws])
            row.update({"replay_reference_us": round(s_ref, 1), "replay_own_us": round(s_own, 1), "replay_own_us_reference_splits": round(s_own3, 1),
                        "replay_weight_gbs_reference": round(n * k * 2 / s_ref / 1e3, 1), "replay_weight_gbs_own": round(n * k * 2 / s_own / 1e3, 1)})
        rows.append(row)
        del ws
    f = 17408
    with guarded("stream GEMM + SwiGLU"):
      w_gus = [bf(2 * f, 5120) for _ in range(3)]
      w_gu = w_gus[0]
      act = torch.zeros(M, f, dtype=torch.bfloat16, device="cuda")
      t_ref = timed(lambda: ref_ops.sg_swiglu(x5120, w_gu))
      t_own = timed(lambda: K.stream_gemm(x5120, w_gu, act, 1, 2, f, f))
      row = {"op": f"stream GEMM + SwiGLU, {M} tokens, 2 x 17408 x 5120 (row layouts differ: timing only)", "reference_us": round(t_ref, 1),
             "own_us": round(t_own, 1)}
      with guarded("stream GEMM + SwiGLU, graph replay"):
          s_ref = timed_stream([(lambda w_=w_: ref_ops.sg_swiglu(x5120, w_)) for w_ in w_gus])
          s_own = timed_stream([(lambda w_=w_: K.stream_gemm(x5120, w_, act, 1, 2, f, f)) for w_ in w_gus])
          row.update({"replay_reference_us": round(s_ref, 1), "replay_own_us": round(s_own, 1),
                      "replay_weight_gbs_reference": round(2 * f * 5120 * 2 / s_ref / 1e3, 1), "replay_weight_gbs_own": round(2 * f * 5120 * 2 / s_own / 1e3, 1)})
      rows.append(row)
      del w_gus
    with guarded("output gate"):
      # output gate
      xa = bf(M, 24 * 256, scale=1.0)
      gate = bf(M, 24 * 256, scale=1.0)
      t_ref = timed(lambda: ref_ops.output_gate(xa, gate))
      rows.append({"op": "output gate x * sigmoid(g), 128 x 6144 (here: fused into the attention epilogue, no kernel of its own)", "reference_us": round(t_ref, 1),
                   "own_us": 0.0})
    with guarded("sampler"):
      # fused sampler
      R, V = 128, 248320
      logits = torch.randn(R, V, device="cuda", generator=g) * 2
      q = torch.empty(R, V, device="cuda").exponential_(generator=g)
      temp = torch.ones(R, device="cuda")
      t_ref = timed(lambda: ref_ops.fused_sample(logits, q, temp, 32, 32))  # 32 chunks per row: the reference's own launch shape
      i32 = dict(dtype=torch.int32, device="cuda")
      B, T = 32, 4
      tok_in, ctx, step_ctr = torch.zeros(B * T, **i32), torch.zeros(B, **i32), torch.zeros(1, **i32)
      recs = torch.zeros(B * T * 2 * K.rec_bytes(), dtype=torch.uint8, device="cuda")
      ptrs = K._ptr_array([recs.data_ptr()])
      outs = [torch.zeros(B, T, **i32), torch.zeros(B, T, device="cuda")] + [torch.zeros(B, **i32) for _ in range(3)] + [torch.zeros(B * T, **i32), torch.zeros(T, B, **i32)]
      ncommit, parity = torch.zeros(B, **i32), torch.zeros(B, **i32)

      def own_sampler():
          ctx.zero_()
          K.verify_chunks(logits, V, 0, 1.0, tok_in, ctx, B, T, 2, 1, step_ctr, ptrs, 0, 1, None, 0)
          K.verify_finish(recs, 0, None, 1, 2, B, T, 1, step_ctr, tok_in, ctx, ncommit, parity, *outs)

      t_own = timed(own_sampler)
      rows.append({"op": f"sampler over {R} rows x {V} (reference: temperature sampling + top-32 log-probs from a caller-made noise tensor; "
                         "here: rejection sampling of greedy drafts with in-kernel Philox, no top-32)", "reference_us": round(t_ref, 1), "own_us": round(t_own, 1)})
    with guarded("verify attention"):
      # verify attention: 32 requests x 4 rows, 24 q / 4 kv heads, 8192-token context with a 6144-token shared prefix
      n, T, Hq, Hkv, D, ctx_len, prefix = 32, 4, 24, 4, 256, 8192, 6144
      pages64 = prefix // 64 + n * ((ctx_len - prefix + T) // 64 + 1) + 1
      kv = bf(pages64, Hkv, 64, 2 * D, scale=1.0)
      table64 = torch.zeros(n, (ctx_len + T) // 64 + 1, **i32)
      shared = torch.arange(1, 1 + prefix // 64, dtype=torch.int32)
      per = (ctx_len - prefix + T) // 64 + 1
      for b in range(n):
          own = torch.arange(1 + prefix // 64 + b * per, 1 + prefix // 64 + (b + 1) * per, dtype=torch.int32)
          table64[b, : prefix // 64 + per] = torch.cat([shared, own]).cuda()
      qv, kn, vn = bf(n * T, Hq, D, scale=1.0), bf(n * T, Hkv, D, scale=1.0), bf(n * T, Hkv, D, scale=1.0)
      pos = torch.arange(ctx_len, ctx_len + T)
      slot = torch.stack([table64[b, (pos // 64)].cpu().long() * 64 + pos % 64 for b in range(n)]).reshape(-1).cuda()
      seq_lens = torch.full((n,), ctx_len + T, **i32)
      ctas = 148
      part_o = torch.zeros((ctas + n * Hkv) * 48 * D, device="cuda")
      part_ml = torch.zeros((ctas + n * Hkv) * 48 * 2, device="cuda")
      o_ref = torch.zeros(n * T, Hq, D, dtype=torch.bfloat16, device="cuda")
      t_ref = timed(lambda: ref_ops.verify_attention(qv, kn, vn, slot, kv, table64, seq_lens, o_ref, part_o, part_ml, n, T, D ** -0.5, ctas))
      # the same keys and values in this repository's layout: 16-token pages [page, 16, Hkv, 256], K and V separate
      pages16 = pages64 * 4
      kc = kv[..., :D].permute(0, 2, 1, 3).reshape(pages64, 4, 16, Hkv, D).reshape(pages16, 16, Hkv, D).contiguous()
      vc = kv[..., D:].permute(0, 2, 1, 3).reshape(pages64, 4, 16, Hkv, D).reshape(pages16, 16, Hkv, D).contiguous()
      table16 = (table64.long()[:, :, None] * 4 + torch.arange(4, device="cuda")).reshape(n, -1).int().contiguous()
      ctxv = torch.full((n,), ctx_len, **i32)
      o_own = torch.zeros(n * T, Hq * D, dtype=torch.bfloat16, device="cuda")
      gate_src = torch.zeros(n * T, 2 * Hq * D, device="cuda")
      splits = 6
      items = [[1, prefix, -1, 0, 1 + splits, 1 + 8, 0, 0, b] + [0] * 15 for b in range(n)]
      tiles = prefix // 128
      for i in range(0, n, 5):
          sub = list(range(i, min(n, i + 5)))
          for sp in range(splits):
              items.append([len(sub), tiles * sp // splits * 128, tiles * (sp + 1) // splits * 128, 1 + sp, 0, 0, 0, 0] + sub + [0] * (16 - len(sub)))
      items_t = torch.tensor(items, **i32)
      po, pml = torch.zeros(9, n * T, Hq, D, device="cuda"), torch.zeros(9, n * T, Hq, 2, device="cuda")
      t_own_items = timed(lambda: K.paged_attention(qv, kc, vc, table16, ctxv, n, T, Hq, Hkv, D, D ** -0.5, gate_src, False, o_own, True, items_t, 9, po, pml))
      err_items = float((o_own.view(n * T, Hq, D).float() - o_ref.float()).abs().max())
      t_own_direct = timed(lambda: K.paged_attention(qv, kc, vc, table16, ctxv, n, T, Hq, Hkv, D, D ** -0.5, gate_src, False, o_own, True))
      row = {"op": f"paged verify attention, {n} requests x {T} rows, {Hq} q / {Hkv} kv heads, context {ctx_len} ({prefix} shared); reference pages of 64 "
                         "tokens, here 16 (the reference also writes the step's K / V into the cache inside the kernel)", "reference_us": round(t_ref, 1),
                   "own_us": round(t_own_items, 1), "own_us_without_prefix_sharing": round(t_own_direct, 1), "max_abs_diff": err_items}
      with guarded("verify attention, graph replay"):  # one launch reads 290 MB of pages: larger than L2 by itself
          row["replay_reference_us"] = round(timed_stream([lambda: ref_ops.verify_attention(qv, kn, vn, slot, kv, table64, seq_lens, o_ref, part_o, part_ml, n, T, D ** -0.5, ctas)]), 1)
          row["replay_own_us"] = round(timed_stream([lambda: K.paged_attention(qv, kc, vc, table16, ctxv, n, T, Hq, Hkv, D, D ** -0.5, gate_src, False, o_own, True, items_t, 9, po, pml)]), 1)
      rows.append(row)
    K.check_status()
    out["kernels"] = rows
    out["note"] = ("x_us: CUDA events around single launches on an idle GPU, L2 flushed (256 MB write) before each, host launch path included; "
                   "replay_x_us: device time per launch of a replayed CUDA graph cycling operand copies larger than L2; microseconds")
    print(json.dumps(out))


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="pear_clocks_", suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); smax.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def load_peaks() -> dict:
    try:
        return json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
    except OSError:
        return {}


# ---------------------------------------------------------------------------------------------------------------------
# rollout decode, tensor-parallel over the ranks
# ---------------------------------------------------------------------------------------------------------------------
def build_rollout(args, rank: int, world: int, symm):
    import torch

    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.parallel.tensor_parallel import tp_config
    from pear_b200.rollout.fast_step import FastDecoder

    full = HybridConfig.small_gpu() if args.small else HybridConfig.qwen3_8_27b()
    shards = max(world, args.emulate_tp)
    cfg = tp_config(full, shards) if shards > 1 else full
    if args.emulate_tp > 1:  # one rank's share of a tensor-parallel step, without the exchange: for kernel-by-kernel profiling
        full = dataclasses.replace(full, vocab_size=full.vocab_size // args.emulate_tp)
        cfg = dataclasses.replace(cfg, vocab_size=full.vocab_size)
    B, T = args.seqs_per_gpu * shards, 1 + args.drafts
    prefix, suffix, bs = args.prefix_len, args.suffix_len, 16
    assert prefix % bs == 0 and suffix % bs == 0
    total_steps = 2 * args.steps + max(3, args.warmup) + 8
    new_pages = (total_steps * T + bs - 1) // bs + 1
    per_seq = suffix // bs + new_pages
    pages = 1 + prefix // bs + B * per_seq
    dev = torch.device("cuda", torch.cuda.current_device())
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = HybridForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.init_weights_device(seed=0).eval()  # the same seed on every rank: replicated tensors (norms, embedding, head) agree
    g = torch.Generator(device=dev).manual_seed(1)

    def kv():
        return torch.empty(pages, bs, cfg.num_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device=dev).normal_(0.0, 1.0, generator=g)

    kc = {li: kv() for li in cfg.attention_layers}
    vc = {li: kv() for li in cfg.attention_layers}
    mk, mv = [kv() for _ in model.mtp.layers], [kv() for _ in model.mtp.layers]
    rs = {li: torch.empty(B, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_head_dim, dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=g)
          for li in cfg.gdn_layers}
    dec = FastDecoder(model, kc, vc, rs, mk, mv, num_slots=B, max_batch=B, n_draft=args.drafts, max_blocks_per_seq=prefix // bs + per_seq,
                      temperature=1.0, seed=1234, symm=symm, use_graph=not args.no_graph, ar_mode=args.ar_mode)
    tok = torch.Generator().manual_seed(7)
    shared = list(range(1, 1 + prefix // bs))
    tables = []
    for b in range(B):
        own = list(range(1 + prefix // bs + b * per_seq, 1 + prefix // bs + (b + 1) * per_seq))
        tables.append(shared + own)
        conv = {li: torch.empty(3, cfg.gdn_conv_dim, device=dev).normal_(0.0, 0.5, generator=g) for li in cfg.gdn_layers}
        dec.assign(b, b, prefix + suffix, tables[b], int(torch.randint(0, full.vocab_size, (1,), generator=tok)), conv)
    if not args.no_prefix_sharing:
        dec.set_shared_prefixes([(list(range(B)), prefix)])  # what the engine derives from equal leading pages of the block tables
    return full, cfg, model, dec, tables, dict(B=B, T=T, pages=pages, per_seq=per_seq)


def rollout_bytes(full, cfg, world: int, B: int, T: int, ctx: int, prefix: int, drafts: int, reduction: str = "one") -> dict:
    """Algorithmic traffic and work of one step on one rank. ``reduction``: the form of the fused all-reduce, which sets the
    bytes that enter a GPU over NVLink per reduced row of H bf16 values: one-shot pull (W - 1) rows, two-shot
    2 (W - 1) / W (its share of the partial rows in, everyone else's results in), switch-side (nvls) 1 / W + (W - 1) / W."""
    h, V = full.hidden_size, full.vocab_size
    n_attn, n_gdn = len(cfg.attention_layers), len(cfg.gdn_layers)
    attn_w = h * (2 * cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * h
    gdn_w = h * (cfg.gdn_conv_dim + cfg.gdn_value_dim + 2 * cfg.gdn_v_heads) + cfg.gdn_value_dim * h
    mlp_w = 3 * h * cfg.intermediate_size
    main_w = n_attn * (attn_w + mlp_w) + n_gdn * (gdn_w + mlp_w)
    head_w = V // world * h
    mtp_w = 2 * h * h // world + attn_w + mlp_w
    weights = 2.0 * (main_w + head_w + drafts * (mtp_w + head_w))
    kv_row = 2 * cfg.num_kv_heads * cfg.head_dim * 2  # K and V bytes per token per layer
    # the shared prefix is read from HBM once per layer and then hits L2; every sequence reads its own suffix
    kv = (n_attn + drafts) * (prefix + B * (ctx - prefix)) * kv_row
    state = n_gdn * B * cfg.gdn_v_heads * cfg.gdn_head_dim * cfg.gdn_head_dim * 4 * 2
    M = B * T
    flops = 2.0 * M * (main_w + head_w) + 2.0 * (M + (drafts - 1) * B) * mtp_w + 2.0 * drafts * B * head_w
    flops += 4.0 * (n_attn) * M * cfg.num_attention_heads * cfg.head_dim * ctx
    n_ar = 2 * (n_attn + n_gdn) + 3 + 2 * (drafts - 1)  # reductions over M rows (main + first drafter pass) ...
    nvlink = 0.0
    if world > 1:
        per_row = {"one": float(world - 1), "two": 2.0 * (world - 1) / world, "nvls": 1.0}[reduction]
        nvlink = per_row * h * 2.0 * (M * (2 * (n_attn + n_gdn) + 3) + B * 3 * (drafts - 1))
    return dict(weight_bytes=weights, kv_bytes=float(kv), state_bytes=float(state), flops=flops, nvlink_in_bytes=nvlink, reductions=n_ar)


def run_rollout(args, rank, local_rank, world, dist, symm) -> dict:
    import torch

    from pear_b200.ops import lib as kernel_lib

    warmup = max(3, args.warmup)
    t0 = time.time()
    full, cfg, model, dec, tables, shape = build_rollout(args, rank, world, symm)
    B, T = shape["B"], shape["T"]
    torch.cuda.synchronize()
    build_s = time.time() - t0

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    l0 = kernel_lib.LAUNCH_COUNT
    dec.step()  # eager: counts this library's launches of one step
    torch.cuda.synchronize()
    launches_per_step = kernel_lib.LAUNCH_COUNT - l0
    for _ in range(warmup + 1):  # second eager step, capture, replays
        dec.step()
    barrier()
    dec.check()
    ctx0 = dec.ctx.clone()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        dec.step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    dec.check()
    ctx1 = dec.ctx.clone()
    tokens = int((ctx1 - ctx0).sum().item())
    ctx_mid = int(((ctx0 + ctx1) // 2).float().mean().item())

    # ---- end to end through the engine object's public calls: every step the host copies the block tables from pinned
    # memory (pages for the next tokens), launches the step, copies the result record back and reads the tokens
    pinned = torch.zeros(dec.block_table.shape, dtype=torch.int32).pin_memory()
    for b in range(B):
        pinned[b, : len(tables[b])] = torch.tensor(tables[b], dtype=torch.int32)
    barrier()
    t0 = time.perf_counter()
    e2e_tokens = 0
    for _ in range(args.steps):
        dec.block_table.copy_(pinned, non_blocking=True)
        dec.step()
        res = dec.results()
        e2e_tokens += int((res.tokens >= 0).sum())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    dec.check()
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = t.tolist()
    peaks = load_peaks()
    hbm, tf = peaks.get("hbm_gbs", 6650.0), peaks.get("bf16_tflops_sustained", 1400.0)
    src = "measured" if peaks else "fallback"
    step_ms = ms / args.steps
    reduction = "one" if (world == 1 or not dec._two_shot(B * T)) else ("nvls" if (dec.ar_mode == "nvls" or dec.nvls_auto) else "two")
    acct = rollout_bytes(full, cfg, world, B, T, ctx_mid, args.prefix_len, args.drafts, reduction)
    hbm_bytes = acct["weight_bytes"] + acct["kv_bytes"] + acct["state_bytes"]
    t_hbm, t_flop, t_link = hbm_bytes / (hbm * 1e9), acct["flops"] / (tf * 1e12), acct["nvlink_in_bytes"] / 770e9
    bound = max(t_hbm, t_flop, t_link)
    value = tokens / (ms / 1e3)
    return {
        "metric": "rollout decode tokens/s" if args.emulate_tp <= 1 else f"NOT A BENCHMARK: one rank's share of a tp{args.emulate_tp} step without the exchange",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (weights, activations, KV), fp32 accumulate / residual / recurrent state", "data": "synthetic",
        "config": {
            "model": ("27B-shape hybrid GDN+gated-attention (64 layers, hidden 5120, vocab 248320), random init" if not args.small
                      else "SMALL smoke model (4 layers of the 27B shape)"),
            "global_batch": B, "seq_len": args.prefix_len + args.suffix_len, "parallelism": f"tp{world}",
            "sequences_per_gpu": args.seqs_per_gpu, "shared_prefix": args.prefix_len, "unique_suffix": args.suffix_len,
            "mean_context": ctx_mid, "draft_tokens": args.drafts, "kv_block": 16, "temperature": 1.0,
            "reduction": {"one": "one-shot pull", "two": "two-shot (peer loads / stores)", "nvls": "two-shot through the switch (multimem)"}[reduction] if world > 1 else "none",
            "accepted_per_step": round(tokens / max(1, args.steps * B) - 1.0, 4),
            "l2": "inputs larger than L2: every step streams %.1f GB of weights + %.1f GB of KV pages and recurrent state per GPU"
                  % (acct["weight_bytes"] / 1e9, (acct["kv_bytes"] + acct["state_bytes"]) / 1e9),
            "caches": "synthetic values of the shapes a prefill leaves (prefill is not part of the metric)",
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(pinned.numel() * 4),
                "d2h_bytes_per_step": int(dec._host.numel() * 4), "steps": args.steps, "api": "FastDecoder.step + results"},
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "roofline": {
            "peaks": src, "hbm_gbs_peak": hbm, "bf16_tflops_peak": tf, "nvlink_gbs_per_dir": 770.0,
            "weight_gb_per_step": round(acct["weight_bytes"] / 1e9, 3), "kv_state_gb_per_step": round((acct["kv_bytes"] + acct["state_bytes"]) / 1e9, 3),
            "tflop_per_step": round(acct["flops"] / 1e12, 3), "nvlink_in_gb_per_step": round(acct["nvlink_in_bytes"] / 1e9, 4),
            "t_hbm_ms": round(t_hbm * 1e3, 3), "t_flop_ms": round(t_flop * 1e3, 3), "t_nvlink_ms": round(t_link * 1e3, 3),
            "bound": "hbm" if bound == t_hbm else ("compute" if bound == t_flop else "nvlink"),
            f"frac_of_{src}_roofline": round(bound * 1e3 / step_ms, 3),
        },
        "setup": {"build_s": round(build_s, 1), "pages": shape["pages"]},
    }


# ---------------------------------------------------------------------------------------------------------------------
# NVFP4 batch-1 decode on the persistent megakernel (secondary, one GPU)
# ---------------------------------------------------------------------------------------------------------------------
def run_megakernel(args, local_rank: int) -> dict:
    import torch

    from pear_b200.deploy.engine import MegakernelEngine, RandomWeights
    from pear_b200.models.config import HybridConfig

    steps, warmup = args.mk_steps, 4
    cfg = HybridConfig.small_gpu() if args.small else HybridConfig.qwen3_8_27b()
    dcfg = HybridConfig.drafter(cfg.hidden_size, cfg.vocab_size)
    prompt_len = args.mk_prompt_len
    eng = MegakernelEngine(cfg, dcfg, RandomWeights("cuda", seed=0), max_len=prompt_len + 4 * (steps + warmup) + 256, n_draft=3, seed=1234, temperature=1.0)
    prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    eng.start(prompt)
    eng.prefill()
    for _ in range(warmup):
        eng.decode_step(copy_out=False)
    torch.cuda.synchronize()
    eng.check_status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    n0 = int(eng.rec[eng.step & 1][6].item())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.decode_step(copy_out=False)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    tokens = int(eng.rec[eng.step & 1][6].item()) - n0
    eng.check_status()
    stats = eng._prog_dev["decode"][2]
    hbm = load_peaks().get("hbm_gbs", 6650.0)
    value = tokens / (ms / 1e3)
    return {"metric": "NVFP4 batch-1 decode tok/s", "value": round(value, 2), "ms_per_step": round(ms / steps, 4), "steps": steps,
            "vs_baseline": round(value / BASELINE_TOK_S, 4) if not args.small else None, "prompt_len": prompt_len, "draft_tokens": 3,
            "accepted_per_step": round(tokens / steps - 1.0, 4), "weight_gb_per_step": round(stats["weight_bytes"] / 1e9, 3),
            "frac_of_copy_bw": round(stats["weight_bytes"] / 1e9 / (ms / steps / 1e3) / hbm, 3), "clocks": clocks}


# ---------------------------------------------------------------------------------------------------------------------
# component timings (not the headline): trainer step on one GPU, Gated-DeltaNet scan
# ---------------------------------------------------------------------------------------------------------------------
def run_trainer_step(args) -> dict:
    """Forward + backward + optimizer step of the trainer engine on one GPU for ``--layers`` layers of the 27B shape over a
    packed batch of ``--tokens`` tokens (synthetic tokens, random init), CUDA events; ``--breakdown N`` adds the N kernels
    with the most device time of one more step under the torch profiler (after the timed region, on stderr)."""
    import torch

    from pear_b200.models.config import HybridConfig
    from pear_b200.train.engine import EngineConfig, TrainEngine, synthetic_batch

    cfg = HybridConfig(num_layers=args.layers, vocab_size=args.vocab)  # the 27B per-layer shape
    ecfg = EngineConfig(lr=1e-6, param_dtype="bf16", enable_gradient_checkpointing=True, topk_log_probs=0,
                        gradient_checkpointing_retain_attention=args.retain_attention)
    eng = TrainEngine(cfg, ecfg, device="cuda", seed=0)
    batches = [synthetic_batch(cfg, args.tokens, args.seqs, 0, s).to("cuda") for s in range(2)]

    def step(i: int) -> dict:
        m = eng.forward_backward_batch([batches[i % 2]])
        m.update(eng.optimizer_step())
        return m

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        m = step(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 3.0 * cfg.flops_per_token(context=args.tokens // args.seqs // 2) * args.tokens  # fwd + 2x bwd (recompute not counted)
    out = {"metric": "trainer step tokens/s (1 GPU)", "layers": args.layers, "tokens": args.tokens, "seqs": args.seqs, "ms_per_step": round(ms, 2),
           "tokens_per_s": round(args.tokens / ms * 1e3, 1), "model_tflops": round(flops / ms / 1e9, 1), "grad_norm": float(m.get("actor/grad_norm", 0.0)),
           "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2), "data": "synthetic", "dtype": "bf16 operands, fp32 residual and head",
           "clocks": clocks}
    peaks = load_peaks()
    if peaks:
        out["frac_of_measured_bf16_sustained"] = round(out["model_tflops"] / peaks["bf16_tflops_sustained"], 3)
    if args.breakdown:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(0)
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.breakdown, max_name_column_width=70), file=sys.stderr)
    return out


def run_gdn_scan(args) -> dict:
    """The Gated-DeltaNet scan of one sequence without gradients: the chunk-loop kernel path against the torch loop."""
    import torch

    from pear_b200.ops import kernels as K
    from pear_b200.ops import reference as ref

    g = torch.Generator(device="cuda").manual_seed(0)
    t, hk, hv, d = args.tokens, 16, 48, 128
    q = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g)) * d ** -0.5
    k = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g))
    v = torch.randn(t, hv, d, device="cuda", generator=g)
    gate = -torch.rand(t, hv, device="cuda", generator=g) * 0.2
    beta = torch.rand(t, hv, device="cuda", generator=g)

    def timed(fn, n=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    with torch.no_grad():
        kernel_ms = timed(lambda: K.gdn_scan(q, k, v, gate, beta))
        torch_ms = timed(lambda: ref.gdn_chunked(q, k, v, gate, beta))
        operands_ms = timed(lambda: ref.gdn_chunk_operands(q, k, v, gate, beta))
        o1, _ = K.gdn_scan(q, k, v, gate, beta)
        o2, _ = ref.gdn_chunked(q, k, v, gate, beta)
    return {"op": "gdn_scan", "tokens": t, "value_heads": hv, "kernel_path_ms": round(kernel_ms, 3), "torch_loop_ms": round(torch_ms, 3),
            "operands_ms": round(operands_ms, 3), "max_abs_diff": float((o1 - o2).abs().max())}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="pear_b200")
    ap.add_argument("--kernels", action="store_true", help="with --impl reference: time the reference's own sm_100 rollout kernels beside ours")
    ap.add_argument("--seqs-per-gpu", type=int, default=32)
    ap.add_argument("--prefix-len", type=int, default=6144)
    ap.add_argument("--suffix-len", type=int, default=2048)
    ap.add_argument("--drafts", type=int, default=3)
    ap.add_argument("--mk-steps", type=int, default=128)
    ap.add_argument("--mk-prompt-len", type=int, default=4096)
    ap.add_argument("--no-megakernel", action="store_true")
    ap.add_argument("--ar-mode", default="auto", choices=["auto", "one", "two", "nvls"], help="form of the fused all-reduce + add + RMSNorm (N > 1)")
    ap.add_argument("--no-prefix-sharing", action="store_true", help="attention reads the shared prefix pages once per sequence instead of once per group")
    ap.add_argument("--emulate-tp", type=int, default=0, help="profiling aid (one GPU): run ONE rank's share of a tensor-parallel step of this size, "
                    "without the inter-GPU exchange; not a benchmark of anything")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly (kernel-by-kernel profiling); the headline uses graph replay")
    ap.add_argument("--small", action="store_true", help="4-layer model of the 27B layer shape (smoke runs only; not the headline)")
    ap.add_argument("--trainer-step", action="store_true", help="component timing: trainer engine step on one GPU (prints its own JSON line)")
    ap.add_argument("--gdn-scan", action="store_true", help="component timing: Gated-DeltaNet scan of one sequence (prints its own JSON line)")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--seqs", type=int, default=2)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--retain-attention", action="store_true")
    ap.add_argument("--breakdown", type=int, default=0)
    args = ap.parse_args()
    if args.impl == "reference":
        if args.kernels:
            reference_kernels_arm(args)
        else:
            reference_arm()
        return
    if args.trainer_step or args.gdn_scan:
        print(json.dumps(run_trainer_step(args) if args.trainer_step else run_gdn_scan(args)))
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    symm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from pear_b200.parallel.symm import SymmWorld

        symm = SymmWorld()
    out = run_rollout(args, rank, local_rank, world, dist, symm)
    if world == 1 and not args.no_megakernel:
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        try:
            out["nvfp4_bs1"] = run_megakernel(args, local_rank)
        except Exception as e:  # noqa: BLE001  the secondary number never takes the headline down
            out["nvfp4_bs1"] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

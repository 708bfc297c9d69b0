#!/usr/bin/env python
"""Headline benchmark: NVFP4 batch-1 decode tokens/s of the 27B-shape hybrid model on the persistent decode megakernel
(the configuration upstream publishes 921 tok/s for on one GB300, README.md:52).

    python bench.py --gpus N --steps K --warmup W        # N > 1: launched by torch.distributed.run, one rank per GPU

One step = one megakernel launch = one speculative verify step (1 committed token + 3 drafts) of one sequence.
N > 1 runs N independent replicas (data-parallel serving, one session per GPU): weak scaling, `value` is the sum.
Weights are random-init and quantised to NVFP4 on the device; the prompt is 4096 uniform-random token ids (synthetic).
Every step streams the whole quantised model (~15 GB >> the 126 MB L2), so no L2 flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

BASELINE_TOK_S = 921.0  # upstream README.md:52, 1 x GB300, NVFP4 batch-1 decode with the DFlash-2 draft


def reference_arm() -> None:
    """The reference's own path for this metric is its sm_103a decode megakernel under a patched vLLM server. The
    reference package itself installs offline (pure Python, into baseline/_ref); what decides is its own GPU check."""
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "pear")):
        why = "baseline/_ref is missing: python -m pip install --no-index --no-build-isolation --target baseline/_ref <reference> was not run"
    else:
        sys.path.insert(0, ref)
        try:
            import torch
            from pear.models.qwen3_5.gpu_generation import GpuGeneration  # the reference's own module, unmodified
            cap = torch.cuda.get_device_capability() if torch.cuda.is_available() else None
            if not GpuGeneration.BLACKWELL_ULTRA.includes(cap):
                why = (f"the reference's decode megakernel backend requires its GpuGeneration.BLACKWELL_ULTRA (compute capability 10.3, "
                       f"built for sm_103a); this GPU is {cap}: pear/models/qwen3_5/deploy/blackwell/gpu_backend.py selects no backend here")
            else:
                why = ("the reference's deploy path needs its patched vLLM server and a ModelOpt NVFP4 checkpoint of the 27B model, "
                       "neither of which exists offline")
        except Exception as e:  # noqa: BLE001
            why = f"reference import failed: {type(e).__name__}: {e}"
    print(json.dumps({"impl": "reference", "unavailable": why}))


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
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="pear_b200")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--drafts", type=int, default=3)
    ap.add_argument("--small", action="store_true", help="4-layer model of the 27B layer shape (smoke runs only; not the headline)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from pear_b200.deploy.engine import MegakernelEngine, RandomWeights
    from pear_b200.models.config import HybridConfig
    from pear_b200.ops import lib as kernel_lib

    warmup = max(3, args.warmup)
    cfg = HybridConfig.small_gpu() if args.small else HybridConfig.qwen3_8_27b()
    dcfg = HybridConfig.drafter(cfg.hidden_size, cfg.vocab_size)
    max_len = args.prompt_len + 4 * (2 * args.steps + warmup) + 256
    t0 = time.time()
    eng = MegakernelEngine(cfg, dcfg, RandomWeights("cuda", seed=rank), max_len=max_len, n_draft=args.drafts, seed=1234 + rank,
                           temperature=1.0)
    build_s = time.time() - t0
    gen = torch.Generator().manual_seed(rank)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=gen, dtype=torch.int32)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def n_out_total() -> int:
        return int(eng.rec[eng.step & 1][6].item())

    # ---- prefill (untimed) and warm-up
    eng.start(prompt)
    t0 = time.time()
    eng.prefill()
    torch.cuda.synchronize()
    prefill_s = time.time() - t0
    for _ in range(warmup):
        eng.decode_step(copy_out=False)
    barrier()
    eng.check_status()

    # ---- device-timed region: exactly K steps, CUDA events on the launching stream
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0, tokens0 = kernel_lib.LAUNCH_COUNT, n_out_total()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eng.decode_step(copy_out=False)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    tokens = n_out_total() - tokens0
    launches = kernel_lib.LAUNCH_COUNT - launches0
    eng.check_status()

    # ---- end to end through the public API: per step a pinned->device control record, the launch, a device->pinned
    # copy of the step output, and the host reading the emitted tokens (two launches of lookahead)
    barrier()
    t0 = time.perf_counter()
    res = eng.decode(args.steps, by_steps=True)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_tokens = len(res.tokens)
    eng.check_status()

    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = t.tolist()
        c = torch.tensor([tokens, e2e_tokens, launches], device="cuda", dtype=torch.float64)
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
        tokens, e2e_tokens, launches = (int(x) for x in c.tolist())
    value = tokens / (ms / 1e3)
    stats = eng._prog_dev["decode"][2]
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
        except OSError:
            pass
        hbm = peaks.get("hbm_gbs", 6650.0)
        step_ms = ms / args.steps
        out = {
            "metric": "NVFP4 batch-1 decode tok/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": round(step_ms, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": round(value / BASELINE_TOK_S, 4) if not args.small else None,
            "dtype": "nvfp4 weights (e2m1 + e4m3 block scales), f16 activations, fp32 accumulate", "data": "synthetic",
            "config": {
                "model": "27B-shape hybrid GDN+gated-attention (64 layers, hidden 5120), random init" if not args.small
                         else "SMALL smoke model (4 layers of the 27B shape)",
                "drafter": "2-layer block drafter, random init", "global_batch": world, "seq_len": args.prompt_len,
                "prompt_len": args.prompt_len, "generated": tokens, "draft_tokens": args.drafts,
                "parallelism": f"dp{world} (one session per GPU)", "temperature": 1.0,
                "l2": "inputs larger than L2: every step streams %.1f GB of weights" % (stats["weight_bytes"] / 1e9),
                "accepted_per_step": round(tokens / max(1, args.steps * world) - 1.0, 4),
            },
            "clocks": clocks,
            "e2e": {"value": round(e2e_tokens / e2e_s, 2), "unit": "tokens/s", "h2d_bytes_per_step": 32,
                    "d2h_bytes_per_step": 64, "steps": args.steps, "api": "MegakernelEngine.decode"},
            "gpu_launches": launches,
            "roofline": {"weight_gb_per_step": round(stats["weight_bytes"] / 1e9, 3),
                         "hbm_gbs_achieved": round(stats["weight_bytes"] / 1e9 / (step_ms / 1e3), 1),
                         "hbm_gbs_peak": hbm, "frac_of_measured_copy_bw": round(stats["weight_bytes"] / 1e9 / (step_ms / 1e3) / hbm, 3)},
            "setup": {"build_s": round(build_s, 1), "prefill_s": round(prefill_s, 2), "prefill_steps": eng.prefill_steps},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

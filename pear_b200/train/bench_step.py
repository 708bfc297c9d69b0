"""``python -m pear_b200.train.bench_step [--layers L] [--tokens T] [--seqs S] [--steps K] [--warmup W]``: time the trainer
engine's forward + backward + optimizer step on one GPU for ``L`` layers of the 27B shape over a packed batch of ``T``
tokens in ``S`` sequences (synthetic tokens, random init), with CUDA events, and print one JSON line (tokens/s, model
FLOP/s against the measured bf16 peak when ``MEASURED_PEAKS.json`` is present)."""

from __future__ import annotations

import argparse
import dataclasses
import json
import os

import torch

from ..models.config import HybridConfig
from .engine import EngineConfig, PackedBatch, TrainEngine


def synthetic_batch(cfg: HybridConfig, tokens: int, seqs: int, topk: int, seed: int) -> PackedBatch:
    g = torch.Generator().manual_seed(seed)
    per = tokens // seqs
    cu = [i * per for i in range(seqs)] + [tokens]
    ids = torch.randint(0, cfg.vocab_size, (tokens,), generator=g)
    pos = torch.cat([torch.arange(e - s) for s, e in zip(cu[:-1], cu[1:])])
    mask = torch.ones(tokens)
    for s, e in zip(cu[:-1], cu[1:]):
        mask[s: s + (e - s) // 2] = 0
        mask[e - 1] = 0
    return PackedBatch(ids, pos, cu, torch.roll(ids, -1), mask, torch.randn(tokens, generator=g) * mask,
                       sampler_log_probs=-torch.rand(tokens, generator=g) * 3,
                       head_ids=torch.randint(0, cfg.vocab_size, (tokens, topk), generator=g, dtype=torch.int32) if topk else None,
                       head_log_probs=torch.log_softmax(torch.randn(tokens, topk + 2, generator=g), -1)[:, :topk] if topk else None)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seqs", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--vocab", type=int, default=32768)
    ap.add_argument("--retain-attention", action="store_true", help="keep attention outputs from the first pass of a checkpointed layer")
    ap.add_argument("--breakdown", type=int, default=0, help="after the timed steps, run one step under the torch profiler and "
                    "print the N kernels with the most device time (stderr)")
    a = ap.parse_args()
    cfg = HybridConfig(num_layers=a.layers, vocab_size=a.vocab)  # the 27B per-layer shape
    ecfg = EngineConfig(lr=1e-6, param_dtype="bf16", enable_gradient_checkpointing=True, topk_log_probs=0,
                        gradient_checkpointing_retain_attention=a.retain_attention)
    eng = TrainEngine(cfg, ecfg, device="cuda", seed=0)
    batches = [synthetic_batch(cfg, a.tokens, a.seqs, 0, s).to("cuda") for s in range(2)]

    def step(i: int) -> dict:
        m = eng.forward_backward_batch([batches[i % 2]])
        m.update(eng.optimizer_step())
        return m

    for i in range(a.warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        m = step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    flops = 3.0 * cfg.flops_per_token(context=a.tokens // a.seqs // 2) * a.tokens  # fwd + 2x bwd (recompute not counted)
    out = {"metric": "trainer step tokens/s (1 GPU)", "layers": a.layers, "tokens": a.tokens, "seqs": a.seqs, "ms_per_step": round(ms, 2),
           "tokens_per_s": round(a.tokens / ms * 1e3, 1), "model_tflops": round(flops / ms / 1e9, 1), "grad_norm": float(m.get("actor/grad_norm", 0.0)),
           "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2), "data": "synthetic", "dtype": "bf16 operands, fp32 residual and head"}
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        out["frac_of_measured_bf16_sustained"] = round(out["model_tflops"] / json.load(open(peaks))["bf16_tflops_sustained"], 3)
    print(json.dumps(out))
    if a.breakdown:
        import sys
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(0)
            torch.cuda.synchronize()
        print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=a.breakdown, max_name_column_width=70), file=sys.stderr)


if __name__ == "__main__":
    main()

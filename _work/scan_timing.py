"""``python -m pear_b200.ops.scan_timing [--tokens T] [--heads HV] [--qk-heads HK]``: time the Gated-DeltaNet scan of one
sequence without gradients on one GPU (CUDA events, 2 warm-up + 5 timed calls): the chunk-loop kernel path
(``ops/kernels.py: gdn_scan``), the torch loop (``ops/reference.py: gdn_chunked``) and the chunk-local operands alone,
and print one JSON line with the largest difference between the two outputs."""

from __future__ import annotations

import argparse
import json

import torch

from . import kernels as K
from . import reference as ref


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=48)
    ap.add_argument("--qk-heads", type=int, default=16)
    a = ap.parse_args()
    g = torch.Generator(device="cuda").manual_seed(0)
    t, hk, hv, d = a.tokens, a.qk_heads, a.heads, 128
    q = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g)) * d ** -0.5
    k = ref.l2norm(torch.randn(t, hk, d, device="cuda", generator=g))
    v = torch.randn(t, hv, d, device="cuda", generator=g)
    gate = -torch.rand(t, hv, device="cuda", generator=g) * 0.2
    beta = torch.rand(t, hv, device="cuda", generator=g)

    def timed(fn, n=5):
        for _ in range(2):
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
    print(json.dumps({"op": "gdn_scan", "tokens": t, "value_heads": hv, "kernel_path_ms": round(kernel_ms, 3), "torch_loop_ms": round(torch_ms, 3),
                      "operands_ms": round(operands_ms, 3), "max_abs_diff": float((o1 - o2).abs().max())}))


if __name__ == "__main__":
    main()

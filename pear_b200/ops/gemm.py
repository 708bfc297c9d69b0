"""bf16 GEMM bindings: ``C = A @ B^T`` on the tcgen05/TMEM/TMA kernel (``csrc/gemm_tcgen05.cu``).

``linear_bf16`` is the forward of every bf16 linear layer of the trainer model; its backward (dX = dY @ W,
dW = dY^T @ X) runs on the same kernel's MN-major operand forms (``gemm_nn``, ``gemm_tn``): no library GEMM in a linear
layer's forward or backward.
"""

from __future__ import annotations

import ctypes

import torch

from .lib import check, count_launch, lib, ptr, stream

_status = {}
_sms = {}


def _dev_state(device: torch.device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
        _sms[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _status[key], _sms[key]


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out_dtype=torch.float32, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a`` [M, K] bf16, ``b`` [N, K] bf16 (row-major, K contiguous) -> [M, N] in fp32 or bf16."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape[1] == b.shape[1]
    if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
        a = a.contiguous()
    if b.stride(1) != 1 or b.stride(0) % 8 or b.data_ptr() % 16:
        b = b.contiguous()
    m, k = a.shape
    n = b.shape[0]
    if k % 8:
        raise ValueError("K must be a multiple of 8 (16-byte rows for TMA)")
    c = out if out is not None else torch.empty(m, n, dtype=out_dtype, device=a.device)
    status, sms = _dev_state(a.device)
    check(lib().pear_gemm_bf16_nt(ptr(a), ptr(b), ptr(c), m, n, k, a.stride(0), b.stride(0), c.stride(0),
                                  1 if c.dtype == torch.bfloat16 else 0, ptr(status), sms, stream()), "gemm_bf16_nt")
    count_launch()
    return c


def _aligned(t: torch.Tensor) -> torch.Tensor:
    return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """``a`` [M, K] @ ``b`` [K, N], both row-major bf16 (``b`` is read MN-major: no transpose is materialised). The input
    gradient of a linear layer: dX = dY @ W."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape[1] == b.shape[0]
    a, b = _aligned(a), _aligned(b)
    m, k = a.shape
    n = b.shape[1]
    if k % 8 or n % 8:
        return (a.float() @ b.float()).to(out_dtype)
    c = torch.empty(m, n, dtype=out_dtype, device=a.device)
    status, sms = _dev_state(a.device)
    check(lib().pear_gemm_bf16_form(ptr(a), ptr(b), ptr(c), m, n, k, a.stride(0), b.stride(0), c.stride(0), 0, 1,
                                    1 if c.dtype == torch.bfloat16 else 0, ptr(status), sms, stream()), "gemm_bf16_nn")
    count_launch()
    return c


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """``a`` [K, M]^T @ ``b`` [K, N], both row-major bf16 and both read MN-major. The weight gradient of a linear layer:
    dW = dY^T @ X (the reduction runs over the tokens)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.shape[0] == b.shape[0]
    a, b = _aligned(a), _aligned(b)
    k, m = a.shape
    n = b.shape[1]
    if m % 8 or n % 8:
        return (a.float().t() @ b.float()).to(out_dtype)
    c = torch.empty(m, n, dtype=out_dtype, device=a.device)
    status, sms = _dev_state(a.device)
    check(lib().pear_gemm_bf16_form(ptr(a), ptr(b), ptr(c), m, n, k, a.stride(0), b.stride(0), c.stride(0), 1, 1,
                                    1 if c.dtype == torch.bfloat16 else 0, ptr(status), sms, stream()), "gemm_bf16_tn")
    count_launch()
    return c


def split_operand(x: torch.Tensor, role: str) -> torch.Tensor:
    """fp32 [R, K] -> bf16 [R, 3K] for :func:`matmul_split3`: ``x = hi + lo`` with ``hi = bf16(x)``, ``lo = bf16(x - hi)``;
    role "a" lays out [hi | hi | lo], role "b" [hi | lo | hi], so that one K-concatenated GEMM sums hi.hi + hi.lo + lo.hi."""
    xf = x.float()
    hi = xf.to(torch.bfloat16)
    lo = (xf - hi.float()).to(torch.bfloat16)
    return torch.cat([hi, hi, lo] if role == "a" else [hi, lo, hi], dim=1)


def matmul_split3(a: torch.Tensor, b: torch.Tensor, b_split: torch.Tensor | None = None) -> torch.Tensor:
    """``a @ b^T`` for fp32 ``a`` [M, K], ``b`` [N, K] on the bf16 tensor cores with close to fp32 accuracy: both operands are
    split into two bf16 terms and the three leading products are accumulated in fp32 by ONE GEMM over 3K (the lo.lo term,
    2^-16 of the result, is dropped). The fp32 head of the trainer uses it (upstream keeps the head in fp32 through a
    two-term fp16 operand scheme: pear/models/qwen3_5/trainer/operands.py). ``b_split`` = ``split_operand(b, "b")`` when
    the caller reuses it over several calls."""
    if a.shape[1] % 8:
        return a.float() @ b.float().t()
    bs = b_split if b_split is not None else split_operand(b, "b")
    return gemm_nt(split_operand(a, "a"), bs, torch.float32)


def gemm_status(device=None) -> int:
    status, _ = _dev_state(torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device))
    return int(status.item())


class _LinearBF16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, output_unused=False):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16)
        ctx.save_for_backward(x2, weight)
        ctx.in_dtype, ctx.shape = x.dtype, shape
        if output_unused:  # a checkpoint recompute whose caller only backpropagates through this node: no GEMM
            y = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.float32, device=x.device)
        else:
            y = gemm_nt(x2, weight, torch.float32)
        return y.view(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16)
        dx = dw = None
        # both products on the own kernel's MN-major operand forms (fp32 accumulation and fp32 results: the weight gradient
        # is accumulated over micro-batches in fp32)
        if ctx.needs_input_grad[0]:
            dx = gemm_nn(dy2, weight, torch.float32).to(ctx.in_dtype).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw = gemm_tn(dy2, x2, torch.float32).to(weight.dtype)
        return dx, dw, None


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, output_unused: bool = False) -> torch.Tensor:
    """``output_unused``: the forward value is never read (the last GEMM of a layer inside a checkpoint recompute, upstream
    ``trainer/mlp.py:132-134``): the node is built for the backward, the forward GEMM is skipped."""
    if weight.shape[1] % 8 or x.numel() == 0:
        return torch.nn.functional.linear(x.to(weight.dtype), weight).float()
    return _LinearBF16.apply(x, weight, output_unused)


def _main() -> None:
    """``python -m pear_b200.ops.gemm M N K [--iters I]``: time the tcgen05 GEMM against cuBLAS (CUDA events, L2 flushed
    between iterations) and print one JSON line; the command profiles of this kernel are taken with."""
    import argparse
    import json

    ap = argparse.ArgumentParser()
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(a.m, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2

    def timed(fn) -> float:
        for _ in range(a.warmup):
            fn()
        total = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / a.iters

    out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device="cuda")
    t_own = timed(lambda: gemm_nt(x, w, torch.bfloat16, out=out))
    t_lib = timed(lambda: torch.matmul(x, w.t(), out=out))
    ref = x.float() @ w.float().t()
    err = float((gemm_nt(x, w, torch.float32) - ref).abs().max() / ref.abs().max())
    fl = 2.0 * a.m * a.n * a.k
    print(json.dumps({"m": a.m, "n": a.n, "k": a.k, "tcgen05_ms": round(t_own, 4), "cublas_ms": round(t_lib, 4),
                      "tcgen05_tflops": round(fl / t_own / 1e9, 1), "cublas_tflops": round(fl / t_lib / 1e9, 1),
                      "rel_err": err, "status": gemm_status()}))


if __name__ == "__main__":
    _main()

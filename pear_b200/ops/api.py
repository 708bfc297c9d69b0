"""The op surface the models call. CPU tensors run the fp32 torch statement in :mod:`reference`; CUDA tensors run the
sm_100a kernels of :mod:`pear_b200.ops.kernels` (which raise if the in-tree extension is missing on a GPU machine,
so a GPU run can never silently fall back to eager torch for an op that has a kernel).

The role of upstream ``pear/models/kernels.py`` + ``pear/models/qwen3_5/trainer/training_kernels.py``: one seam
through which a model family's kernels are installed under a generic model.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import reference as ref


def _k():
    from . import kernels

    return kernels


def _cuda(*tensors) -> bool:
    return any(t is not None and torch.is_tensor(t) and t.is_cuda for t in tensors)


# when set (tests, baseline arm of a benchmark) CUDA tensors also take the torch statement
FORCE_REFERENCE = False
PRECISE_OPERANDS = False  # set during an overflow rerun: GEMM operands stay fp32 (IEEE fp32 library GEMM) instead of bf16


def _use_kernels(*tensors) -> bool:
    return _cuda(*tensors) and not FORCE_REFERENCE


def linear(x: torch.Tensor, weight: torch.Tensor, output_unused: bool = False) -> torch.Tensor:
    """``x @ weight^T`` with operands in the weight's dtype, fp32 result. While ``PRECISE_OPERANDS`` is set (the rerun of
    a batch whose fast pass produced a non-finite loss) both operands are taken to fp32 and multiplied without any
    reduced-precision tensor-core mode: slower, with the full fp32 range and mantissa."""
    if PRECISE_OPERANDS:
        return F.linear(x.float(), weight.float())
    if _use_kernels(x, weight) and weight.dtype == torch.bfloat16:
        return _k().linear_bf16(x, weight, output_unused)
    return F.linear(x.to(weight.dtype), weight).float()


def rms_norm(x, weight, eps=1e-6, one_plus=True):
    if _use_kernels(x):
        return _k().rms_norm(x, weight, eps, one_plus)
    return ref.rms_norm(x, weight, eps, one_plus)


def add_rms_norm(x, residual, weight, eps=1e-6):
    if _use_kernels(x):
        return _k().add_rms_norm(x, residual, weight, eps)
    return ref.add_rms_norm(x, residual, weight, eps)


def gated_rms_norm(o, z, weight, eps=1e-6):
    if _use_kernels(o):
        return _k().gated_rms_norm(o, z, weight, eps)
    return ref.gated_rms_norm(o, z, weight, eps)


def swiglu(gate, up):
    if _use_kernels(gate):
        return _k().swiglu(gate, up)
    return ref.swiglu(gate, up)


def sigmoid_gate(x, gate):
    if _use_kernels(x):
        return _k().sigmoid_gate(x, gate)
    return ref.sigmoid_gate(x, gate)


def l2norm(x, eps=1e-6):
    return ref.l2norm(x, eps)


def mrope_cos_sin(position_ids, rotary_dim, theta, sections):
    return ref.mrope_cos_sin(position_ids, rotary_dim, theta, sections)


def apply_rope(x, cos, sin):
    if _use_kernels(x):
        return _k().apply_rope(x, cos, sin)
    return ref.apply_rope(x, cos, sin)


def causal_attention(q, k, v, cu_seqlens, scale=None):
    if _use_kernels(q):
        return _k().causal_attention(q, k, v, cu_seqlens, scale)
    return ref.causal_attention(q, k, v, cu_seqlens, scale)


def causal_conv_silu(x, weight, bounds, init_state=None):
    if _use_kernels(x):
        return _k().causal_conv_silu(x, weight, bounds, init_state)
    return ref.causal_conv_silu(x, weight, bounds, init_state)


def gdn_gates(a, b, A_log, dt_bias):
    return ref.gdn_gates(a, b, A_log, dt_bias)


def gdn_scan(q, k, v, g, beta, state=None):
    """One sequence; returns (o, final_state)."""
    if _use_kernels(q):
        return _k().gdn_scan(q, k, v, g, beta, state)
    return ref.gdn_chunked(q, k, v, g, beta, state)


def gdn_scan_packed(q, k, v, g, beta, bounds, init_states=None, return_states: bool = False):
    """Packed sequences delimited by ``bounds`` (a list of cut points); state never crosses a boundary."""
    outs, finals = [], []
    for i, (s, e) in enumerate(zip(bounds[:-1], bounds[1:])):
        st = init_states[i] if init_states is not None else None
        o, f = gdn_scan(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e], st)
        outs.append(o)
        finals.append(f)
    o = torch.cat(outs, dim=0) if outs else v.new_zeros(v.shape, dtype=torch.float32)
    return (o, finals) if return_states else o


def logprob_entropy(hidden, weight, ids, temperature=1.0, chunk=4096):
    if _use_kernels(hidden):
        return _k().logprob_entropy(hidden, weight, ids, temperature, chunk)
    return ref.logprob_entropy(hidden, weight, ids, temperature, chunk)

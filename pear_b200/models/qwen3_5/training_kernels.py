"""Training kernel façade of the family (upstream ``trainer/training_kernels.py:21-112``).

Install order on any device: fp32 residual stream -> fp32 head (fused log-prob / entropy, logits never stored whole)
-> precise RMSNorm; on a B200 ``install_gpu_backend`` then routes the module's ops to the CUDA kernels through
``pear_b200.ops.api`` (CUDA tensors dispatch to the kernels, CPU tensors to the fp32 reference). ``run_checked``
implements the overflow rerun of upstream ``operands.py:105-122``: the fast path runs GEMM operands in bf16 with a
device-side non-finite flag on the loss; if it is raised the whole batch reruns with fp32 operands.
"""

from __future__ import annotations

from typing import Any, Callable

import torch

from ...ops import api as ops
from ..hybrid import HybridForCausalLM
from ..kernels import TrainingKernels
from .gpu_backend import REQUIREMENTS, GpuGeneration, detect


class Qwen3_5TrainingKernels(TrainingKernels):
    overflow_reruns = 0
    _precise = False

    @classmethod
    def check_config(cls, engine_config) -> None:
        REQUIREMENTS.check_training(engine_config)

    @classmethod
    def install(cls, module, fp32_residual: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        if not isinstance(module, HybridForCausalLM):
            raise TypeError("these kernels serve HybridForCausalLM")
        module.fp32_residual = bool(fp32_residual)
        module.use_fused_head = bool(use_fused_kernels)

    @classmethod
    def check_model(cls, module, use_remove_padding: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        if not use_remove_padding:
            raise ValueError("the kernels take packed (padding-free) batches: use_remove_padding must be true")
        if not use_fused_kernels:
            raise ValueError("the fused head is the only path that never materialises the logits: use_fused_kernels must be true")

    @classmethod
    def install_gpu_backend(cls, module) -> None:
        if detect() is GpuGeneration.NONE:
            return  # CPU plumbing: reference ops
        ops.FORCE_REFERENCE = False
        from ...ops import lib
        lib.lib()  # fail loudly now if the extension is missing on a GPU box

    @classmethod
    def install_checkpointing(cls, module) -> None:
        module.recompute_skips_down_proj = True  # a recompute only needs what the backward reads (upstream mlp.py:132-134)

    @classmethod
    def run_checked(cls, run: Callable[[], Any], before_rerun: Callable[[], None]) -> Any:
        out = run()
        bad = False
        if isinstance(out, dict):
            bad = any(isinstance(v, float) and (v != v or v in (float("inf"), float("-inf"))) for v in out.values())
        if not bad:
            return out
        cls.overflow_reruns += 1
        before_rerun()
        prev = torch.get_float32_matmul_precision()
        torch.set_float32_matmul_precision("highest")
        ops.PRECISE_OPERANDS = True
        try:
            return run()
        finally:
            ops.PRECISE_OPERANDS = False
            torch.set_float32_matmul_precision(prev)

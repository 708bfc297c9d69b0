"""Rollout kernel façade of the family (upstream ``rollout/rollout_kernels.py:9-72``, ``gpu_backend.py:10-65``)."""

from __future__ import annotations

from ..hybrid import HybridForCausalLM
from ..kernels import RolloutKernels
from .gpu_backend import REQUIREMENTS, GpuGeneration, detect


class Qwen3_5RolloutKernels(RolloutKernels):
    @classmethod
    def configure_server(cls, engine_config: dict, max_num_seqs: int, max_num_batched_tokens: int) -> None:
        REQUIREMENTS.check_rollout(engine_config)
        engine_config.setdefault("block_size", 16)
        # decode / verify rows run the batched GPU-resident step (rollout/fast_step.py). It has ONE shape, max_num_seqs x
        # (1 + drafts) rows with empty batch slots skipped inside every kernel, so a single captured CUDA graph serves every
        # batch size (upstream captures one graph per token-count bucket: rollout/blackwell/cudagraph.py:4-34)
        engine_config.setdefault("fast_decode", True)
        engine_config["max_num_seqs"] = max_num_seqs
        engine_config["max_num_batched_tokens"] = max_num_batched_tokens

    @classmethod
    def install_worker(cls, engine) -> None:
        if detect() is GpuGeneration.NONE:
            return
        from ...ops import lib
        lib.lib()

    @classmethod
    def check_model(cls, model, engine_config) -> None:
        if not isinstance(model, HybridForCausalLM):
            raise TypeError(f"expected the hybrid GDN + attention model, got {type(model).__name__}")

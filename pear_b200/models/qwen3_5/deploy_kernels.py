"""Deploy kernel façade of the family: the batch-1 NVFP4 decode megakernel (upstream ``deploy/blackwell/nvfp4/runner.py:
228-703`` patches a vLLM runner so that a single request's decode/verify step is one launch; here the engine IS the
runner)."""

from __future__ import annotations

from typing import Optional

from ..kernels import DeployKernels
from .gpu_backend import GpuGeneration, detect


class Qwen3_5DeployKernels(DeployKernels):
    @classmethod
    def configure_server(cls, engine_config: dict, max_num_seqs: int, max_num_batched_tokens: int) -> None:
        if max_num_seqs != 1:
            raise ValueError("the decode megakernel serves one session at a time (max_num_seqs 1)")
        engine_config["max_num_seqs"] = 1
        engine_config.setdefault("max_model_len", 260096)

    @classmethod
    def build_engine(cls, model_dir: Optional[str], draft_dir, engine_config: dict):
        if detect() is GpuGeneration.NONE:
            raise RuntimeError("the decode megakernel needs a B200")
        from ...deploy.engine import MegakernelEngine, ModuleWeights, RandomWeights
        from .. import io as model_io
        from ..config import HybridConfig
        from ..hybrid import HybridForCausalLM

        max_len = int(engine_config.get("max_model_len", 8192))
        n_draft = int(engine_config.get("num_speculative_tokens", 3))
        if model_dir is None or str(model_dir).startswith("preset:"):
            cfg = getattr(HybridConfig, str(model_dir or "preset:qwen3_8_27b").split(":", 1)[1])()
            weights = RandomWeights("cuda", seed=int(engine_config.get("seed", 0)))
        else:
            cfg = model_io.load_config(model_dir)
            m = HybridForCausalLM(cfg, with_mtp=False)
            model_io.load_model_dir(model_dir, m)
            drafter = None
            if n_draft > 0:
                from ..drafter import BlockDrafter
                drafter = BlockDrafter(HybridConfig.drafter(cfg.hidden_size, cfg.vocab_size))
                if draft_dir:
                    model_io.load_model_dir(draft_dir, drafter)
            weights = ModuleWeights(m, drafter, "cuda")
        dcfg = HybridConfig.drafter(cfg.hidden_size, cfg.vocab_size) if n_draft > 0 else None
        return MegakernelEngine(cfg, dcfg, weights, max_len=max_len, n_draft=n_draft, seed=int(engine_config.get("seed", 0)))

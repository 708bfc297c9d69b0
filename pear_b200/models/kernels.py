"""Hooks through which a model family installs its kernels under the generic trainer, rollout engine and deploy server.

The three ABCs mirror upstream ``pear/models/kernels.py`` (``TrainingKernels`` :16, ``RolloutKernels`` :60,
``DeployKernels`` :107): classes are named by class path in the recipe (``actor.fsdp_config.kernels``,
``rollout.kernels``, ``kernels`` of the server config) and exported to child processes through environment variables.
The generic runtime never names a model family (tests/test_layering.py).
"""

from __future__ import annotations

import importlib
import os
from abc import ABC, abstractmethod
from typing import Any, Callable


def _from_env(env: str):
    path = os.environ.get(env)
    if not path:
        return None
    module_path, _, class_name = path.rpartition(".")
    return getattr(importlib.import_module(module_path), class_name)


class TrainingKernels(ABC):
    """A family's training kernels for the module the engine built."""

    @classmethod
    @abstractmethod
    def check_config(cls, engine_config) -> None:
        """Called first, with the trainer engine's config and no module yet: refuse (raise) settings the family's GPU code cannot honour."""

    @classmethod
    @abstractmethod
    def install(cls, module, fp32_residual: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        """Device-independent changes to the freshly built, still unsharded module (precision of the residual stream, which head it uses)."""

    @classmethod
    @abstractmethod
    def check_model(cls, module, use_remove_padding: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        """Second check, now with the module: the options chosen must be the ones whose code paths the family's kernels stand in for."""

    @classmethod
    @abstractmethod
    def install_gpu_backend(cls, module) -> None:
        """Select the kernels for the GPU this process sees; runs after ``install`` and before the parameters are sharded."""

    @classmethod
    @abstractmethod
    def install_checkpointing(cls, module) -> None:
        """Tell the gradient-checkpointing layer runner what this family's recompute pass may leave out or must keep."""

    @classmethod
    @abstractmethod
    def run_checked(cls, run: Callable[[], Any], before_rerun: Callable[[], None]) -> Any:
        """Call ``run``; if its result shows the fast numeric path failed (non-finite loss), call ``before_rerun`` and run once more on the safe path."""


class _Exported(ABC):
    ENV = ""

    @classmethod
    def export(cls, path: str):
        os.environ[cls.ENV] = path
        return cls.from_env()

    @classmethod
    def from_env(cls):
        return _from_env(cls.ENV)

    @classmethod
    def is_enabled(cls) -> bool:
        return cls.from_env() is cls


class RolloutKernels(_Exported):
    """A family's model runner pieces for the rollout replicas."""

    ENV = "PEAR_ROLLOUT_KERNELS"

    @classmethod
    @abstractmethod
    def configure_server(cls, engine_config: dict, max_num_seqs: int, max_num_batched_tokens: int) -> None:
        """Fill in the engine settings this family needs (KV page size, batched-step switch, token budget) in the launcher's process."""

    @classmethod
    @abstractmethod
    def install_worker(cls, engine) -> None:
        """Runs inside a replica before its model exists: load the kernel library so a missing build fails here, not mid-step."""

    @classmethod
    @abstractmethod
    def check_model(cls, model, engine_config) -> None:
        """Refuse a replica whose model is not the architecture these kernels were written for."""


class DeployKernels(_Exported):
    """A family's kernels for a server of one session (the batch-1 decode megakernel)."""

    ENV = "PEAR_DEPLOY_KERNELS"

    @classmethod
    @abstractmethod
    def configure_server(cls, engine_config: dict, max_num_seqs: int, max_num_batched_tokens: int) -> None:
        ...

    @classmethod
    @abstractmethod
    def build_engine(cls, model_dir: str, draft_dir, engine_config: dict):
        """The decode engine for one session on this process's GPU."""

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
        """Raise unless the engine config is one the GPU backend computes under, before the module is built."""

    @classmethod
    @abstractmethod
    def install(cls, module, fp32_residual: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        """Apply what the family installs on any device, before the module is sharded."""

    @classmethod
    @abstractmethod
    def check_model(cls, module, use_remove_padding: bool, use_fused_kernels: bool, fused_kernels_backend) -> None:
        """Raise unless the module runs the paths the GPU backend replaces."""

    @classmethod
    @abstractmethod
    def install_gpu_backend(cls, module) -> None:
        """Patch the module with the backend of the process's GPU after install(), before sharding."""

    @classmethod
    @abstractmethod
    def install_checkpointing(cls, module) -> None:
        """Extend the module's gradient checkpoints with what the GPU backend needs in a recompute."""

    @classmethod
    @abstractmethod
    def run_checked(cls, run: Callable[[], Any], before_rerun: Callable[[], None]) -> Any:
        """The result of run() on the fast path, or after before_rerun() of a second run() off it."""


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
        """Settings of the process that builds the engine config (graph capture sizes, block size ...)."""

    @classmethod
    @abstractmethod
    def install_worker(cls, engine) -> None:
        """Install the family's kernels in a worker before it builds its model."""

    @classmethod
    @abstractmethod
    def check_model(cls, model, engine_config) -> None:
        """Raise unless a worker built the family's model."""


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

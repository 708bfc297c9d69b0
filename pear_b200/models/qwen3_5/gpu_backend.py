"""GPU generation and backend selection (upstream ``pear/models/qwen3_5/gpu_generation.py:4-21``,
``gpu_backend.py:12-69``).

Upstream picks the first backend whose compute capability and engine config match among HOPPER (9,0),
DATACENTER_BLACKWELL (10,*), BLACKWELL_ULTRA (10,3) and RTX_BLACKWELL (12,0). This framework is written for ONE
generation: datacenter Blackwell, sm_100a (B200). Every other capability is refused by name instead of being
dispatched to a second code path, and a process without a GPU runs the fp32 reference ops (CPU plumbing and tests).
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Optional

import torch


class GpuGeneration(str, Enum):
    NONE = "none"                         # no GPU: reference ops
    DATACENTER_BLACKWELL = "sm_100a"      # B200: the only generation with kernels here


SUPPORTED_CAPABILITY = (10, 0)


def detect(device: Optional[int] = None) -> GpuGeneration:
    if not torch.cuda.is_available():
        return GpuGeneration.NONE
    cap = torch.cuda.get_device_capability(device if device is not None else torch.cuda.current_device())
    if cap != SUPPORTED_CAPABILITY:
        raise RuntimeError(f"compute capability {cap[0]}.{cap[1]} has no backend: the kernels are built for sm_100a (B200) only")
    return GpuGeneration.DATACENTER_BLACKWELL


@dataclass(frozen=True)
class BackendRequirements:
    """What an engine config must satisfy for the GPU backend (upstream ``training_kernels.py:34-46`` requires FSDP2,
    an fp32 residual stream and fp32 modules on TF32)."""

    fp32_residual: bool = True
    remove_padding: bool = True
    max_tp: int = 8

    def check_training(self, engine_config) -> None:
        if getattr(engine_config, "param_dtype", "bf16") not in ("bf16", "fp32"):
            raise ValueError("the sm_100a training kernels compute in bf16 with fp32 accumulation (param_dtype bf16 or fp32)")

    def check_rollout(self, engine_config: dict) -> None:
        tp = int(engine_config.get("tensor_parallel_size", 1))
        if tp < 1 or tp > self.max_tp or (tp & (tp - 1)):
            raise ValueError(f"tensor_parallel_size {tp}: the NVSwitch kernels take a power of two up to {self.max_tp}")
        if int(engine_config.get("block_size", 16)) != 16:
            raise ValueError("paged attention kernels are built for 16-token blocks")


REQUIREMENTS = BackendRequirements()

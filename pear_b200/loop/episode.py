"""Episode record and end reasons (upstream ``pear/agent_loop/episode.py:9-56``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Optional


class EndReason(str, Enum):
    ENV = "env"        # the environment ended the episode (done)
    PARSE = "parse"    # the model's answer had no valid action
    BUDGET = "budget"  # the episode's token budget ran out
    LOST = "lost"      # the environment process was lost more often than restarts allow
    ABORTED = "aborted"


class LoopState(str, Enum):
    PENDING = "pending"
    GENERATING = "generating"
    PROCESSING_TOOLS = "processing_tools"
    TERMINATED = "terminated"


@dataclass
class Episode:
    env_args: dict
    family: str
    uid: str = ""
    session: str = "0"
    turns: int = 0
    restarts: int = 0
    end_reason: Optional[EndReason] = None
    success: bool = False
    # the trajectory, token by token
    tokens: list[int] = field(default_factory=list)
    response_mask: list[int] = field(default_factory=list)      # 1 = sampled by the policy, 0 = prompt / user turns
    logprobs: list[float] = field(default_factory=list)          # rollout log-prob at sampled tokens, 0 elsewhere
    topk_ids: list[list[int]] = field(default_factory=list)      # rollout top-k head ids (placeholders on masked tokens)
    topk_logprobs: list[list[float]] = field(default_factory=list)
    embeds: list = field(default_factory=list)                   # (position, [tokens, hidden] array) vision blocks
    grids: list = field(default_factory=list)                    # (rows, columns) of every picture's block, in token order (checkpoint positions)
    images: list = field(default_factory=list)                   # (position, uint8 [H, W, 3] picture) of the blocks that came from pixels
    prompt_len: int = 0
    policy_versions: list[int] = field(default_factory=list)

    @property
    def response_tokens(self) -> int:
        return sum(self.response_mask)

"""NVTX ranges around the phases a timeline viewer should show (trainer phases, rollout steps, weight sync).

Off by default: ``PEAR_NVTX=1`` (or :func:`enable`) turns :func:`annotate` into ``torch.cuda.nvtx`` push / pop pairs; without
it, or without CUDA, it costs one attribute test. Upstream marks the same places through torch.profiler record functions
(``pear/trainer/trainer.py`` phase timers, ``pear/rollout/monitor.py``).
"""

from __future__ import annotations

import contextlib
import os

import torch

_enabled = os.environ.get("PEAR_NVTX", "0") == "1"
ranges_opened = 0  # for tests: how many ranges were pushed


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled and torch.cuda.is_available()


@contextlib.contextmanager
def annotate(name: str):
    global ranges_opened
    if not enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    ranges_opened += 1
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()

"""Activation offload: checkpointed layers' inputs go to pinned host memory on a side stream during forward and come
back, one layer ahead of use, during backward (upstream ``3rdparty/verl/patches/0032-*``: ``CheckpointInputOffload``).

The copies run on the copy engines (no kernel): D2H on ``d2h_stream`` after an event on the compute stream, H2D on
``h2d_stream``; the compute stream only waits on the event of the tensor it needs. Pinned buffers are pooled by size so
a step allocates nothing after the first one. On CPU tensors the manager keeps references (no copies).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class _Slot:
    host: Optional[torch.Tensor]
    shape: tuple
    dtype: torch.dtype
    device: torch.device
    d2h_done: Optional[object] = None
    dev: Optional[torch.Tensor] = None
    h2d_done: Optional[object] = None
    keep: Optional[torch.Tensor] = None


class CheckpointInputOffload:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.slots: dict[int, _Slot] = {}
        self.pool: dict[tuple, list[torch.Tensor]] = {}
        self.d2h_stream = self.h2d_stream = None
        self.bytes_offloaded = 0

    def _streams(self, device) -> None:
        if self.d2h_stream is None:
            self.d2h_stream = torch.cuda.Stream(device)
            self.h2d_stream = torch.cuda.Stream(device)

    def _host(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        free = self.pool.get(key)
        if free:
            return free.pop()
        return torch.empty(shape, dtype=dtype).pin_memory()

    # -- forward ------------------------------------------------------------------------------------------------------
    def stash(self, i: int, t: torch.Tensor) -> int:
        if not (self.enabled and t.is_cuda):
            self.slots[i] = _Slot(None, tuple(t.shape), t.dtype, t.device, keep=t.detach())
            return i
        self._streams(t.device)
        host = self._host(t.shape, t.dtype)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(self.d2h_stream):
            self.d2h_stream.wait_event(ev)
            host.copy_(t.detach(), non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.d2h_stream)
        t.record_stream(self.d2h_stream)  # the device copy may be freed once the D2H has read it
        self.slots[i] = _Slot(host, tuple(t.shape), t.dtype, t.device, d2h_done=done)
        self.bytes_offloaded += t.numel() * t.element_size()
        return i

    # -- backward -----------------------------------------------------------------------------------------------------
    def prefetch(self, i: int) -> None:
        s = self.slots.get(i)
        if s is None or s.host is None or s.dev is not None:
            return
        with torch.cuda.stream(self.h2d_stream):
            self.h2d_stream.wait_event(s.d2h_done)
            s.dev = torch.empty(s.shape, dtype=s.dtype, device=s.device)
            s.dev.copy_(s.host, non_blocking=True)
            s.h2d_done = torch.cuda.Event()
            s.h2d_done.record(self.h2d_stream)

    def fetch(self, i: int) -> torch.Tensor:
        s = self.slots.pop(i)
        if s.host is None:
            return s.keep
        if s.dev is None:
            self.slots[i] = s
            self.prefetch(i)
            self.slots.pop(i)
        torch.cuda.current_stream(s.device).wait_event(s.h2d_done)
        s.dev.record_stream(torch.cuda.current_stream(s.device))
        self.pool.setdefault((s.shape, s.dtype), []).append(s.host)
        return s.dev

    def clear(self) -> None:
        for s in self.slots.values():
            if s.host is not None:
                self.pool.setdefault((s.shape, s.dtype), []).append(s.host)
        self.slots.clear()

"""AdamW whose fp32 moments live in pinned host memory and stream through the device during ``step()``.

Upstream ``pear/trainer/engine.py:155-309`` (``StreamedAdamW``): the step walks the parameters in chunks; for each
chunk the moments are copied host -> device on a dedicated stream into one of three staging slots, the fused update
runs on the compute stream, and the new moments go device -> host on a third stream, so copies of chunk ``i+1`` / ``i-1``
overlap the math of chunk ``i``. The result is bit-identical to ``torch.optim.AdamW`` with the same hyper-parameters
(tests/test_streamed_adamw.py). On CPU parameters the same chunk walk runs without streams.
"""

from __future__ import annotations

import math
from typing import Iterable

import torch


class StreamedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, chunk_bytes: int = 2 << 30, slots: int = 3):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.chunk_elems = max(1, chunk_bytes // 8)  # two fp32 moments per element
        self.nslots = slots
        self._streams = None
        self._staging: list[torch.Tensor] = []

    def _moments(self, p: torch.Tensor):
        st = self.state[p]
        if not st:
            st["step"] = 0
            pin = p.is_cuda
            st["exp_avg"] = torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin)
            st["exp_avg_sq"] = torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin)
        return st

    def _setup(self, device) -> None:
        if self._streams is None:
            self._streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
            self._staging = [torch.empty(2, self.chunk_elems, dtype=torch.float32, device=device) for _ in range(self.nslots)]

    @staticmethod
    def _update(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int, lr, b1, b2, eps, wd) -> None:
        """The single-tensor AdamW update of torch (same operation order, so results match bit for bit)."""
        p.mul_(1 - lr * wd)
        m.lerp_(g, 1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1 = 1 - b1 ** step
        bc2 = 1 - b2 ** step
        step_size = lr / bc1
        denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
        p.addcdiv_(m, denom, value=-step_size)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._moments(p)
                st["step"] += 1
                pf, gf = p.data.view(-1), p.grad.view(-1).float()
                n = pf.numel()
                if not p.is_cuda:
                    for s in range(0, n, self.chunk_elems):
                        e = min(n, s + self.chunk_elems)
                        self._update(pf[s:e], gf[s:e], st["exp_avg"][s:e], st["exp_avg_sq"][s:e], st["step"], lr, b1, b2, eps, wd)
                    continue
                self._setup(p.device)
                h2d, d2h = self._streams
                compute = torch.cuda.current_stream(p.device)
                chunks = [(s, min(n, s + self.chunk_elems)) for s in range(0, n, self.chunk_elems)]
                loaded: list = [None] * len(chunks)
                stored: list = [None] * self.nslots

                def load(ci: int) -> None:
                    s, e = chunks[ci]
                    slot = ci % self.nslots
                    with torch.cuda.stream(h2d):
                        if stored[slot] is not None:
                            h2d.wait_event(stored[slot])  # the slot's previous contents have reached the host
                        self._staging[slot][0, : e - s].copy_(st["exp_avg"][s:e], non_blocking=True)
                        self._staging[slot][1, : e - s].copy_(st["exp_avg_sq"][s:e], non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(h2d)
                    loaded[ci] = ev

                load(0)
                for ci, (s, e) in enumerate(chunks):
                    if ci + 1 < len(chunks):
                        load(ci + 1)
                    slot = ci % self.nslots
                    compute.wait_event(loaded[ci])
                    m, v = self._staging[slot][0, : e - s], self._staging[slot][1, : e - s]
                    self._update(pf[s:e], gf[s:e], m, v, st["step"], lr, b1, b2, eps, wd)
                    done = torch.cuda.Event()
                    done.record(compute)
                    with torch.cuda.stream(d2h):
                        d2h.wait_event(done)
                        st["exp_avg"][s:e].copy_(m, non_blocking=True)
                        st["exp_avg_sq"][s:e].copy_(v, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(d2h)
                    stored[slot] = ev
                for ev in stored:
                    if ev is not None:
                        compute.wait_event(ev)
        return loss

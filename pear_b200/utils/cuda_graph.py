"""CUDA-graph replay of launch-bound steps.

A decode step of the batched rollout path is a few hundred small launches; replaying it as one graph removes the host
launch cost (upstream captures piecewise / full graphs per token-count bucket: ``rollout/blackwell/cudagraph.py:4-34``,
``rollout/hopper/cudagraph.py:12-136``). ``GraphRunner`` captures a callable once per key (e.g. the padded token count)
over static input buffers and replays it afterwards; inputs are copied into the static buffers, outputs are views of the
captured outputs (valid until the next replay of the same key). Capture happens on a side stream after warm-up runs, so
lazy initialisation (workspace look-ups, module loads) never lands inside a capture.
"""

from __future__ import annotations

from typing import Callable, Hashable, Sequence

import torch


class GraphRunner:
    def __init__(self, fn: Callable[..., object], warmup: int = 2):
        self.fn, self.warmup = fn, warmup
        self.graphs: dict[Hashable, tuple[torch.cuda.CUDAGraph, list[torch.Tensor], object]] = {}
        self.replays = 0

    def _capture(self, key: Hashable, inputs: Sequence[torch.Tensor]):
        static = [t.clone() for t in inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):
                self.fn(*static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.fn(*static)
        self.graphs[key] = (graph, static, out)
        return self.graphs[key]

    def __call__(self, key: Hashable, *inputs: torch.Tensor):
        entry = self.graphs.get(key)
        if entry is None:
            entry = self._capture(key, inputs)
        graph, static, out = entry
        for s, t in zip(static, inputs):
            if s.shape != t.shape or s.dtype != t.dtype:
                raise ValueError(f"graph {key!r} was captured for {tuple(s.shape)} {s.dtype}, got {tuple(t.shape)} {t.dtype}")
            s.copy_(t)
        graph.replay()
        self.replays += 1
        return out

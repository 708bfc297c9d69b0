"""Episode dataset (upstream ``pear/agent_loop/dataset.py:15-66``): rows are the cartesian product of the environment
arguments listed in an episode JSON file, e.g. ``{"family": "synthetic", "args": {"task": ["reach"], "seed": [0, 1]}}``
gives one row per (task, seed)."""

from __future__ import annotations

import itertools
import json
import random
from dataclasses import dataclass
from typing import Iterator, Optional


@dataclass
class EpisodeRow:
    index: int
    family: str
    env_args: dict
    tool: str


class EpisodeDataset:
    def __init__(self, spec, shuffle: bool = True, seed: int = 0):
        if isinstance(spec, str):
            with open(spec) as f:
                spec = json.load(f)
        specs = spec if isinstance(spec, list) else [spec]
        self.rows: list[EpisodeRow] = []
        for s in specs:
            keys = sorted(s.get("args", {}))
            values = [v if isinstance(v, list) else [v] for v in (s["args"][k] for k in keys)]
            for combo in itertools.product(*values):
                self.rows.append(EpisodeRow(len(self.rows), s["family"], dict(zip(keys, combo)), s.get("tool", s["family"])))
        self.shuffle, self.seed = shuffle, seed
        self.epoch, self.cursor = 0, 0
        self._order = self._make_order()

    def _make_order(self) -> list[int]:
        order = list(range(len(self.rows)))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(order)
        return order

    def __len__(self) -> int:
        return len(self.rows)

    def next(self) -> EpisodeRow:
        """Endless stream: reshuffles at every epoch boundary."""
        if self.cursor >= len(self._order):
            self.epoch, self.cursor = self.epoch + 1, 0
            self._order = self._make_order()
        row = self.rows[self._order[self.cursor]]
        self.cursor += 1
        return row

    def __iter__(self) -> Iterator[EpisodeRow]:
        while True:
            yield self.next()

    # -- resume -------------------------------------------------------------------------------------------------------
    def state(self) -> dict:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed}

    def restore(self, state: Optional[dict]) -> None:
        if state:
            self.seed, self.epoch, self.cursor = state["seed"], state["epoch"], state["cursor"]
            self._order = self._make_order()

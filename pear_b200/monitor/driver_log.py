"""Parser of the driver's ``train.log`` (upstream ``pear/monitor/driver_log.py:13-117``): per step the metric line
``step:<k> - key:value - ...`` is split into phases (timing/*), rewards and staleness, so the panel can show where a
step's time went without talking to the trainer."""

from __future__ import annotations

import os
import re
from dataclasses import dataclass, field

_STEP = re.compile(r"^step:(\d+) - (.*)$")


@dataclass
class StepRecord:
    step: int
    values: dict[str, float] = field(default_factory=dict)

    @property
    def phases(self) -> dict[str, float]:
        return {k.split("/", 1)[1]: v for k, v in self.values.items() if k.startswith("timing/")}


class DriverLog:
    def __init__(self, path: str):
        self.path, self.offset = path, 0
        self.steps: list[StepRecord] = []

    def poll(self) -> list[StepRecord]:
        """Read what was appended since the last poll (the file may not exist yet, or may have been rotated)."""
        if not os.path.exists(self.path):
            return []
        if os.path.getsize(self.path) < self.offset:
            self.offset = 0
        new = []
        with open(self.path) as f:
            f.seek(self.offset)
            for line in f:
                if not line.endswith("\n"):
                    break  # a line still being written
                self.offset += len(line.encode())
                m = _STEP.match(line.strip())
                if not m:
                    continue
                rec = StepRecord(int(m.group(1)))
                for part in m.group(2).split(" - "):
                    k, _, v = part.partition(":")
                    try:
                        rec.values[k] = float(v)
                    except ValueError:
                        pass
                new.append(rec)
        self.steps += new
        return new

    def latest(self):
        return self.steps[-1] if self.steps else None

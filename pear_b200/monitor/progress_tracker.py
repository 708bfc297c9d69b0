"""Tracker of finished trajectories (upstream ``pear/monitor/progress_tracker.py:15-79``, a detached actor there): the
agent loop records every finished episode; the monitor reads running totals per family and end reason."""

from __future__ import annotations

import threading
import time
from collections import Counter, defaultdict, deque


class ProgressTracker:
    def __init__(self, window: int = 512):
        self.lock = threading.Lock()
        self.total = 0
        self.by_family: dict[str, Counter] = defaultdict(Counter)
        self.end_reasons: Counter = Counter()
        self.recent: deque = deque(maxlen=window)
        self.started = time.time()

    def record(self, uid: str, session: str, family: str, reward: float, turns: int, end_reason, tokens: int) -> None:
        with self.lock:
            self.total += 1
            f = self.by_family[family]
            f["episodes"] += 1
            f["successes"] += int(reward > 0)
            f["turns"] += turns
            f["tokens"] += tokens
            self.end_reasons[str(end_reason)] += 1
            self.recent.append((time.time(), family, reward, tokens))

    def snapshot(self) -> dict:
        with self.lock:
            now = time.time()
            rec = [r for r in self.recent if now - r[0] <= 60.0]
            return {
                "episodes": self.total, "elapsed_s": now - self.started,
                "families": {k: {"episodes": v["episodes"], "success_rate": v["successes"] / max(1, v["episodes"]),
                                 "mean_turns": v["turns"] / max(1, v["episodes"]), "mean_tokens": v["tokens"] / max(1, v["episodes"])}
                             for k, v in self.by_family.items()},
                "end_reasons": dict(self.end_reasons),
                "episodes_per_min": float(len(rec)), "tokens_per_s_recent": sum(r[3] for r in rec) / 60.0,
            }

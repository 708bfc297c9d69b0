"""The run's progress panel (upstream ``pear/monitor/progress_panel.py:29-298``): every ``interval_s`` seconds combine
the replica metrics, the trajectory tracker and the driver log into ``progress.json`` (machine readable) and
``progress.log`` (one text block per tick)."""

from __future__ import annotations

import json
import os
import threading
import time
from typing import Optional

from ..utils.files import atomic_write
from .driver_log import DriverLog
from .metrics import MetricsScraper
from .progress_tracker import ProgressTracker


class ProgressPanel:
    def __init__(self, run_dir: str, scraper: Optional[MetricsScraper] = None, tracker: Optional[ProgressTracker] = None,
                 interval_s: float = 10.0):
        self.run_dir, self.scraper, self.tracker, self.interval_s = run_dir, scraper, tracker, interval_s
        self.driver = DriverLog(os.path.join(run_dir, "train.log"))
        self.stop_flag = threading.Event()
        self.thread: Optional[threading.Thread] = None

    def tick(self) -> dict:
        self.driver.poll()
        state = {"time": time.time()}
        if self.scraper is not None:
            self.scraper.scrape()
            state["replicas"] = self.scraper.summary()
            state["replica_errors"] = dict(self.scraper.errors)
        if self.tracker is not None:
            state["trajectories"] = self.tracker.snapshot()
        last = self.driver.latest()
        if last is not None:
            state["trainer"] = {"step": last.step, "phases": last.phases,
                                "reward_mean": last.values.get("data/reward_mean"), "staleness": last.values.get("train/staleness_mean")}
        atomic_write(os.path.join(self.run_dir, "progress.json"), json.dumps(state, indent=1, default=float))
        with open(os.path.join(self.run_dir, "progress.log"), "a") as f:
            f.write(self.render(state) + "\n")
        return state

    @staticmethod
    def render(state: dict) -> str:
        lines = [time.strftime("== %Y-%m-%d %H:%M:%S", time.localtime(state["time"]))]
        tr = state.get("trainer")
        if tr:
            ph = " ".join(f"{k}={v:.1f}s" for k, v in sorted(tr["phases"].items()))
            lines.append(f"trainer  step {tr['step']}  reward {tr['reward_mean']}  staleness {tr['staleness']}  {ph}")
        rp = state.get("replicas")
        if rp:
            lines.append("replicas " + " ".join(f"{k.replace('pear_', '')}={v:.4g}" for k, v in sorted(rp.items())))
        tj = state.get("trajectories")
        if tj:
            fam = " ".join(f"{k}:{v['episodes']}ep/{v['success_rate']:.2f}" for k, v in sorted(tj["families"].items()))
            lines.append(f"episodes {tj['episodes']} ({tj['episodes_per_min']:.0f}/min)  {fam}  ends {tj['end_reasons']}")
        for name, err in state.get("replica_errors", {}).items():
            lines.append(f"replica {name} unreachable: {err}")
        return "\n".join(lines)

    def start(self) -> None:
        def loop():
            while not self.stop_flag.wait(self.interval_s):
                try:
                    self.tick()
                except Exception:  # noqa: BLE001 - the panel never takes the run down
                    pass
        self.thread = threading.Thread(target=loop, daemon=True, name="progress-panel")
        self.thread.start()

    def stop(self) -> None:
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=5)


def main(argv=None) -> int:
    """``python -m pear_b200.monitor.progress_panel --run-dir runs/x --replica replica-0=http://127.0.0.1:8100/metrics``: the
    monitor role as a process of its own: scrape the replicas, follow ``train.log`` and write ``progress.json`` /
    ``progress.log`` every ``--interval`` seconds until terminated (``--ticks N``: stop after N ticks)."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--run-dir", default=None)
    ap.add_argument("--replica", action="append", default=[], help="name=URL of a replica's /metrics (repeatable)")
    ap.add_argument("--interval", type=float, default=10.0)
    ap.add_argument("--ticks", type=int, default=0)
    args, overrides = ap.parse_known_args(argv)
    kv = dict(o.split("=", 1) for o in overrides if "=" in o and not o.startswith("-"))
    run_dir = args.run_dir or kv.get("run_dir", "runs/default")
    os.makedirs(run_dir, exist_ok=True)
    sources = dict(r.split("=", 1) for r in args.replica)
    panel = ProgressPanel(run_dir, MetricsScraper(sources) if sources else None, None, args.interval)
    n = 0
    while args.ticks <= 0 or n < args.ticks:
        panel.tick()
        n += 1
        if args.ticks > 0 and n >= args.ticks:
            break
        time.sleep(args.interval)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

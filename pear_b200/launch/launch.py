"""``python -m pear_b200.launch.launch <recipe> [--trainer-gpus N] [--rollout-tp T] [--dry-run] key=value ...``:
start the roles of a single-node run as child processes that die with this one; ``--dry-run`` prints the plan."""

from __future__ import annotations

import argparse
import json
import os
import sys

from ..utils.process import WorkerProcess  # noqa: F401  (re-exported for callers that supervise roles themselves)
from .roles import command, plan_node, raise_fd_limit


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("recipe")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--trainer-gpus", type=int, default=4)
    ap.add_argument("--rollout-tp", type=int, default=2)
    ap.add_argument("--dry-run", action="store_true")
    args, overrides = ap.parse_known_args(argv)
    plans = plan_node(args.gpus, args.trainer_gpus, args.rollout_tp, args.recipe, overrides)
    if args.dry_run:
        out = []
        for p in plans:
            for i in range(1 if p.role == "trainer" else p.processes):
                cmd, env = command(p, i)
                out.append({"role": p.role, "index": i, "cmd": cmd, "env": env})
        print(json.dumps(out, indent=1))
        return 0
    raise_fd_limit()
    import subprocess
    procs = []
    try:
        for p in plans:
            for i in range(1 if p.role == "trainer" else p.processes):
                cmd, env = command(p, i)
                procs.append(subprocess.Popen(cmd, env={**os.environ, **env}))
        return procs[0].wait()  # the trainer's exit ends the run
    finally:
        for pr in procs[1:]:
            pr.terminate()


if __name__ == "__main__":
    raise SystemExit(main())

"""``python -m pear_b200.launch.launch <recipe> [--trainer-gpus N] [--rollout-tp T] [--dry-run] key=value ...``:
start the roles of a single-node run as child processes that die with this one; ``--dry-run`` prints the plan."""

from __future__ import annotations

import argparse
import json
import os
import sys

from ..utils.process import WorkerProcess  # noqa: F401  (re-exported for callers that supervise roles themselves)
from .roles import command, plan_cluster, plan_node, raise_fd_limit


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("recipe")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--trainer-gpus", type=int, default=4)
    ap.add_argument("--rollout-tp", type=int, default=2)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--node-addrs", default="", help="several nodes: every node's address, comma-separated, the same list on every node (node 0 hosts the rendezvous)")
    ap.add_argument("--node-rank", type=int, default=0, help="this node's position in --node-addrs")
    ap.add_argument("--trainer-nodes", type=int, default=1, help="several nodes: the first K nodes train with all their GPUs, the others serve rollouts")
    ap.add_argument("--master-port", type=int, default=29500, help="rendezvous of the trainer ranks (replica i of several GPUs uses the next ports)")
    ap.add_argument("--replica-master-port", type=int, default=0, help="rendezvous of the ranks of replica 0 (replica i: + i; default: master-port + 1)")
    ap.add_argument("--rollout-port", type=int, default=8100)
    ap.add_argument("--env-port", type=int, default=8200)
    ap.add_argument("--sync-port", type=int, default=29650, help="rendezvous of the weight-sync world")
    args, overrides = ap.parse_known_args(argv)
    if args.node_addrs:
        plans = plan_cluster(args.node_addrs.split(","), args.node_rank, args.gpus, args.trainer_nodes, args.rollout_tp, args.recipe, overrides,
                             rollout_port=args.rollout_port, env_port=args.env_port, sync_port=args.sync_port)
    else:
        plans = plan_node(args.gpus, args.trainer_gpus, args.rollout_tp, args.recipe, overrides, rollout_port=args.rollout_port,
                          env_port=args.env_port, sync_port=args.sync_port)
    if args.dry_run:
        out = []
        for p in plans:
            for i in range(1 if p.role == "trainer" else p.processes):
                cmd, env = command(p, i, args.master_port, args.replica_master_port)
                out.append({"role": p.role, "index": i, "cmd": cmd, "env": env})
        print(json.dumps(out, indent=1))
        return 0
    raise_fd_limit()
    import signal
    import subprocess
    import time

    def on_signal(signum, frame):  # a terminated launcher takes its roles with it (the finally below)
        raise SystemExit(128 + signum)

    signal.signal(signal.SIGTERM, on_signal)
    signal.signal(signal.SIGINT, on_signal)
    procs = []
    try:
        for p in plans:
            for i in range(1 if p.role == "trainer" else p.processes):
                cmd, env = command(p, i, args.master_port, args.replica_master_port)
                # a session per role: the role's own children (torch.distributed.run workers, environment processes) form one
                # process group with it, which is what gets signalled at the end
                # the role's GPU set is the plan's; every other variable of `gpu_process_env` is a default the caller may override
                merged = {**env, **os.environ}
                if "CUDA_VISIBLE_DEVICES" in env:
                    merged["CUDA_VISIBLE_DEVICES"] = env["CUDA_VISIBLE_DEVICES"]
                procs.append(subprocess.Popen(cmd, env=merged, start_new_session=True))
        if plans[0].role == "trainer":
            return procs[0].wait()  # the trainer's exit ends the run (on the other trainer nodes: this node's ranks)
        rc = 0  # a node without trainer ranks runs until its replicas leave (they exit when the trainer's sync world is gone)
        for pr in procs:
            rc = pr.wait() or rc
        return rc
    finally:
        for pr in procs:
            if pr.poll() is None:
                try:
                    os.killpg(pr.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
        deadline = time.time() + 20
        for pr in procs:
            try:
                pr.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(pr.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass


if __name__ == "__main__":
    raise SystemExit(main())

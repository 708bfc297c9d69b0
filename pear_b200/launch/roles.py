"""Cluster roles and per-process environment (upstream ``scripts/start_ray_node.sh:58-61`` starts Ray nodes with the
custom resources trainer / rollout / robodojo / robolab; ``scripts/gpu_process_variables.sh:17-59`` sets the JIT-cache
and thread environment of GPU processes).

Without Ray a "role" is a set of processes started by ``launch.py``: trainer ranks under ``torch.distributed.run``,
rollout replicas (one process group per replica of ``tensor_model_parallel_size`` GPUs), environment server hosts and
the monitor. Roles map to GPU index ranges of a node; the plan is pure data so it can be checked without a cluster.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field


ROLLOUT_PORT, ENV_PORT, SYNC_PORT = 8100, 8200, 29650  # replica i serves on ROLLOUT_PORT + i, environment host j on ENV_PORT + j;
# the weight-sync world {trainer rank 0} + {replicas} meets on SYNC_PORT


@dataclass
class RolePlan:
    role: str
    processes: int
    gpus_per_process: int = 0
    gpu_offset: int = 0
    module: str = ""
    args: list[str] = field(default_factory=list)
    port: int = 0  # process i of the role listens on port + i
    # several nodes: the address this node's servers bind, the job-wide index of this node's first process of the role, and the
    # trainer's rendezvous (torch.distributed.run --nnodes / --node-rank / --master-addr)
    host: str = "127.0.0.1"
    index_offset: int = 0
    nnodes: int = 1
    node_rank: int = 0
    master_addr: str = "127.0.0.1"

    def gpu_ids(self, index: int) -> list[int]:
        lo = self.gpu_offset + index * self.gpus_per_process
        return list(range(lo, lo + self.gpus_per_process))


def plan_node(n_gpus: int, trainer_gpus: int, rollout_tp: int, recipe: str, overrides: list[str], env_hosts: int = 1,
              rollout_port: int = ROLLOUT_PORT, env_port: int = ENV_PORT, sync_port: int = SYNC_PORT) -> list[RolePlan]:
    """Split one node: the first ``trainer_gpus`` GPUs train, the rest serve rollouts in groups of ``rollout_tp``."""
    if trainer_gpus > n_gpus or (n_gpus - trainer_gpus) % max(1, rollout_tp):
        raise ValueError(f"{n_gpus} GPUs cannot hold {trainer_gpus} trainer GPUs plus rollout replicas of {rollout_tp}")
    replicas = (n_gpus - trainer_gpus) // max(1, rollout_tp)
    urls = ",".join(f"http://127.0.0.1:{rollout_port + i}" for i in range(replicas))
    remote = [f"actor_rollout_ref.rollout.checkpoint_engine.replica_urls=[{urls}]",
              f"actor_rollout_ref.rollout.checkpoint_engine.sync_master=127.0.0.1:{sync_port}",
              f"actor_rollout_ref.rollout.tensor_model_parallel_size={max(1, rollout_tp)}"] if replicas else []
    # both sides of the weight-sync world must name one backend: NCCL when both are on GPUs (each side's default), gloo when
    # the trainer has no GPU or the recipe asks for it
    force_gloo = trainer_gpus == 0 or "actor_rollout_ref.rollout.checkpoint_engine.backend=gloo" in overrides
    if force_gloo and replicas:
        remote.append("actor_rollout_ref.rollout.checkpoint_engine.backend=gloo")
    if env_hosts:  # the agent loop borrows environment processes from the env role's hosts
        remote.append("actor_rollout_ref.rollout.agent.env_hosts=[" + ",".join(f"http://127.0.0.1:{env_port + i}" for i in range(env_hosts)) + "]")
    return [
        # trainer_gpus = 0: one trainer process without a GPU (plumbing runs: a CPU trainer beside GPU replicas)
        RolePlan("trainer", max(1, trainer_gpus), 1 if trainer_gpus else 0, 0, "pear_b200.train.main", [recipe] + overrides + remote),
        RolePlan("rollout", replicas, rollout_tp, trainer_gpus, "pear_b200.rollout.server",
                 overrides + ["--sync-world", str(replicas * max(1, rollout_tp) + 1), "--sync-master", f"127.0.0.1:{sync_port}"]
                 + (["--sync-backend", "gloo"] if force_gloo else []), rollout_port),
        RolePlan("env", env_hosts, 0, 0, "pear_b200.sim.server", overrides, env_port),
        RolePlan("monitor", 1, 0, 0, "pear_b200.monitor.progress_panel",
                 overrides + [a for i in range(replicas) for a in ("--replica", f"replica-{i}=http://127.0.0.1:{rollout_port + i}/metrics")]),
    ]


def plan_cluster(node_addrs: list[str], node_rank: int, gpus_per_node: int, trainer_nodes: int, rollout_tp: int, recipe: str,
                 overrides: list[str], rollout_port: int = ROLLOUT_PORT, env_port: int = ENV_PORT, sync_port: int = SYNC_PORT) -> list[RolePlan]:
    """The roles of ONE node of a job over several: the first ``trainer_nodes`` nodes train with all their GPUs (one
    ``torch.distributed.run`` world over them, rendezvous on node 0), every other node serves rollouts in replicas of
    ``rollout_tp`` GPUs. The trainer's rank 0 (node 0) reaches every replica by its node's address and is rank 0 of the
    weight-sync world, whose rendezvous is on node 0 as well; node 0 also runs the environment host and the monitor. The same
    command line runs on every node with its own ``node_rank`` (upstream: scripts/start_ray_node.sh:58-61 gives each node its
    role through Ray resources)."""
    n = len(node_addrs)
    tp = max(1, rollout_tp)
    if not 0 < trainer_nodes < n or gpus_per_node % tp or not 0 <= node_rank < n:
        raise ValueError(f"{n} nodes of {gpus_per_node} GPUs: need 0 < trainer nodes ({trainer_nodes}) < nodes, replicas of {tp} GPUs that fill a node, "
                         f"and a node rank ({node_rank}) below {n}")
    per_node = gpus_per_node // tp
    replicas = (n - trainer_nodes) * per_node
    urls = [f"http://{node_addrs[trainer_nodes + r // per_node]}:{rollout_port + r % per_node}" for r in range(replicas)]
    sync_master = f"{node_addrs[0]}:{sync_port}"
    remote = [f"actor_rollout_ref.rollout.checkpoint_engine.replica_urls=[{','.join(urls)}]",
              f"actor_rollout_ref.rollout.checkpoint_engine.sync_master={sync_master}", f"actor_rollout_ref.rollout.tensor_model_parallel_size={tp}"]
    force_gloo = "actor_rollout_ref.rollout.checkpoint_engine.backend=gloo" in overrides
    plans: list[RolePlan] = []
    if node_rank < trainer_nodes:
        plans.append(RolePlan("trainer", gpus_per_node, 1, 0, "pear_b200.train.main", [recipe] + overrides + remote, nnodes=trainer_nodes,
                              node_rank=node_rank, master_addr=node_addrs[0]))
        if node_rank == 0:
            plans[0].args.append(f"actor_rollout_ref.rollout.agent.env_hosts=[http://{node_addrs[0]}:{env_port}]")
            plans.append(RolePlan("env", 1, 0, 0, "pear_b200.sim.server", overrides, env_port, host=node_addrs[0]))
            plans.append(RolePlan("monitor", 1, 0, 0, "pear_b200.monitor.progress_panel",
                                  overrides + [a for i, u in enumerate(urls) for a in ("--replica", f"replica-{i}={u}/metrics")]))
    else:
        plans.append(RolePlan("rollout", per_node, tp, 0, "pear_b200.rollout.server",
                              overrides + ["--sync-world", str(replicas * tp + 1), "--sync-master", sync_master, "--exit-with-trainer"]
                              + (["--sync-backend", "gloo"] if force_gloo else []), rollout_port, host=node_addrs[node_rank],
                              index_offset=(node_rank - trainer_nodes) * per_node))
    return plans


def gpu_process_env(gpu_ids: list[int], threads: int = 8, cache_dir: str = "") -> dict[str, str]:
    """Environment of one GPU process: visible devices, bounded host thread pools (many processes share a host),
    several NCCL communicators per GPU ordered by host issue order, build cache kept inside the tree."""
    env = {
        "CUDA_VISIBLE_DEVICES": ",".join(map(str, gpu_ids)),
        "OMP_NUM_THREADS": str(threads), "MKL_NUM_THREADS": str(threads), "TOKENIZERS_PARALLELISM": "false",
        "NCCL_LAUNCH_ORDER_IMPLICIT": "1", "NCCL_MNNVL_ENABLE": "0", "CUDA_DEVICE_MAX_CONNECTIONS": "32",
        "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
    }
    if cache_dir:
        env["PEAR_BUILD_DIR"] = cache_dir
    return env


def command(plan: RolePlan, index: int, master_port: int = 29500, replica_master_port: int = 0) -> tuple[list[str], dict[str, str]]:
    """``replica_master_port``: rendezvous of replica 0's ranks when a replica has several (replica i: + i); default: the ports
    after the trainer's."""
    env = gpu_process_env(plan.gpu_ids(index)) if plan.gpus_per_process else {}
    if plan.role == "trainer":
        cmd = ["python", "-m", "torch.distributed.run", f"--nnodes={plan.nnodes}", f"--nproc-per-node={plan.processes}", "--master-addr", plan.master_addr,
               "--master-port", str(master_port)] + ([f"--node-rank={plan.node_rank}"] if plan.nnodes > 1 else []) + ["-m", plan.module] + plan.args
        env = gpu_process_env(list(range(plan.gpu_offset, plan.gpu_offset + plan.processes)) if plan.gpus_per_process else [])
    else:
        cmd = ["python", "-m", plan.module] + plan.args
        if plan.role == "rollout":
            tp = max(1, plan.gpus_per_process)
            if tp > 1:  # the replica's ranks are a world of their own: rank 0 serves, the others follow in lock-step
                cmd = ["python", "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={tp}", "--master-addr", "127.0.0.1",
                       "--master-port", str((replica_master_port or master_port + 1) + index), "-m", plan.module] + plan.args
            job_index = plan.index_offset + index
            cmd += ["--port", str(plan.port + index), "--name", f"replica-{job_index}", "--sync-rank", str(1 + job_index * tp)]
            if plan.host != "127.0.0.1":
                cmd += ["--host", plan.host]
        elif plan.role == "env":
            cmd += ["--port", str(plan.port + index)] + (["--host", plan.host] if plan.host != "127.0.0.1" else [])
    return cmd, env


def raise_fd_limit(target: int = 65536) -> int:
    """Servers hold one pipe pair per environment process and one socket per session: lift the soft FD limit early
    (upstream presizes the FD table in a ``sitecustomize``)."""
    import resource
    soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
    new = min(target, hard) if hard != resource.RLIM_INFINITY else target
    if new > soft:
        resource.setrlimit(resource.RLIMIT_NOFILE, (new, hard))
    return max(new, soft)

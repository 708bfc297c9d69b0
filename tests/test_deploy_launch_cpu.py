"""Deploy memory plan, deploy kernel façade checks and the launcher's role plan (pure host logic)."""

import pytest

from pear_b200.deploy.server import MemoryPlan
from pear_b200.launch.roles import command, gpu_process_env, plan_node
from pear_b200.models.config import HybridConfig
from pear_b200.models.qwen3_5.deploy_kernels import Qwen3_5DeployKernels
from pear_b200.models.qwen3_5.gpu_backend import REQUIREMENTS
from pear_b200.models.qwen3_5.rollout_kernels import Qwen3_5RolloutKernels


def test_memory_plan_moves_the_embedding_out_only_when_short():
    cfg, draft = HybridConfig.qwen3_8_27b(), HybridConfig.drafter()
    p = MemoryPlan.build(cfg, 260096, draft=draft)
    assert not p.embedding_on_host and p.total_device_bytes < 0.9 * (180 << 30)
    assert 13e9 < p.weight_bytes < 17e9  # ~27B parameters at 4.5 bits
    tight = MemoryPlan.build(cfg, 260096, hbm_bytes=int(p.total_device_bytes / 0.9) - (1 << 30), draft=draft)
    assert tight.embedding_on_host and tight.total_device_bytes == p.total_device_bytes - p.embedding_bytes
    with pytest.raises(MemoryError, match="lower max_model_len"):
        MemoryPlan.build(cfg, 260096, hbm_bytes=20 << 30, draft=draft)


def test_deploy_and_rollout_kernel_facades_check_their_configs():
    ecfg = {}
    Qwen3_5DeployKernels.configure_server(ecfg, 1, 8192)
    assert ecfg["max_num_seqs"] == 1
    with pytest.raises(ValueError, match="one session"):
        Qwen3_5DeployKernels.configure_server({}, 4, 8192)
    rcfg = {"tensor_parallel_size": 2}
    Qwen3_5RolloutKernels.configure_server(rcfg, 64, 8192)
    assert rcfg["block_size"] == 16 and rcfg["fast_decode"] is True and rcfg["max_num_seqs"] == 64
    with pytest.raises(ValueError, match="power of two"):
        REQUIREMENTS.check_rollout({"tensor_parallel_size": 3})
    with pytest.raises(ValueError, match="16-token blocks"):
        REQUIREMENTS.check_rollout({"tensor_parallel_size": 2, "block_size": 32})


def test_node_plan_and_commands():
    plans = plan_node(8, 4, 2, "training", ["run_dir=/tmp/r"])
    by = {p.role: p for p in plans}
    assert by["trainer"].processes == 4 and by["rollout"].processes == 2 and by["rollout"].gpu_ids(1) == [6, 7]
    cmd, env = command(by["trainer"], 0, master_port=1234)
    assert "--nproc-per-node=4" in cmd and "127.0.0.1" in cmd and env["CUDA_VISIBLE_DEVICES"] == "0,1,2,3"
    # a replica of two GPUs is a world of two ranks under torch.distributed.run; its ranks are consecutive in the weight-sync
    # world (rank 0 = the sending trainer rank), whose size and rendezvous the trainer gets as config keys
    cmd, env = command(by["rollout"], 1)
    assert cmd[:3] == ["python", "-m", "torch.distributed.run"] and "--nproc-per-node=2" in cmd and env["CUDA_VISIBLE_DEVICES"] == "6,7"
    assert cmd[cmd.index("-m", 3) + 1] == "pear_b200.rollout.server" and cmd[cmd.index("--sync-rank") + 1] == "3" and cmd[cmd.index("--sync-world") + 1] == "5"
    assert any(a.startswith("actor_rollout_ref.rollout.checkpoint_engine.replica_urls=[http://127.0.0.1:8100,http://127.0.0.1:8101]") for a in by["trainer"].args)
    single = {p.role: p for p in plan_node(8, 4, 1, "training", [])}["rollout"]
    cmd, env = command(single, 2)
    assert cmd[:3] == ["python", "-m", "pear_b200.rollout.server"] and env["CUDA_VISIBLE_DEVICES"] == "6" and cmd[cmd.index("--sync-rank") + 1] == "3"
    assert gpu_process_env([3])["NCCL_LAUNCH_ORDER_IMPLICIT"] == "1"
    with pytest.raises(ValueError):
        plan_node(8, 5, 2, "training", [])


@pytest.mark.timeout(600)
def test_roles_recipe_runs_as_processes(tmp_path):
    """The recipe that starts every role as a process (two trainer ranks, one replica of two lock-step ranks, environment
    host, monitor) trains one step on CPU; the launcher leaves no role behind when the trainer exits."""
    import json
    import os
    import subprocess

    from pear_b200.utils.process import free_ports

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = str(tmp_path / "run")
    env = dict(os.environ, PYTHONPATH=root, RUN=run, STEPS="1", OMP_NUM_THREADS="2",
               **dict(zip(("PORT", "ROLLOUT_PORT", "ENV_PORT", "SYNC_PORT", "REPLICA_PORT"), map(str, free_ports(5)))))
    proc = subprocess.run(["bash", os.path.join(root, "examples", "tiny_roles_cpu.sh")], cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          text=True, timeout=500, start_new_session=True)
    assert proc.returncode == 0, proc.stdout[-4000:]
    with open(os.path.join(run, "metrics.jsonl")) as f:
        rows = [json.loads(line) for line in f]
    assert len(rows) == 1 and rows[0]["weight_sync/bytes"] > 0 and rows[0]["actor/grad_norm"] > 0
    left = subprocess.run(["ps", "-eo", "pid,args"], stdout=subprocess.PIPE, text=True).stdout
    assert not [line for line in left.splitlines() if run in line], "a role outlived the launcher"


def test_rollout_kernel_hooks_check_and_complete_a_replicas_settings(monkeypatch):
    """``rollout.kernels`` names a family's hooks: they refuse settings the kernels are not built for, complete the rest, and
    refuse a model of another architecture; the class also reaches child processes through the environment."""
    import torch.nn as nn

    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.models.kernels import RolloutKernels
    from pear_b200.rollout.engine import EngineConfig
    from pear_b200.rollout.server import apply_rollout_kernels

    path = "pear_b200.models.qwen3_5.rollout_kernels.Qwen3_5RolloutKernels"
    model = HybridForCausalLM(HybridConfig.tiny(), with_mtp=False)
    cfg = apply_rollout_kernels(path, EngineConfig(max_num_seqs=8, fast_decode=False), model=model, tensor_parallel_size=2)
    assert cfg.max_num_seqs == 8 and cfg.block_size == 16 and cfg.fast_decode is False  # an explicit choice is kept
    with pytest.raises(ValueError, match="16-token blocks"):
        apply_rollout_kernels(path, EngineConfig(block_size=32))
    with pytest.raises(ValueError, match="power of two"):
        apply_rollout_kernels(path, EngineConfig(), tensor_parallel_size=3)
    with pytest.raises(TypeError, match="hybrid GDN"):
        apply_rollout_kernels(path, EngineConfig(), model=nn.Linear(2, 2))
    plain = EngineConfig(block_size=32)
    assert apply_rollout_kernels(None, plain) is plain  # no hooks named: nothing checked
    monkeypatch.setenv(RolloutKernels.ENV, path)
    with pytest.raises(ValueError, match="16-token blocks"):
        apply_rollout_kernels(None, plain)


def test_cluster_plan_gives_every_node_its_roles():
    from pear_b200.launch.roles import plan_cluster

    addrs = ["10.0.0.1", "10.0.0.2", "10.0.0.3", "10.0.0.4"]
    head = {p.role: p for p in plan_cluster(addrs, 0, 8, 2, 4, "training", ["run_dir=/r"])}
    assert set(head) == {"trainer", "env", "monitor"} and head["trainer"].nnodes == 2 and head["trainer"].master_addr == "10.0.0.1"
    cmd, env = command(head["trainer"], 0, master_port=1234)
    assert "--nnodes=2" in cmd and "--node-rank=0" in cmd and "--nproc-per-node=8" in cmd and env["CUDA_VISIBLE_DEVICES"] == "0,1,2,3,4,5,6,7"
    urls = next(a for a in head["trainer"].args if "replica_urls" in a)
    assert urls.endswith("[http://10.0.0.3:8100,http://10.0.0.3:8101,http://10.0.0.4:8100,http://10.0.0.4:8101]")
    assert "actor_rollout_ref.rollout.checkpoint_engine.sync_master=10.0.0.1:29650" in head["trainer"].args
    second = {p.role: p for p in plan_cluster(addrs, 1, 8, 2, 4, "training", ["run_dir=/r"])}
    assert set(second) == {"trainer"} and "--node-rank=1" in command(second["trainer"], 0)[0]
    last = {p.role: p for p in plan_cluster(addrs, 3, 8, 2, 4, "training", ["run_dir=/r"])}
    cmd, env = command(last["rollout"], 1)
    assert set(last) == {"rollout"} and env["CUDA_VISIBLE_DEVICES"] == "4,5,6,7"
    assert cmd[cmd.index("--name") + 1] == "replica-3" and cmd[cmd.index("--sync-rank") + 1] == "13" and cmd[cmd.index("--sync-world") + 1] == "17"
    assert cmd[cmd.index("--host") + 1] == "10.0.0.4" and "--exit-with-trainer" in cmd
    with pytest.raises(ValueError):
        plan_cluster(addrs, 0, 8, 4, 4, "training", [])  # no node left for rollouts


@pytest.mark.timeout(600)
def test_two_nodes_on_loopback_addresses(tmp_path):
    """The same command line on two "nodes" (127.0.0.1 trains with two ranks, 127.0.0.2 serves one replica of two lock-step
    ranks): the trainer reaches the replica by the other node's address, trains a step, and the rollout node's launcher ends by
    itself once the trainer's weight-sync world is gone."""
    import json
    import os
    import subprocess
    import sys

    from pear_b200.utils.process import free_ports

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = str(tmp_path / "run")
    master, replica_master, rollout, envp, sync = free_ports(5)
    common = [sys.executable, "-m", "pear_b200.launch.launch", "training", "--node-addrs", "127.0.0.1,127.0.0.2", "--trainer-nodes", "1", "--gpus", "2",
              "--rollout-tp", "2", "--master-port", str(master), "--replica-master-port", str(replica_master), "--rollout-port", str(rollout),
              "--env-port", str(envp), "--sync-port", str(sync), f"run_dir={run}", "actor_rollout_ref.model.path=preset:tiny",
              "trainer.total_training_steps=1", "trainer.save_freq=0", "data.train_batch_size=3", "actor_rollout_ref.rollout.n=4", "data.max_response_length=32",
              "actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size=2", "actor_rollout_ref.rollout.multi_turn.synthetic_turns=1",
              "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash", "actor_rollout_ref.rollout.max_model_len=2048",
              "actor_rollout_ref.rollout.max_num_seqs=8", "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=8192", "trainer.logger=[file]"]
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    node1 = subprocess.Popen(common + ["--node-rank", "1"], cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
    try:
        node0 = subprocess.run(common + ["--node-rank", "0"], cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=400,
                               start_new_session=True)
        assert node0.returncode == 0, node0.stdout[-4000:]
        out1, _ = node1.communicate(timeout=90)  # ends by itself: its replicas saw the trainer's world go away
    finally:
        if node1.poll() is None:
            import signal

            os.killpg(node1.pid, signal.SIGTERM)
            node1.communicate(timeout=30)
    with open(os.path.join(run, "metrics.jsonl")) as f:
        rows = [json.loads(line) for line in f]
    assert len(rows) == 1 and rows[0]["weight_sync/bytes"] > 0 and rows[0]["actor/grad_norm"] > 0
    assert "replica-0 rank 0:" in out1 and "replica-0 rank 1:" in out1 and "policy_version=1" in out1, out1[-3000:]

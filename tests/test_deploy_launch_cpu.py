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
    cmd, env = command(by["rollout"], 0)
    assert cmd[:3] == ["python", "-m", "pear_b200.rollout.server"] and env["CUDA_VISIBLE_DEVICES"] == "4,5"
    assert gpu_process_env([3])["NCCL_LAUNCH_ORDER_IMPLICIT"] == "1"
    with pytest.raises(ValueError):
        plan_node(8, 5, 2, "training", [])

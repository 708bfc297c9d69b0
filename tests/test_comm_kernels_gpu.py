"""Fused compute+collective kernels over NVLink peer memory: needs at least two GPUs (skipped otherwise). The ranks run
as child processes, one per GPU, with NVLS off and every device-side wait bounded."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(600)
def test_fused_collective_kernels_two_ranks():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(root, "tests", "multi_gpu", "run_comm.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    for name in ("all_reduce_add_rmsnorm", "ag_gemm", "gemm_rs", "pull_quantize_nvfp4", "weight_sync_symm", "weight_sync_server", "all_gather_logits", "sharded_argmax", "gemm_a2a", "a2a_gemm", "reduce_scatter_adamw", "tp_rollout_fused"):
        assert f"PASS {name}" in out, out[-4000:]


@pytest.mark.timeout(600)
def test_tensor_parallel_fast_step_two_ranks():
    """The batched GPU-resident rollout step sharded over two GPUs against the same step on one."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(root, "tests", "multi_gpu", "run_fast_step.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert "PASS tp_fast_step world 2 reduction one" in out and "PASS tp_fast_step world 2 reduction two" in out and "PASS tp_fast_step_graph" in out, out[-4000:]


@pytest.mark.timeout(600)
def test_trainer_overlap_two_ranks():
    """Prefetched all-gathers and overlapped reduce-scatters of the trainer's sharded units against the same step with every
    collective on the compute stream, with only rank 0 holding the model at construction."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29547", os.path.join(root, "tests", "multi_gpu", "run_train_engine.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert "PASS fsdp_overlap" in out, out[-4000:]


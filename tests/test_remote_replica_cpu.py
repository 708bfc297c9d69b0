"""A rollout replica as a process of its own: requests over HTTP (token ids, top log-probs, vision placeholder rows), weights
through a process group it shares with the trainer side (gloo here; NCCL or the NVSwitch transport on GPUs)."""

import os
import subprocess
import sys
import time

import pytest
import torch

from pear_b200.loop.weight_sync import BroadcastTransport, StandaloneGroup, SyncConfig, WeightSync
from pear_b200.rollout.engine import FinishReason, SamplingParams
from pear_b200.rollout.remote import RemoteReplica, decode_embeds, encode_embeds
from pear_b200.rollout.server import load_rollout_model


from pear_b200.utils.process import free_ports


def _greedy(model, prompt, n):
    toks = list(prompt)
    with torch.no_grad():
        for _ in range(n):
            ids = torch.tensor(toks)
            h = model(ids, torch.arange(len(toks)), [0, len(toks)])
            toks.append(int(model.logits(model.model.norm(h[-1:])).argmax()))
    return toks[len(prompt):]


def test_embeds_travel_as_bf16_rows():
    e = torch.randn(7, 16)
    m = torch.tensor([0, 1, 1, 0, 0, 1, 0], dtype=torch.bool)
    e2, m2 = decode_embeds(encode_embeds(e, m))
    assert torch.equal(m2, m) and torch.equal(e2[m], e[m].to(torch.bfloat16).float()) and not e2[~m].any()
    assert decode_embeds({}) == (None, None)


@pytest.mark.timeout(300)
def test_replica_process_serves_requests_and_receives_weights():
    http_port, sync_port = free_ports(2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.Popen([sys.executable, "-m", "pear_b200.rollout.server", "--model", "preset:tiny", "--port", str(http_port), "--num-blocks", "128",
                             "--max-num-seqs", "4", "--sync-rank", "1", "--sync-world", "2", "--sync-master", f"127.0.0.1:{sync_port}",
                             "--sync-backend", "gloo"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        group = StandaloneGroup(f"127.0.0.1:{sync_port}", 0, 2, "gloo")  # the trainer side of the weight-sync world
        replica = RemoteReplica(f"http://127.0.0.1:{http_port}", name="replica-0")
        replica.wait_ready(120, alive=lambda: proc.poll() is None)
        model = load_rollout_model("preset:tiny", device="cpu")  # the same seeded weights the replica process built
        prompt = list(range(3, 40))
        p = SamplingParams(max_tokens=6, temperature=0.0, topk_logprobs=3)
        r1 = replica.generate(prompt, p, session="s0")
        assert r1.finish == FinishReason.LENGTH and r1.output == _greedy(model, prompt, 6)
        assert len(r1.logprobs) == 6 and len(r1.topk_ids) == 6 and all(len(x) == 3 for x in r1.topk_ids) and r1.policy_version == 0
        # every sampling parameter travels: top-k 1 at temperature 1 is the greedy sequence again
        r_k1 = replica.generate(prompt, SamplingParams(max_tokens=6, temperature=1.0, top_k=1), session="s-k1")
        assert r_k1.output == r1.output
        # a weight sync driven from this process: pause / resume over HTTP, buckets over the process group
        new_state = {k: ((v * 0.5).to(torch.bfloat16).float() if v.dim() >= 2 else v.clone()) for k, v in model.state_dict().items()}
        stats = WeightSync(SyncConfig(bucket_megabytes=1, rollout_dtype=torch.bfloat16), BroadcastTransport(group, 0, "cpu"), [replica]).sync(new_state, version=3)
        assert stats["weight_sync/buckets"] >= 1
        t0 = time.time()
        while replica.policy_version() != 3:  # the receiver thread loads after the last bucket
            assert time.time() - t0 < 60, "the replica never loaded the new weights"
            time.sleep(0.1)
        model.load_state_dict(new_state)
        r2 = replica.generate(prompt, p, session="s1")
        assert r2.policy_version == 3 and r2.output == _greedy(model, prompt, 6)
        assert any(line.split()[-1] in ("3", "3.0") for line in replica.metrics_text().splitlines() if "policy_version" in line and not line.startswith("#"))
    finally:
        proc.terminate()
        try:
            out, _ = proc.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
    assert "Traceback" not in (out or ""), out[-3000:]


@pytest.mark.timeout(600)
def test_training_entry_drives_a_replica_process(tmp_path):
    """``checkpoint_engine.replica_urls`` set: the trainer builds no replica of its own, reaches the replica process over HTTP,
    starts it from the trainer's policy and syncs after each step."""
    from pear_b200.config.loader import compose
    from pear_b200.train.main import RunConfig, build_stack

    http_port, sync_port = free_ports(2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.Popen([sys.executable, "-m", "pear_b200.rollout.server", "--model", "preset:tiny", "--port", str(http_port), "--num-blocks", "512",
                             "--max-num-seqs", "8", "--sync-rank", "1", "--sync-world", "2", "--sync-master", f"127.0.0.1:{sync_port}",
                             "--sync-backend", "gloo"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    overrides = [f"run_dir={tmp_path / 'run'}", "actor_rollout_ref.model.path=preset:tiny", "data.train_batch_size=2", "actor_rollout_ref.rollout.n=2",
                 "data.max_response_length=24", "actor_rollout_ref.rollout.max_model_len=2048", "actor_rollout_ref.rollout.max_num_seqs=8",
                 "actor_rollout_ref.rollout.agent.num_workers=4", "actor_rollout_ref.rollout.topk_log_probs=4", "algorithm.filter_groups.enable=false",
                 "trainer.total_training_steps=1", "trainer.save_freq=0", "transfer_queue.num_data_storage_units=4", "actor_rollout_ref.actor.optim.lr=1e-3",
                 "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=4096", "trainer.logger=[file]",
                 f"actor_rollout_ref.rollout.checkpoint_engine.replica_urls=[http://127.0.0.1:{http_port}]",
                 f"actor_rollout_ref.rollout.checkpoint_engine.sync_master=127.0.0.1:{sync_port}", "actor_rollout_ref.rollout.tensor_model_parallel_size=1"]
    close = None
    try:
        trainer, close = build_stack(RunConfig(compose("training", overrides)).prepare())
        replica = trainer.manager.router.servers[0]
        assert isinstance(replica, RemoteReplica) and replica._health()["weight_loads"] == 1  # started from the trainer's policy
        hist = trainer.fit()
        assert len(hist) == 1 and hist[0]["weight_sync/bytes"] > 0 and replica.policy_version() == 1
    finally:
        if close is not None:
            close()
        proc.terminate()
        try:
            out, _ = proc.communicate(timeout=20)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
    assert "Traceback" not in (out or ""), out[-3000:]


@pytest.mark.timeout(600)
def test_tensor_parallel_replica_runs_in_lock_step_behind_one_endpoint():
    """Two gloo ranks form one replica: rank 0 serves HTTP and broadcasts the control events, both ranks step together; each
    rank receives the weight sync itself and keeps its shard. Tokens equal the unsharded model's before and after a sync."""
    http_port, sync_port, tp_port = free_ports(3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    proc = subprocess.Popen([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                             "--master-port", str(tp_port), "-m", "pear_b200.rollout.server", "--model", "preset:tiny", "--port", str(http_port),
                             "--num-blocks", "128", "--max-num-seqs", "4", "--sync-rank", "1", "--sync-world", "3",
                             "--sync-master", f"127.0.0.1:{sync_port}", "--sync-backend", "gloo"],
                            env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        group = StandaloneGroup(f"127.0.0.1:{sync_port}", 0, 3, "gloo")
        replica = RemoteReplica(f"http://127.0.0.1:{http_port}")
        replica.wait_ready(180, alive=lambda: proc.poll() is None)
        model = load_rollout_model("preset:tiny", device="cpu")
        prompts = [list(range(3, 40)), list(range(50, 61))]
        p = SamplingParams(max_tokens=6, temperature=0.0)
        import concurrent.futures as cf
        with cf.ThreadPoolExecutor(2) as pool:  # two requests in flight: the leader batches them, the follower must too
            outs = list(pool.map(lambda pr: replica.generate(pr, p), prompts))
        assert [o.output for o in outs] == [_greedy(model, pr, 6) for pr in prompts]
        new_state = {k: ((v * 0.5).to(torch.bfloat16).float() if v.dim() >= 2 else v.clone()) for k, v in model.state_dict().items()}
        WeightSync(SyncConfig(bucket_megabytes=1, rollout_dtype=torch.bfloat16), BroadcastTransport(group, 0, "cpu"), [replica]).sync(new_state, version=5)
        model.load_state_dict(new_state)
        r2 = replica.generate(prompts[0], p)
        assert r2.policy_version == 5 and r2.output == _greedy(model, prompts[0], 6)
    finally:
        proc.terminate()
        try:
            out, _ = proc.communicate(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
            out, _ = proc.communicate()
    assert "Traceback" not in (out or "") or "SignalException" in out, out[-3000:]


def _replica(http_port, sync_port, world=2):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    return subprocess.Popen([sys.executable, "-m", "pear_b200.rollout.server", "--model", "preset:tiny", "--port", str(http_port), "--num-blocks", "128",
                             "--max-num-seqs", "4", "--sync-rank", "1", "--sync-world", str(world), "--sync-master", f"127.0.0.1:{sync_port}",
                             "--sync-backend", "gloo"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("how", ["killed", "terminated"])
def test_a_lost_replica_is_named_before_the_sync_starts(how):
    """The replica's ranks beat into the weight-sync world's store; the sender checks before a sync. A replica that was killed
    stops beating and is reported after the heartbeat timeout; one that was terminated says that it leaves. Neither is waited
    for inside a broadcast."""
    from pear_b200.parallel.heartbeat import PeerLost

    http_port, sync_port = free_ports(2)
    proc = _replica(http_port, sync_port)
    try:
        group = StandaloneGroup(f"127.0.0.1:{sync_port}", 0, 2, "gloo")
        replica = RemoteReplica(f"http://127.0.0.1:{http_port}")
        replica.wait_ready(120, alive=lambda: proc.poll() is None)
        sync = WeightSync(SyncConfig(bucket_megabytes=1, rollout_dtype=torch.bfloat16), BroadcastTransport(group, 0, "cpu"), [replica],
                          heartbeat=group.heartbeat(timeout_s=2.5))
        state = load_rollout_model("preset:tiny", device="cpu").state_dict()
        sync.sync(state, version=1)  # a live replica: the sync goes through
        assert replica.policy_version() == 1
        if how == "killed":
            proc.kill()
            proc.wait(30)
            time.sleep(3.0)
            with pytest.raises(PeerLost, match=r"ranks \[1\] lost: no heartbeat"):
                sync.sync(state, version=2)
        else:
            proc.terminate()
            proc.wait(60)
            with pytest.raises(PeerLost, match=r"ranks \[1\] lost: left the job"):
                sync.sync(state, version=2)
        with pytest.raises(Exception):  # requests to it fail at once as well
            replica.generate([1, 2, 3], SamplingParams(max_tokens=2))
    finally:
        if proc.poll() is None:
            proc.kill()
        proc.communicate()

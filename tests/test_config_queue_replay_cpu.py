"""Config composition, transfer queue, replay buffer, checkpoint retention, weight-sync bucketing: host-side units."""

import os

import pytest
import torch

from pear_b200.config.loader import compose
from pear_b200.loop.transfer_queue import TransferQueue
from pear_b200.loop.weight_sync import SyncConfig, buckets, cast_for_rollout
from pear_b200.train.replay_buffer import GroupStatus, PromptGroup, ReplayBuffer


def test_compose_overrides_interpolation_and_missing():
    cfg = compose("training", ["run_dir=/tmp/r", "actor_rollout_ref.model.path=preset:tiny", "data.train_batch_size=7"])
    assert cfg.data.train_batch_size == 7 and cfg.algorithm.filter_groups.enable is True  # training.yaml over base.yaml
    assert cfg.env_vars.PEAR_LOG_DIR == "/tmp/r/sim"  # ${run_dir} interpolation
    assert cfg.actor_rollout_ref.rollout.checkpoint_engine.engine_kwargs.rollout_dtype == "bfloat16"
    with pytest.raises(Exception):
        compose("training", ["actor_rollout_ref.model.path=preset:tiny"])  # run_dir is ??? (mandatory)
    d = compose("server", ["model=preset:tiny", "+qwen3_5=deploy"])
    assert d.kernels.endswith("Qwen3_5DeployKernels") and d.engine.max_num_seqs == 1


def test_transfer_queue_sealing_snapshot_and_torn_keys(tmp_path):
    q = TransferQueue(4)
    q.put_trajectory("g0/0", {"tokens": [1, 2, 3], "reward": 1.0}, family="synthetic")
    q.put("g0/1", tokens=[4, 5])  # never sealed: a write torn by a crash
    assert q.has("g0/0") and not q.has("g0/1") and q.get("g0/1") is None
    assert q.keys("g0/") == ["g0/0"] and q.keys("g0/", sealed_only=False) == ["g0/0", "g0/1"]
    q.snapshot(str(tmp_path / "tq"))
    assert sorted(f for f in os.listdir(tmp_path / "tq") if f.startswith("unit_")) == [f"unit_{i:03d}.pkl" for i in range(4)]
    q2 = TransferQueue(4)
    assert q2.restore(str(tmp_path / "tq")) == 1  # the half-written key is dropped
    assert q2.get("g0/0")["reward"] == 1.0 and q2.get("g0/0")["__meta__"]["family"] == "synthetic" and not q2.has("g0/1")
    with pytest.raises(ValueError, match="4 storage units cannot load into 8"):
        TransferQueue(8).restore(str(tmp_path / "tq"))


def _finish(q, g, rewards):
    for s, r in zip(g.session_ids, rewards):
        q.put_trajectory(f"{g.uid}/{s}", {"tokens": [1], "reward": r})


def test_replay_buffer_filter_staleness_and_caps():
    q = TransferQueue(2)
    rb = ReplayBuffer(q, n=2, max_off_policy_threshold=2, filter_groups=True, max_inflight_sessions=4)
    issued = []

    def refill(k, evicted):
        for _ in range(k):
            g = PromptGroup(uid=f"g{len(issued)}", prompt={}, n=2, issued_version=version[0], tool="t")
            rb.add_group(g)
            issued.append(g)
            # all-equal rewards for the first group (filtered), mixed afterwards
            _finish(q, g, [0.0, 0.0] if len(issued) == 1 else [1.0, 0.0])
        return k

    version = [0]
    out = rb.sample(0, 1, refill=refill, timeout_s=5)
    assert len(out) == 1 and out[0].uid != "g0" and rb.evicted_filtered == 1  # DAPO: the all-zero group was replaced
    assert rb.inflight_sessions() <= 4
    rb.release(out)
    assert not q.has(f"{out[0].uid}/0")
    # a group issued at version 0 is too stale at version 2 (threshold 2: versions 0 and 1 may train on it)
    old = PromptGroup(uid="old", prompt={}, n=2, issued_version=0)
    rb.add_group(old)
    _finish(q, old, [1.0, 0.0])
    version[0] = 2
    got = rb.sample(2, 1, refill=refill, timeout_s=5)
    assert got[0].uid != "old" and rb.dropped_stale >= 1
    assert "train/filter_groups/avg@n" in rb.metrics and "train/filter_groups/passrate/zero" in rb.metrics


def test_replay_buffer_restore_keeps_sealed_sessions():
    q = TransferQueue(2)
    rb = ReplayBuffer(q, n=2, max_off_policy_threshold=5)
    g = PromptGroup(uid="ga", prompt={"family": "synthetic", "env_args": {}}, n=2, issued_version=3)
    stale = PromptGroup(uid="gb", prompt={"family": "synthetic", "env_args": {}}, n=2, issued_version=0)
    rb.add_group(g)
    rb.add_group(stale)
    q.put_trajectory("ga/0", {"tokens": [1], "reward": 1.0})   # one session finished before the crash
    q.put_trajectory("gb/0", {"tokens": [1], "reward": 1.0})
    q.put_trajectory("zz/0", {"tokens": [1], "reward": 0.0})   # an orphan whose group is gone
    state = rb.state()
    rb2 = ReplayBuffer(q, n=2, max_off_policy_threshold=5)
    rep = rb2.restore(state, step_version=6)
    assert rep == {"kept_sessions": 1, "rerun_sessions": 1, "restarted_groups": 1, "cleared_orphans": 1}
    assert rb2.groups["ga"].status == GroupStatus.QUEUED and rb2.groups["ga"].unfinished == ["1"]
    assert rb2.groups["gb"].unfinished is None and rb2.groups["gb"].issued_version == 6 and not q.has("gb/0") and not q.has("zz/0")
    assert [x.uid for x in rb2.queued()] == ["ga", "gb"]


def test_weight_sync_buckets_and_cast():
    cfg = SyncConfig(bucket_megabytes=1, rollout_dtype=torch.bfloat16, fp32_modules=("lm_head",))
    state = {"a.weight": torch.zeros(300, 512), "lm_head.weight": torch.zeros(300, 512), "b.weight": torch.zeros(300, 512), "idx": torch.zeros(4, dtype=torch.int64)}
    assert cast_for_rollout("a.weight", state["a.weight"], cfg).dtype == torch.bfloat16
    assert cast_for_rollout("lm_head.weight", state["lm_head.weight"], cfg).dtype == torch.float32
    bl = list(buckets(state.items(), cfg))
    assert sum(len(b) for b in bl) == 4 and len(bl) >= 2
    assert all(sum(t.numel() * t.element_size() for _, t in b) <= (1 << 20) or len(b) == 1 for b in bl)


def test_checkpoint_retention_prunes_before_writing(tmp_path):
    from pear_b200.train.checkpoint import CheckpointManager

    class FakeEngine:
        def train_state(self):
            return {"shards": {}, "optimizer": {}, "step": 0, "policy_version": 0, "world_size": 1}

    cm = CheckpointManager(str(tmp_path), max_ckpt_to_keep=2)
    for step in (1, 2, 3, 4):
        cm.save(step, FakeEngine())
        assert len(cm.steps_on_disk()) <= 2
    assert cm.steps_on_disk() == [3, 4] and cm.latest() == 4


def test_metrics_log_commits_one_wandb_row_per_step(tmp_path, monkeypatch):
    import json
    import sys
    import types

    from pear_b200.train.main import MetricsLog

    calls = {"init": [], "log": []}
    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: calls["init"].append(kw)
    fake.log = lambda data, step=None, commit=None: calls["log"].append((dict(data), step, commit))
    monkeypatch.setitem(sys.modules, "wandb", fake)
    log = MetricsLog(str(tmp_path), ("file", "wandb"))
    log(1, {"actor/pg_loss": 0.5, "note": "text"})
    log(2, {"actor/pg_loss": 0.25})
    assert calls["init"][0]["dir"] == str(tmp_path) and len(calls["log"]) == 2
    assert calls["log"][0][1:] == (1, True) and calls["log"][0][0]["actor/pg_loss"] == 0.5 and "note" not in calls["log"][0][0]
    with open(tmp_path / "metrics.jsonl") as f:
        assert [json.loads(line)["step"] for line in f] == [1, 2]


def test_unimplemented_settings_are_refused_at_start(tmp_path):
    from pear_b200.config.loader import ConfigError
    from pear_b200.train.main import RunConfig

    base = [f"run_dir={tmp_path}", "actor_rollout_ref.model.path=preset:tiny"]
    RunConfig(compose("training", base)).prepare()  # the shipped recipe is all implemented values
    with pytest.raises(ConfigError, match=r"adv_estimator='gae'.*\n.*use_kl_loss=True|use_kl_loss=True"):
        RunConfig(compose("training", base + ["algorithm.adv_estimator=gae", "actor_rollout_ref.actor.use_kl_loss=true"])).prepare()


def test_metrics_log_writes_tensorboard_events(tmp_path, monkeypatch):
    import glob

    monkeypatch.delenv("TENSORBOARD_DIR", raising=False)  # (a recipe's env_vars may have set it in this process: it would win)

    from pear_b200.train.main import MetricsLog

    log = MetricsLog(str(tmp_path), ("tensorboard",))
    log(1, {"actor/pg_loss": 0.5})
    log(2, {"actor/pg_loss": 0.25, "note": "text"})
    files = glob.glob(str(tmp_path / "tensorboard" / "events.out.tfevents.*"))
    assert files and sum(os.path.getsize(f) for f in files) > 0


def test_pass_rate_metrics_of_judged_groups():
    """Groups with pass rates 1, 0 and three times 0.5: avg@n one half, a fifth of the groups unsolved, a fifth solved."""
    import torch

    from pear_b200.train import grpo

    m = grpo.pass_rate_metrics(torch.tensor([[1.0, 1.0], [0.0, 0.0], [0.0, 1.0], [0.0, 1.0], [0.0, 1.0]]), "validation/filter_groups")
    assert m["validation/filter_groups/avg@n"] == pytest.approx(0.5)
    assert m["validation/filter_groups/passrate/zero"] == pytest.approx(1 / 5) and m["validation/filter_groups/passrate/one"] == pytest.approx(1 / 5)

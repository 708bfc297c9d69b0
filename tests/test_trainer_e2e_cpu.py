"""The whole training loop on CPU with the tiny model and the synthetic environment: rollout through the agent loop,
replay buffer, GRPO step, weight sync into the rollout replica, checkpoint, resume with in-flight groups."""

import os

import numpy as np
import pytest
import torch

from pear_b200.config.loader import compose
from pear_b200.models import io as model_io
from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM
from pear_b200.train.main import RunConfig, build_stack
from pear_b200.train.trainer import balanced_partition, micro_batches, pack_rows, trajectory_to_rows

OVERRIDES = [
    "actor_rollout_ref.model.path=preset:tiny", "actor_rollout_ref.model.enable_gradient_checkpointing=true",
    "data.train_batch_size=2", "actor_rollout_ref.rollout.n=2", "data.max_response_length=24",
    "actor_rollout_ref.rollout.max_model_len=2048", "actor_rollout_ref.rollout.max_num_seqs=8",
    "actor_rollout_ref.rollout.agent.num_workers=4", "actor_rollout_ref.rollout.topk_log_probs=4",
    "algorithm.filter_groups.enable=false", "trainer.total_training_steps=2", "trainer.save_freq=1",
    "trainer.max_actor_ckpt_to_keep=1", "transfer_queue.num_data_storage_units=4", "actor_rollout_ref.actor.optim.lr=1e-3",
    "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=4096", "trainer.logger=[file]",
]


def _cfg(run_dir, extra=()):
    return RunConfig(compose("training", [f"run_dir={run_dir}"] + OVERRIDES + list(extra))).prepare()


def test_rows_packing_and_partition():
    tr = {"tokens": np.arange(10), "response_mask": np.array([0] * 6 + [1] * 4, dtype=np.int8), "rollout_logprobs": -np.arange(10, dtype=np.float32),
          "topk_ids": np.zeros((10, 4), dtype=np.int64), "topk_logprobs": np.zeros((10, 4), dtype=np.float32),
          "embeds": [(2, np.ones((2, 8), dtype=np.float16))], "reward": 1.0}
    r = trajectory_to_rows(tr, 0.5, 8, 4)
    # the label of position t is token t+1; position 5 predicts the first sampled token
    assert r["labels"][:9].tolist() == list(range(1, 10)) and r["loss_mask"].tolist() == [0] * 5 + [1] * 4 + [0]
    assert r["sampler_log_probs"][5].item() == -6.0 and r["advantages"][5].item() == 0.5 and r["advantages"][0].item() == 0.0
    assert r["embeds_mask"].nonzero().flatten().tolist() == [2, 3]
    b = pack_rows([r, r])
    assert b.cu_seqlens == [0, 10, 20] and b.num_tokens == 20 and b.head_ids.shape == (20, 4)
    parts = balanced_partition([10, 3, 8, 5, 4], 2)
    assert sorted(sum(parts, [])) == [0, 1, 2, 3, 4] and abs(sum([10, 3, 8, 5, 4][i] for i in parts[0]) - 15) <= 1
    assert [len(mb) for mb in micro_batches([r] * 5, 25)] == [2, 2, 1]


@pytest.mark.timeout(900)
def test_two_steps_checkpoint_and_resume(tmp_path):
    run = str(tmp_path / "run")
    trainer, close = build_stack(_cfg(run))
    try:
        w0 = {k: v.clone() for k, v in trainer.engine.full_state_dict().items()}
        hist = trainer.fit()
        assert len(hist) == 2 and trainer.engine.policy_version == 2
        assert all(np.isfinite(h["actor/grad_norm"]) for h in hist) and "weight_sync/bytes" in hist[0]
        assert all(h["ctx_total_length/max"] >= h["ctx_total_length/mean"] > 0 and h["perf/mfu"] > 0 and h["perf/tokens_per_s"] > 0 for h in hist)
        # the rollout replica serves the trained policy
        srv = trainer.manager.router.servers[0]
        assert srv.engine.policy_version == 2
        w_train = trainer.engine.full_state_dict()
        w_roll = dict(srv.engine.model.named_parameters())
        name = "lm_head.weight"
        assert torch.allclose(w_roll[name].float(), w_train[name].to(torch.bfloat16).float())
        assert os.path.exists(os.path.join(run, "metrics.jsonl"))
        assert sorted(d for d in os.listdir(os.path.join(run, "ckpt")) if d.startswith("global_step")) == ["global_step_2"]
    finally:
        close()
    # resume: same command on the same run directory continues at step 2 with the trained weights
    trainer2, close2 = build_stack(_cfg(run, ["trainer.total_training_steps=3"]))
    try:
        rep = trainer2.resume()
        assert rep["step"] == 2 and trainer2.engine.policy_version == 2
        w2 = trainer2.engine.full_state_dict()
        assert all(torch.equal(w2[k], w_train[k]) for k in w_train)
        hist2 = trainer2.fit()
        assert len(hist2) == 1 and trainer2.step == 3
        # export as a model directory and read it back
        out = str(tmp_path / "export")
        from pear_b200.train.checkpoint import export_model
        export_model(trainer2.engine, out)
        m = HybridForCausalLM(model_io.load_config(out), with_mtp=False)
        missing, unexpected = model_io.load_model_dir(out, m)
        assert not unexpected and all(k.startswith("mtp.") for k in missing)
        # the offline merger rebuilds the same tensors from the shard files of the run directory
        from pear_b200.utils import model_merger
        merged_dir = str(tmp_path / "merged")
        trainer2.checkpoints.save(3, trainer2.engine, trainer2.dataset, trainer2.replay, trainer2.queue)
        assert model_merger.main([run, merged_dir]) == 0
        a, b = model_io.load_safetensors(os.path.join(out, "model.safetensors")), model_io.load_safetensors(os.path.join(merged_dir, "model.safetensors"))
        assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    finally:
        close2()


def test_checkpoint_of_another_world_size_is_refused(tmp_path):
    from pear_b200.train.checkpoint import CheckpointManager
    run = str(tmp_path / "run")
    trainer, close = build_stack(_cfg(run, ["trainer.total_training_steps=0"]))
    try:
        trainer.checkpoints.save(1, trainer.engine, trainer.dataset, trainer.replay, trainer.queue)
        other = CheckpointManager(run, rank=0, world_size=4)
        with pytest.raises(ValueError, match=r"world size \[1\].*world size 4"):
            other.load(trainer.engine)
    finally:
        close()


@pytest.mark.timeout(600)
def test_training_step_on_pixel_observations(tmp_path):
    """Cameras that deliver pixels: the training entry builds the vision encoder, the rollouts carry its rows and a GRPO step
    trains on them."""
    fam = {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "num_processes": 2, "env_kwargs": {"pixels": 16}}}
    cfg = _cfg(str(tmp_path / "run"), ["actor_rollout_ref.model.vision.enable=true", "trainer.total_training_steps=1", "trainer.save_freq=0",
                                        "actor_rollout_ref.rollout.multi_turn.synthetic_turns=1", "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash"])
    trainer, close = build_stack(cfg, env_families=fam)
    try:
        hist = trainer.fit()
        enc = trainer.manager.loop.vision
        assert len(hist) == 1 and np.isfinite(hist[0]["actor/grad_norm"]) and enc is not None and enc.encoded >= 1 and enc.hits >= 1
    finally:
        close()


@pytest.mark.timeout(600)
def test_batch_trained_in_mini_batches(tmp_path):
    """``ppo_mini_batch_size`` below the batch: one optimizer step per mini-batch of prompt groups, one policy version (and one
    weight sync) per batch."""
    cfg = _cfg(str(tmp_path / "run"), ["data.train_batch_size=4", "actor_rollout_ref.actor.ppo_mini_batch_size=2", "trainer.total_training_steps=1",
                                        "trainer.save_freq=0", "actor_rollout_ref.rollout.multi_turn.synthetic_turns=1",
                                        "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash"])
    trainer, close = build_stack(cfg)
    try:
        hist = trainer.fit()
        assert hist[0]["actor/updates"] == 2.0 and trainer.engine.step_count == 2 and trainer.engine.policy_version == 1
        assert hist[0]["data/sessions"] == 8.0 and hist[0]["train/policy_version"] == 1.0 and hist[0]["weight_sync/buckets"] >= 1
        assert trainer.manager.router.servers[0].engine.policy_version == 1
    finally:
        close()


@pytest.mark.timeout(600)
def test_vision_tower_trains_under_the_policy_loss_and_the_agent_loop_follows_it(tmp_path):
    fam = {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "num_processes": 2, "env_kwargs": {"pixels": 16}}}
    cfg = _cfg(str(tmp_path / "run"), ["actor_rollout_ref.model.vision.enable=true", "actor_rollout_ref.model.vision.train=true",
                                        "data.train_batch_size=3", "actor_rollout_ref.rollout.n=4",  # (a step of uniform-reward groups only would have no gradient)
                                        "trainer.total_training_steps=1", "trainer.save_freq=1", "actor_rollout_ref.rollout.multi_turn.synthetic_turns=1",
                                        "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash"])
    trainer, close = build_stack(cfg, env_families=fam)
    try:
        before = {k: v.clone() for k, v in trainer.engine.full_state_dict().items() if k.startswith("visual.")}
        enc = trainer.manager.loop.vision
        assert before and all(torch.equal(enc.tower.state_dict()[k[len("visual."):]], v) for k, v in before.items())  # starts from the trainer's tower
        hist = trainer.fit()
        after = {k: v for k, v in trainer.engine.full_state_dict().items() if k.startswith("visual.")}
        moved = [k for k in before if not torch.equal(before[k], after[k])]
        assert len(hist) == 1 and np.isfinite(hist[0]["actor/grad_norm"]) and len(moved) >= len(before) // 2, moved
        assert all(torch.allclose(enc.tower.state_dict()[k[len("visual."):]], v) for k, v in after.items()) and not enc.cache  # followed, old encodings dropped
        # the tower is part of the checkpoint and of the exported model directory
        from pear_b200.train.checkpoint import export_model

        export_model(trainer.engine, str(tmp_path / "export"))
        names = [model_io.from_hf_name(n) for n in model_io.model_tensor_names(str(tmp_path / "export"))]
        assert any(n.startswith("visual.") for n in names)
    finally:
        close()


@pytest.mark.timeout(600)
def test_checkpoint_picture_positions_in_rollout_and_training(tmp_path):
    """``rollout.picture_positions=checkpoint``: the agent loop sends (temporal, row, column) positions with every request, the
    engine runs such requests on its per-request path, trajectories carry the positions and the trainer trains on them."""
    fam = {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "num_processes": 2, "env_kwargs": {"pixels": 16, "cameras": ("front", "wrist")}}}
    cfg = _cfg(str(tmp_path / "run"), ["actor_rollout_ref.model.vision.enable=true", "actor_rollout_ref.model.vision.preset=family_tiny",
                                        "actor_rollout_ref.model.vision.train=true", "actor_rollout_ref.rollout.picture_positions=checkpoint",
                                        "data.train_batch_size=3", "actor_rollout_ref.rollout.n=4",  # (a step of uniform-reward groups only would have no gradient)
                                        "trainer.total_training_steps=1", "trainer.save_freq=0", "actor_rollout_ref.rollout.multi_turn.synthetic_turns=2",
                                        "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash"])
    trainer, close = build_stack(cfg, env_families=fam)
    seen = []
    try:
        q = trainer.queue
        put = q.put_trajectory

        def spy(key, tr, **kw):
            seen.append(tr)
            return put(key, tr, **kw)

        q.put_trajectory = spy
        hist = trainer.fit()
        assert len(hist) == 1 and np.isfinite(hist[0]["actor/grad_norm"]) and hist[0]["actor/grad_norm"] > 0
        tr = seen[0]
        pos = tr["position_ids"]
        tr = max(seen, key=lambda t: len(t["images"]))
        pos = tr["position_ids"]
        assert pos.shape == (3, len(tr["tokens"])) and len(tr["images"]) >= 4 and len(tr["images"]) % 2 == 0  # two cameras a turn
        first = tr["images"][0][0]
        n_tok = 4  # 16 x 16 pixels, patch 4, merge 2: a 2 x 2 block
        assert pos[0, first:first + n_tok].tolist() == [pos[0, first]] * n_tok and pos[1, first:first + n_tok].tolist() == [pos[1, first] + d for d in (0, 0, 1, 1)]
        assert pos[2, first:first + n_tok].tolist() == [pos[2, first] + d for d in (0, 1, 0, 1)]
        assert int(pos.max()) < len(tr["tokens"]) - 1  # pictures used fewer positions than tokens
    finally:
        close()

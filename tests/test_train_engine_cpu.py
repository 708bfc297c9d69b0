"""Trainer engine on CPU: the sharded / checkpointed / sequence-parallel step equals the plain single-process step."""

import os

import pytest
import torch

from dist_utils import run_ranks
from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM
from pear_b200.ops import reference as ref
from pear_b200.train import grpo
from pear_b200.train.engine import EngineConfig, PackedBatch, TrainEngine


def make_batch(cfg: HybridConfig, seed: int = 0, lens=(70, 58), k: int = 4) -> PackedBatch:
    g = torch.Generator().manual_seed(seed)
    ids, pos, labels, mask, adv, cu = [], [], [], [], [], [0]
    for i, n in enumerate(lens):
        x = torch.randint(0, cfg.vocab_size, (n,), generator=g)
        ids.append(x)
        pos.append(torch.arange(n))
        labels.append(torch.cat([x[1:], x[:1]]))
        m = torch.zeros(n)
        m[n // 2 : n - 1] = 1
        mask.append(m)
        adv.append(torch.full((n,), float(torch.randn((), generator=g))))
        cu.append(cu[-1] + n)
    t = cu[-1]
    head_ids = torch.randint(0, cfg.vocab_size, (t, k), generator=g, dtype=torch.int32)
    head_lp = torch.log_softmax(torch.randn(t, k + 3, generator=g), -1)[:, :k]
    return PackedBatch(torch.cat(ids), torch.cat(pos), cu, torch.cat(labels), torch.cat(mask), torch.cat(adv),
                       sampler_log_probs=torch.randn(t, generator=g) * 0.1 - 3, head_ids=head_ids, head_log_probs=head_lp)


def reference_step(cfg: HybridConfig, ecfg: EngineConfig, batches: list[PackedBatch], seed: int):
    model = HybridForCausalLM(cfg, with_mtp=False).init_weights(seed)
    opt = torch.optim.AdamW(model.parameters(), lr=ecfg.lr, betas=ecfg.betas, eps=ecfg.eps, weight_decay=ecfg.weight_decay,
                            foreach=False, fused=False)
    denom = torch.tensor(float(sum(int(b.loss_mask.sum()) for b in batches)))
    for b in batches:
        h = model(b.input_ids, b.position_ids, b.cu_seqlens)
        ids = torch.cat([b.labels[:, None].long(), b.head_ids.long()], 1)
        lp, ent = ref.logprob_entropy_dense(h, model.lm_head.weight, ids, ecfg.temperature)
        loss, _ = grpo.policy_loss(lp[:, 0], b.advantages, b.loss_mask, ecfg.loss, lp[:, 1:], b.head_log_probs, b.sampler_log_probs,
                                   ent, denom)
        loss.backward()
    norm = torch.sqrt(sum(p.grad.pow(2).sum() for p in model.parameters() if p.grad is not None))
    scale = min(1.0, ecfg.clip_grad / (float(norm) + 1e-6))
    for p in model.parameters():
        if p.grad is not None:
            p.grad.mul_(scale)
    opt.step()
    return {k: v.detach().clone() for k, v in model.state_dict().items()}, float(norm)


def _ecfg(sp: int = 1) -> EngineConfig:
    return EngineConfig(lr=1e-3, eps=1e-3, clip_grad=1.0, param_dtype="fp32", ulysses_sequence_parallel_size=sp,
                        enable_gradient_checkpointing=True, temperature=0.9, topk_log_probs=4)


def test_single_process_engine_matches_plain_autograd():
    cfg = HybridConfig.tiny()
    ecfg = _ecfg()
    batches = [make_batch(cfg, 0), make_batch(cfg, 1, lens=(40, 33, 21))]
    want, want_norm = reference_step(cfg, ecfg, batches, seed=5)
    eng = TrainEngine(cfg, ecfg, seed=5)
    eng.forward_backward_batch(batches)
    m = eng.optimizer_step()
    got = eng.full_state_dict()
    assert abs(m["actor/grad_norm"] - want_norm) < 1e-4 * max(1.0, want_norm)
    for k, v in want.items():
        assert torch.allclose(got[k], v, atol=2e-5, rtol=1e-4), k


def _rank_fn(rank, world, out_dir, sp):
    cfg = HybridConfig.tiny()
    ecfg = _ecfg(sp)
    import torch.distributed as dist

    eng = TrainEngine(cfg, ecfg, world_group=dist.group.WORLD, seed=5)
    all_batches = [make_batch(cfg, 0), make_batch(cfg, 1, lens=(40, 33, 21))]
    mine = all_batches if eng.dp_size == 1 else [all_batches[eng.dp_rank]]
    eng.forward_backward_batch(mine)
    m = eng.optimizer_step()
    state = eng.full_state_dict()
    if rank == 0:
        torch.save({"state": state, "norm": m["actor/grad_norm"]}, os.path.join(out_dir, "out.pt"))


@pytest.mark.parametrize("sp", [1, 2])
def test_two_rank_fsdp_and_sequence_parallel_match_single_process(tmp_path, sp):
    """world 2: sp=1 is FSDP x DP2 (one micro-batch per rank); sp=2 is FSDP with Ulysses attention + GDN state chaining
    (every packed sequence crosses the rank boundary or ends inside a slice)."""
    cfg = HybridConfig.tiny()
    ecfg = _ecfg()
    batches = [make_batch(cfg, 0), make_batch(cfg, 1, lens=(40, 33, 21))]
    want, want_norm = reference_step(cfg, ecfg, batches, seed=5)
    run_ranks(_rank_fn, 2, tmp_path, str(tmp_path), sp)
    got = torch.load(os.path.join(str(tmp_path), "out.pt"))
    assert abs(got["norm"] - want_norm) < 2e-4 * max(1.0, want_norm)
    for k, v in want.items():
        assert torch.allclose(got["state"][k], v, atol=5e-5, rtol=2e-4), k


def _hsdp_rank_fn(rank, world, out_dir, sp):
    cfg = HybridConfig.tiny()
    ecfg = _ecfg(sp)
    ecfg.fsdp_size = 2
    import torch.distributed as dist

    eng = TrainEngine(cfg, ecfg, world_group=dist.group.WORLD, seed=5)
    assert eng.shard_world == 2 and eng.shard_rank == rank % 2 and dist.get_world_size(eng.replicate_group) == 2
    assert eng.world == 4 and eng.dp_size == 4 // sp and eng.dp_rank == rank // sp
    all_batches = _hsdp_batches(cfg)
    per = len(all_batches) // eng.dp_size
    eng.forward_backward_batch(all_batches[eng.dp_rank * per:(eng.dp_rank + 1) * per])
    m = eng.optimizer_step()
    state = eng.full_state_dict()
    torch.save({"state": state, "norm": m["actor/grad_norm"]}, os.path.join(out_dir, f"out{rank}.pt"))
    # the checkpoint's shard files: the offline merger rebuilds the tensors from the first replica's shards
    from pear_b200.train.checkpoint import CheckpointManager

    mgr = CheckpointManager(os.path.join(out_dir, "run"), rank, world, barrier=dist.barrier)
    mgr.save(1, eng)
    # every rank of every replica restores from the first replica's files
    with torch.no_grad():
        for p in eng.sharded.parameters():
            p.zero_()
    assert mgr.load(eng)["step"] == 1
    again = eng.full_state_dict()
    assert all(torch.equal(again[k], state[k]) for k in state)


def _hsdp_batches(cfg):
    return [make_batch(cfg, 0), make_batch(cfg, 1, lens=(40, 33, 21)), make_batch(cfg, 2, lens=(64,)), make_batch(cfg, 3, lens=(30, 50))]


@pytest.mark.parametrize("sp", [1, 2])
def test_hsdp_two_replicas_of_two_shards_match_single_process(tmp_path, sp):
    """world 4 with ``fsdp_size`` 2: two replicas of a 2-way sharded model. sp=1: four data-parallel ranks, one micro-batch each;
    sp=2: each replica is one sequence-parallel pair with two micro-batches. Gradients are reduce-scattered inside a shard
    group and all-reduced across the replicas on the last micro-batch; every rank ends with the single-process step's weights."""
    cfg = HybridConfig.tiny()
    ecfg = _ecfg()
    want, want_norm = reference_step(cfg, ecfg, _hsdp_batches(cfg), seed=5)
    run_ranks(_hsdp_rank_fn, 4, tmp_path, str(tmp_path), sp)
    for rank in range(4):
        got = torch.load(os.path.join(str(tmp_path), f"out{rank}.pt"))
        assert abs(got["norm"] - want_norm) < 2e-4 * max(1.0, want_norm), (rank, got["norm"], want_norm)
        for k, v in want.items():
            assert torch.allclose(got["state"][k], v, atol=5e-5, rtol=2e-4), (rank, k)
    from pear_b200.utils.model_merger import merge_shards

    actor = os.path.join(str(tmp_path), "run", "ckpt", "global_step_1", "actor")
    assert sorted(f for f in os.listdir(actor) if f.startswith("model_")) == ["model_world_size_4_rank_0.pt", "model_world_size_4_rank_1.pt"]
    merged = merge_shards(actor)
    assert all(torch.equal(merged[k], got["state"][k]) for k in want)


def test_memory_plan_of_the_27b_recipe_fits_and_names_what_does_not():
    from pear_b200.train.memory_plan import plan

    cfg = HybridConfig.qwen3_8_27b()
    ecfg = EngineConfig(ulysses_sequence_parallel_size=8, enable_gradient_checkpointing=True, enable_activation_offload=True, topk_log_probs=32)
    p = plan(cfg, ecfg, tokens_per_micro_batch=8 * 16384, shard_world=8)  # 8 sequences of 16k tokens per micro-batch over SP 8
    assert p.total_device_bytes < 0.92 * (180 << 30) and p.checkpoints_on_host and p.host_bytes > 0
    assert p.master_bytes == 4 * cfg.num_parameters() // 8 and p.optimizer_bytes == 2 * p.master_bytes
    streamed = plan(cfg, EngineConfig(ulysses_sequence_parallel_size=8, enable_activation_offload=True, streamed_adamw=True), 8 * 16384, 8)
    assert streamed.total_device_bytes == p.total_device_bytes - p.optimizer_bytes - (p.head_bytes - streamed.head_bytes) and streamed.optimizer_on_host
    with pytest.raises(MemoryError, match="shard over more ranks"):  # one GPU cannot hold the 27B model's optimizer state
        plan(cfg, ecfg, 8 * 16384, shard_world=1)
    with pytest.raises(MemoryError):  # nor can eight hold every layer's intermediates of 16k-token sequences without checkpointing
        plan(cfg, EngineConfig(ulysses_sequence_parallel_size=8, enable_gradient_checkpointing=False), 8 * 16384, 8)
    assert "device total" in p.table()


def test_engine_installs_the_family_kernels_in_order_and_runs_the_step_through_them():
    """The hooks of a model family's training kernels are called in the order the GPU backend relies on: config check before
    the model exists, install, model check, GPU backend (only when asked), checkpointing; the step runs inside ``run_checked``,
    whose rerun path zeroes the gradients first."""
    from pear_b200.models.kernels import TrainingKernels

    calls = []

    class Recording(TrainingKernels):
        @classmethod
        def check_config(cls, engine_config):
            calls.append("check_config")

        @classmethod
        def install(cls, module, fp32_residual, use_fused_kernels, fused_kernels_backend):
            calls.append(("install", fp32_residual, use_fused_kernels, type(module).__name__))

        @classmethod
        def check_model(cls, module, use_remove_padding, use_fused_kernels, fused_kernels_backend):
            calls.append(("check_model", use_remove_padding))

        @classmethod
        def install_gpu_backend(cls, module):
            calls.append("install_gpu_backend")

        @classmethod
        def install_checkpointing(cls, module):
            calls.append("install_checkpointing")

        @classmethod
        def run_checked(cls, run, before_rerun):
            calls.append("run_checked")
            first = run()  # a run whose result is thrown away (as after an overflow), then the rerun
            before_rerun()
            calls.append("rerun")
            return run()

    cfg = HybridConfig.tiny()
    ecfg = _ecfg()
    batches = [make_batch(cfg, 0)]
    want, want_norm = reference_step(cfg, ecfg, batches, seed=5)
    eng = TrainEngine(cfg, ecfg, kernels=Recording, seed=5)
    assert calls == ["check_config", ("install", True, True, "HybridForCausalLM"), ("check_model", True), "install_checkpointing"]
    eng.forward_backward_batch(batches)
    assert calls[-2:] == ["run_checked", "rerun"]
    m = eng.optimizer_step()  # the thrown-away run's gradients were cleared: the step equals a single run's
    assert abs(m["actor/grad_norm"] - want_norm) < 1e-4 * max(1.0, want_norm)
    calls.clear()
    ecfg2 = _ecfg()
    ecfg2.use_gpu_backend = True
    TrainEngine(cfg, ecfg2, kernels=Recording, seed=5)
    assert calls.index("install_gpu_backend") == calls.index(("check_model", True)) + 1 and calls[-1] == "install_checkpointing"


def test_engine_resolves_the_family_kernels_the_recipe_names(tmp_path):
    """``+qwen3_5=config`` names the family's training kernels by class path; the engine installs them (fp32 residual, fused head,
    recompute that skips down_proj) and runs the step through their overflow check."""
    from pear_b200.config.loader import compose
    from pear_b200.models.qwen3_5.training_kernels import Qwen3_5TrainingKernels

    cfg = compose("training", [f"run_dir={tmp_path}", "actor_rollout_ref.model.path=preset:tiny", "+qwen3_5=config"])
    ecfg = EngineConfig.from_config(cfg)
    assert ecfg.kernels.endswith("Qwen3_5TrainingKernels")
    ecfg.param_dtype, ecfg.lr = "fp32", 1e-3
    eng = TrainEngine(HybridConfig.tiny(), ecfg, seed=5)
    assert eng.kernels is Qwen3_5TrainingKernels and eng.model.fp32_residual and eng.model.use_fused_head and eng.model.recompute_skips_down_proj
    eng.forward_backward_batch([make_batch(HybridConfig.tiny(), 0, k=ecfg.topk_log_probs or 4)])
    assert eng.optimizer_step()["actor/grad_norm"] > 0


def _vision_rank_fn(rank, world, out_dir, sp):
    import torch.distributed as dist

    from pear_b200.models.vision import VisionConfig

    cfg = HybridConfig.tiny()
    eng = TrainEngine(cfg, _ecfg(sp), world_group=dist.group.WORLD, seed=5, vision=VisionConfig.tiny(out_hidden=cfg.hidden_size))
    eng.forward_backward_batch([_vision_batch(cfg)])
    m = eng.optimizer_step()
    state = eng.full_state_dict()
    if rank == 0:
        torch.save({"state": state, "norm": m["actor/grad_norm"]}, os.path.join(out_dir, "out.pt"))


def _vision_batch(cfg):
    from pear_b200.models.vision import VisionConfig, VisionTower

    b = make_batch(cfg, 0)
    g = torch.Generator().manual_seed(9)
    n_tok = VisionTower(VisionConfig.tiny()).tokens_per_image(16, 16)
    # three pictures: inside the first sequence, across the middle of the batch (the boundary of two sequence-parallel slices), near the end
    b.images = [(pos, torch.randint(0, 256, (16, 16, 3), generator=g, dtype=torch.uint8)) for pos in (3, b.num_tokens // 2 - n_tok // 2, b.num_tokens - n_tok - 2)]
    return b


def test_pictures_are_encoded_once_over_the_sequence_parallel_ranks_and_train_the_tower(tmp_path):
    """The trainer's own vision tower: a batch with pictures gives the same step on two sequence-parallel ranks (each picture
    encoded by one rank, rows all-gathered with gradients, one picture's rows straddling the slice boundary) as on one."""
    from pear_b200.models.vision import VisionConfig

    cfg = HybridConfig.tiny()
    eng = TrainEngine(cfg, _ecfg(), seed=5, vision=VisionConfig.tiny(out_hidden=cfg.hidden_size))
    w0 = {k: v.clone() for k, v in eng.full_state_dict().items()}
    eng.forward_backward_batch([_vision_batch(cfg)])
    m = eng.optimizer_step()
    want = eng.full_state_dict()
    assert any(k.startswith("visual.") and not torch.equal(w0[k], want[k]) for k in want)  # the tower moved
    run_ranks(_vision_rank_fn, 2, tmp_path, str(tmp_path), 2)
    got = torch.load(os.path.join(str(tmp_path), "out.pt"))
    assert abs(got["norm"] - m["actor/grad_norm"]) < 2e-4 * max(1.0, m["actor/grad_norm"])
    for k, v in want.items():
        assert torch.allclose(got["state"][k], v, atol=5e-5, rtol=2e-4), k

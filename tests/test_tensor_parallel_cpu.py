"""Tensor-parallel rollout on two gloo ranks: the sharded model's hidden states and a whole engine generation equal
the single-rank model's."""

import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM, set_tensor_parallel_group
from pear_b200.parallel.tensor_parallel import shard_state, tp_config
from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams


def _cfg() -> HybridConfig:
    return HybridConfig.tiny()


def _worker(rank, world, path, q):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = _cfg()
    full = HybridForCausalLM(cfg, with_mtp=False).init_weights(3)
    ids = torch.arange(1, 48) % cfg.vocab_size
    ref_h = full(ids, cu_seqlens=[0, 20, 47])
    prompts = [list(range(1, 30)), list(range(5, 22))]
    ref_out = [r.output for r in RolloutEngine(full, EngineConfig(num_blocks=128, max_num_seqs=4)).generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))]
    tp = HybridForCausalLM(tp_config(cfg, world), with_mtp=False)
    missing, unexpected = tp.load_state_dict(shard_state(full.state_dict(), cfg, rank, world), strict=True)
    set_tensor_parallel_group(dist.group.WORLD)
    try:
        h = tp(ids, cu_seqlens=[0, 20, 47])
        out = [r.output for r in RolloutEngine(tp, EngineConfig(num_blocks=128, max_num_seqs=4)).generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))]
    finally:
        set_tensor_parallel_group(None)
    q.put((rank, float((h - ref_h).abs().max()), float(ref_h.abs().max()), out == ref_out))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_tp2_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_worker, args=(r, 2, os.path.join(d, "rdzv"), q)) for r in range(2)]
        for p in procs:
            p.start()
        res = sorted(q.get(timeout=240) for _ in range(2))
        for p in procs:
            p.join(30)
    for rank, err, scale, same in res:
        assert err <= 1e-4 * max(1.0, scale), (rank, err, scale)
        assert same, f"rank {rank}: generated tokens differ from the single-rank model"


def test_tp_config_refuses_uneven_splits():
    with pytest.raises(ValueError, match="num_attention_heads=4"):
        tp_config(_cfg(), 3)


def test_kv_heads_are_replicated_when_ranks_outnumber_them():
    """4 ranks over 2 KV heads: ranks 0, 1 hold KV head 0 and ranks 2, 3 hold head 1; each rank keeps one query head."""
    cfg = _cfg()
    full = HybridForCausalLM(cfg, with_mtp=False).init_weights(1).state_dict()
    local = tp_config(cfg, 4)
    assert (local.num_attention_heads, local.num_kv_heads) == (1, 1)
    name = "model.layers.3.self_attn.k_proj.weight"
    d = cfg.head_dim
    for rank in range(4):
        part = shard_state(full, cfg, rank, 4)
        assert torch.equal(part[name], full[name][(rank // 2) * d:(rank // 2 + 1) * d])
        HybridForCausalLM(local, with_mtp=False).load_state_dict(part, strict=True)


def _vision_worker(rank, world, path, q):
    from pear_b200.models.vision import VisionConfig, VisionTower
    from pear_b200.parallel.vision_sp import encode_sharded, reduce_tower_grads

    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    images = [torch.randn(3, 16, 16, generator=g), torch.randn(3, 32, 16, generator=g), torch.randn(3, 16, 16, generator=g)]
    tower = VisionTower(VisionConfig.tiny(out_hidden=32)).init_weights(1)
    ref_tower = VisionTower(VisionConfig.tiny(out_hidden=32)).init_weights(1)
    want = ref_tower(images)
    torch.cat(want).pow(2).sum().backward()
    got = encode_sharded(tower, images, dist.group.WORLD)
    # every rank consumes every image's rows; the loss is counted once per rank, so scale by 1 / world
    (torch.cat(got).pow(2).sum() / world).backward()
    reduce_tower_grads(tower, dist.group.WORLD)
    err_f = max(float((a - b).abs().max()) for a, b in zip(got, want))
    err_g = max(float((p.grad - r.grad).abs().max()) for p, r in zip(tower.parameters(), ref_tower.parameters()))
    q.put((rank, err_f, err_g))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_vision_tower_sharded_over_ranks_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_vision_worker, args=(r, 2, os.path.join(d, "rdzv"), q)) for r in range(2)]
        for p in procs:
            p.start()
        res = [q.get(timeout=240) for _ in range(2)]
        for p in procs:
            p.join(30)
    for rank, err_f, err_g in res:
        assert err_f < 1e-5 and err_g < 1e-4, (rank, err_f, err_g)

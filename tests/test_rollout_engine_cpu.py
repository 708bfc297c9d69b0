"""Rollout engine on CPU with the tiny hybrid model: paged decode equals the dense cached oracle, prefix caching across
turns resumes from the recurrent-state snapshot, chunked prefill, preemption, pause/abort, weight update invalidation,
host tier promotion, and lossless MTP speculative decoding."""

import pytest
import torch

from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import DenseCache, HybridForCausalLM, forward_cached
from pear_b200.rollout.engine import EngineConfig, FinishReason, RolloutEngine, SamplingParams


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    m = HybridForCausalLM(HybridConfig.tiny(), with_mtp=True).init_weights(3).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.mul_(3.0)  # peaked enough distributions for greedy comparisons to be stable
    return m


def greedy_oracle(model, prompt, n):
    cache = DenseCache(model.config)
    h = forward_cached(model, torch.tensor(prompt), cache)
    out = []
    for _ in range(n):
        tok = int(model.logits(h[-1:]).argmax())
        out.append(tok)
        h = forward_cached(model, torch.tensor([tok]), cache)
    return out


def test_paged_greedy_decode_matches_dense_oracle(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16, max_num_batched_tokens=48))
    prompts = [list(range(3, 40)), list(range(100, 170)), [7, 8, 9]]
    reqs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, r in zip(prompts, reqs):
        assert r.finish == FinishReason.LENGTH
        assert r.output == greedy_oracle(model, p, 12)
    assert eng.blocks.num_free == 63  # everything released (block 0 is the null block)


def test_prefix_cache_across_turns_resumes_recurrent_state(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16))
    turn1 = list(range(5, 5 + 40))
    r1 = eng.generate([turn1], SamplingParams(max_tokens=9, temperature=0.0), sessions=["s"])[0]
    turn2 = turn1 + r1.output + list(range(200, 230))
    r2 = eng.generate([turn2], SamplingParams(max_tokens=6, temperature=0.0), sessions=["s"])[0]
    # 49 tokens were committed by turn 1 -> 3 full blocks, the last one carrying the state snapshot
    assert r2.cached_prefix == 48
    assert r2.output == greedy_oracle(model, turn2, 6)
    st = eng.stats()
    assert st["prefix_cache_hits"] >= 48


def test_weight_update_invalidates_prefix_cache(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16))
    p = list(range(5, 60))
    eng.generate([p], SamplingParams(max_tokens=4, temperature=0.0))
    assert eng.stats()["cached_blocks"] > 0
    eng.pause(abort=True)
    eng.update_weights({k: v.clone() for k, v in model.state_dict().items()})
    eng.resume()
    assert eng.stats()["cached_blocks"] == 0 and eng.policy_version == 1
    r = eng.generate([p], SamplingParams(max_tokens=4, temperature=0.0))[0]
    assert r.cached_prefix == 0 and r.policy_version == 1


def test_pause_in_abort_mode_returns_inflight_requests(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16))
    a = eng.add_request(list(range(5, 50)), SamplingParams(max_tokens=50, temperature=0.0))
    for _ in range(3):
        eng.step()
    aborted = eng.pause(abort=True)
    assert aborted == [a] and a.finish == FinishReason.ABORTED and len(a.output) >= 1
    rejected = eng.add_request([1, 2, 3])
    assert rejected.finish == FinishReason.ABORTED
    eng.resume()
    again = eng.generate([a.prompt + a.output], SamplingParams(max_tokens=5, temperature=0.0))[0]
    assert again.output == greedy_oracle(model, a.prompt + a.output, 5)
    assert eng.blocks.num_free == 63


def test_preemption_under_memory_pressure_keeps_results_exact(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=12, block_size=16, enable_prefix_caching=False))
    prompts = [list(range(10, 58)), list(range(60, 108)), list(range(110, 150))]
    reqs = eng.generate(prompts, SamplingParams(max_tokens=20, temperature=0.0))
    assert eng.metrics["preemptions"] > 0
    for p, r in zip(prompts, reqs):
        assert r.output == greedy_oracle(model, p, 20)


def test_host_tier_brings_back_evicted_prefix(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=10, block_size=16, host_blocks=32))
    a = list(range(5, 5 + 64))
    ra = eng.generate([a], SamplingParams(max_tokens=1, temperature=0.0), sessions=["a"])[0]
    # other traffic evicts a's blocks from the device
    eng.generate([list(range(300, 420))], SamplingParams(max_tokens=2, temperature=0.0), sessions=["b"])
    rb = eng.generate([a + ra.output + [9, 9, 9]], SamplingParams(max_tokens=4, temperature=0.0), sessions=["a"])[0]
    assert rb.cached_prefix == 64 and eng.stats()["external_prefix_cache_hits"] > 0
    assert rb.output == greedy_oracle(model, a + ra.output + [9, 9, 9], 4)


def test_mtp_speculative_decoding_is_lossless_for_greedy(model):
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16, num_speculative_tokens=3))
    p = list(range(20, 61))
    r = eng.generate([p], SamplingParams(max_tokens=24, temperature=0.0))[0]
    # temperature 0 is served as temperature -> 0: rejection sampling at a tiny temperature is greedy up to ties
    want = greedy_oracle(model, p, 24)
    assert r.output == want
    assert r.spec_drafted > 0


def test_prefill_fills_the_drafter_kv_cache(model):
    """Every prompt position but the last gets its drafter KV during prefill (the last one when its successor is sampled): the
    pages of the drafter's layer hold the same keys as a dense MTP pass over the whole prompt."""
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, block_size=16, num_speculative_tokens=3, max_num_batched_tokens=24))
    p = list(range(20, 61))  # 41 tokens: two prefill chunks of 24 and 17 rows
    req = eng.add_request(p, SamplingParams(max_tokens=2, temperature=0.0))
    while req.finish is None and len(req.output) < 1:
        eng.step()
    table = req.block_table
    mk = eng.runner.mtp_k[0]
    got = torch.stack([mk[table[i // 16], i % 16] for i in range(len(p))]).float()
    assert (got.abs().sum(dim=(1, 2)) > 0).all()  # no prompt position was left empty
    # dense oracle: the MTP layer's keys over the prompt with the sampled token as the last successor
    from pear_b200.rollout.model_runner import linear_fp32  # noqa: F401  (the same projection helpers as the runner)
    m, mtp = model, model.mtp
    toks = torch.tensor(p + req.output[:1])
    hidden = m(toks[:-1], torch.arange(len(p)), [0, len(p)])
    x = torch.cat([mtp.pre_fc_norm_embedding(m.model.embed_tokens(toks[1:]).float()), mtp.pre_fc_norm_hidden(hidden)], dim=-1)
    r = torch.nn.functional.linear(x, mtp.fc.weight.float())
    attn = mtp.layers[0].self_attn
    h = mtp.layers[0].input_layernorm(r)
    cos, sin = m.rope(torch.arange(len(p)))
    k = attn.k_norm(torch.nn.functional.linear(h, attn.k_proj.weight.float()).view(len(p), -1, m.config.head_dim))
    from pear_b200.ops import reference as ref
    k = ref.apply_rope(k, cos, sin)
    assert torch.allclose(got, k.to(got.dtype).float(), atol=2e-2, rtol=2e-2)


def test_lookup_keeps_matched_chain_blocks_out_of_eviction():
    """A prefix whose head sits on the device (oldest LRU entry) and whose tail sits in the host tier: promoting the tail
    needs a device block while the free list is empty, and must not evict (and overwrite) the matched head."""
    from pear_b200.rollout.block_manager import BlockManager
    from pear_b200.rollout.host_tier import HostTier

    bs = 4
    kv = [torch.zeros(4, bs, 2)]
    mgr = BlockManager(4, bs, 4, True, needs_state=False)  # block 0 is the null block: three usable blocks
    mgr.host_tier = HostTier(8, kv, [], pin=False)
    toks = list(range(12))
    blocks = [mgr.allocate() for _ in range(3)]
    parent = None
    for i, blk in enumerate(blocks):
        kv[0][blk] = float(i + 1)  # block i holds the payload i + 1
        parent = mgr.publish(blk, parent, toks[i * bs:(i + 1) * bs])
    # tail blocks 1 and 2 leave the device first (into the host tier), then the head is released: it is the only LRU entry
    mgr.release(blocks[1]); mgr.release(blocks[2])
    x, y = mgr.allocate(), mgr.allocate()  # evicts blocks 1 and 2 into the host tier
    mgr.release(blocks[0])
    mgr.release(x)  # one unpublished free block: enough for ONE promotion; the second has only the LRU to take from
    hit = mgr.lookup(toks)
    assert hit.blocks[0] == blocks[0] and len(set(hit.blocks)) == len(hit.blocks), hit.blocks
    for i, blk in enumerate(hit.blocks):
        assert float(kv[0][blk].mean()) == float(i + 1), "a chain block was overwritten by a promotion"
    assert hit.tokens in (4, 8)  # the head always; the tail as far as free blocks allowed
    mgr.release(y)


def test_host_tier_sized_in_bytes_prefaulted_and_local_to_the_bound_node():
    """``host_bytes`` holds as many blocks as fit; the tier is touched at construction; after binding the process to NUMA node 0
    the tier's resident pages are reported on it (the platform may not answer: then no figure, never a wrong one)."""
    import os

    from pear_b200.rollout.host_tier import HostTier
    from pear_b200.utils.process import node_cpus, numa_locality, set_numa_affinity, visible_gpu_index

    before = os.sched_getaffinity(0)
    try:
        bound = os.path.exists("/sys/devices/system/node/node0/cpulist") and set_numa_affinity(0)
        if bound:
            assert os.sched_getaffinity(0) == set(node_cpus(0)) & before or os.sched_getaffinity(0) == set(node_cpus(0))
        assert not set_numa_affinity(4095)  # no such node: refused, nothing changed
        model = HybridForCausalLM(HybridConfig.tiny(), with_mtp=False).init_weights(0)
        probe = RolloutEngine(model, EngineConfig(num_blocks=32, max_num_seqs=2))
        per_block = HostTier.bytes_per_block(probe.runner.kv_tensors(), probe.runner.state_tensors())
        assert per_block > 0
        eng = RolloutEngine(model, EngineConfig(num_blocks=32, max_num_seqs=2, host_bytes=10 * per_block + per_block // 2, host_numa_node=0 if bound else None))
        assert eng.host is not None and eng.host.capacity == 10
        if bound and eng.host_locality is not None:
            assert eng.host_locality >= 0.95
        t = torch.ones(1 << 20)
        frac = numa_locality(t.data_ptr(), t.numel() * 4, 0)
        assert frac is None or 0.0 <= frac <= 1.0
    finally:
        os.sched_setaffinity(0, before)
    os.environ["CUDA_VISIBLE_DEVICES"], saved = "5,2", os.environ.get("CUDA_VISIBLE_DEVICES")
    try:
        assert visible_gpu_index(0) == 5 and visible_gpu_index(1) == 2
    finally:
        if saved is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES")
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = saved


def test_a_seeded_request_draws_the_same_tokens_whatever_shares_its_batch():
    model = HybridForCausalLM(HybridConfig.tiny(), with_mtp=False).init_weights(0)
    p = SamplingParams(max_tokens=8, temperature=1.0, seed=1234)
    prompt = list(range(5, 25))
    alone = RolloutEngine(model, EngineConfig(num_blocks=64, max_num_seqs=4, seed=1)).generate([prompt], p)[0].output
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, max_num_seqs=4, seed=99))
    a = eng.add_request(list(range(40, 70)), SamplingParams(max_tokens=8, temperature=1.0))
    b = eng.add_request(prompt, p)
    c = eng.add_request(list(range(3, 9)), SamplingParams(max_tokens=8, temperature=1.0, seed=7))
    while eng.has_work():
        eng.step()
    assert b.output == alone and len(a.output) == 8 and len(c.output) == 8
    other_seed = RolloutEngine(model, EngineConfig(num_blocks=64, max_num_seqs=4, seed=1)).generate([prompt], SamplingParams(max_tokens=8, temperature=1.0, seed=4321))[0].output
    assert other_seed != alone

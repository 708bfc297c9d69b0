"""The rollout engine on a GPU with the batched GPU-resident step: sampled tokens and their reported log-probs against the
fp32 PyTorch oracle of the model run over the finished sequences (teacher forcing), across prefill -> fast-step hand-off,
speculative verification, stop cuts and a second turn that resumes from the prefix cache."""

import pytest
import torch

from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM

pytestmark = pytest.mark.gpu


def _models():
    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256, gdn_qk_heads=2,
                       gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=1, init_std=0.05)
    oracle = HybridForCausalLM(cfg).init_weights(3)
    with torch.no_grad():
        for p in oracle.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    fast = HybridForCausalLM(cfg)
    fast.load_state_dict(oracle.state_dict())
    fast = fast.cuda().eval()
    for name, p in fast.named_parameters():
        if p.dim() >= 2 and "conv1d" not in name:
            p.data = p.data.to(torch.bfloat16)
    return cfg, oracle.cuda().eval(), fast


def _oracle_logprobs(oracle, tokens: list[int], n_prompt: int, temperature: float) -> torch.Tensor:
    from pear_b200.ops import api

    prev, api.FORCE_REFERENCE = api.FORCE_REFERENCE, True
    try:
        with torch.no_grad():
            ids = torch.tensor(tokens, device="cuda")
            h = oracle(ids)
            lp = torch.log_softmax(oracle.logits(h[n_prompt - 1:-1]) / temperature, -1)
        return lp.gather(1, ids[n_prompt:, None])[:, 0].cpu()
    finally:
        api.FORCE_REFERENCE = prev


@pytest.mark.parametrize("spec", [0, 3])
def test_engine_fast_step_against_oracle(spec):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.rollout.engine import EngineConfig, FinishReason, RolloutEngine, SamplingParams

    cfg, oracle, model = _models()
    eng = RolloutEngine(model, EngineConfig(num_blocks=256, max_num_seqs=8, num_speculative_tokens=spec, seed=11), device="cuda")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (19, 67, 37, 16, 51)]  # the first two end their turn on a page boundary (33 and 81 tokens)
    temp = 0.8
    params = SamplingParams(max_tokens=14, temperature=temp)
    reqs = eng.generate(prompts, params, sessions=[f"s{i}" for i in range(len(prompts))])
    assert eng.fast is not None and eng.fast.steps > 0, "decode rows did not go through the batched GPU-resident step"
    for r, pr in zip(reqs, prompts):
        assert r.finish == FinishReason.LENGTH and len(r.output) == 14
        want = _oracle_logprobs(oracle, pr + r.output, len(pr), temp)
        got = torch.tensor(r.logprobs)
        assert (got - want).abs().max() < 0.15, (got, want)
    if spec:
        assert eng.metrics["spec_drafted"] > 0
    # second turn of two sessions: the prompt extends the first turn; it must hit the prefix the first turn published
    # (KV pages and the recurrent-state snapshot the fast step's release wrote back) and still follow the oracle
    follow = []
    for r, pr in list(zip(reqs, prompts))[:2]:
        follow.append(pr + r.output + torch.randint(0, cfg.vocab_size, (9,), generator=g).tolist())
    stop_tok = None
    reqs2 = eng.generate(follow, SamplingParams(max_tokens=10, temperature=temp), sessions=["s0", "s1"])
    for r, pr in zip(reqs2, follow):
        assert r.cached_prefix >= 16, r.cached_prefix
        want = _oracle_logprobs(oracle, pr + r.output, len(pr), temp)
        assert (torch.tensor(r.logprobs) - want).abs().max() < 0.15
        stop_tok = r.output[4]
    # a stop token in the middle of what a verify step accepts: the sequence ends there, later turns resume from the cut
    reqs3 = eng.generate([follow[1]], SamplingParams(max_tokens=10, temperature=temp, stop_token_ids=(stop_tok,)), sessions=["s1"])
    assert reqs3[0].finish in (FinishReason.STOP, FinishReason.LENGTH)
    assert eng.stats()["num_running"] == 0 and not eng._fast_slot


def test_fast_path_returns_top_logprobs():
    """Requests that ask for top log-probs (what the training recipe's score centering reads) stay on the batched step; the
    lists agree with the top of log_softmax of the oracle's logits at every generated position."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import api
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    cfg, oracle, model = _models()
    eng = RolloutEngine(model, EngineConfig(num_blocks=128, max_num_seqs=4, num_speculative_tokens=3, seed=3), device="cuda")
    prompts = [list(range(5, 30)), list(range(40, 52))]
    temp, k = 0.9, 5
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, temperature=temp, topk_logprobs=k))
    assert eng.fast is not None and eng.fast.topk and eng.fast.steps > 0  # the batched step ran and produced the lists
    prev, api.FORCE_REFERENCE = api.FORCE_REFERENCE, True
    try:
        for p, r in zip(prompts, outs):
            assert len(r.topk_ids) == len(r.output) == 6 and all(len(x) == k for x in r.topk_ids)
            with torch.no_grad():
                ids = torch.tensor(p + r.output, device="cuda")
                lp = torch.log_softmax(oracle.logits(oracle(ids)[len(p) - 1:-1]) / temp, -1)
            for j in range(6):
                row = lp[j]
                got_lp = torch.tensor(r.topk_logprobs[j], device="cuda")
                got_id = torch.tensor(r.topk_ids[j], device="cuda")
                assert (got_lp[:-1] >= got_lp[1:]).all() and len(set(r.topk_ids[j])) == k
                # bf16 activations in the step against the fp32 oracle: values to a bf16-level bound, and every listed token is
                # within that bound of the oracle's k-th value
                assert torch.allclose(got_lp, row[got_id], atol=0.15), (j, got_lp, row[got_id])
                assert float(row[got_id].min()) >= float(row.topk(k).values[-1]) - 0.3
                assert abs(r.logprobs[j] - float(row[r.output[j]])) < 0.15
    finally:
        api.FORCE_REFERENCE = prev

"""NVTX ranges: a no-op unless switched on, push / pop pairs around the annotated phases when on."""

import pytest
import torch

from pear_b200.utils import nvtx


def test_annotate_is_a_no_op_without_cuda_or_when_off():
    nvtx.enable(False)
    before = nvtx.ranges_opened
    with nvtx.annotate("x"):
        pass
    assert nvtx.ranges_opened == before
    if not torch.cuda.is_available():
        nvtx.enable(True)
        try:
            with nvtx.annotate("x"):
                pass
            assert nvtx.ranges_opened == before
        finally:
            nvtx.enable(False)


@pytest.mark.gpu
def test_rollout_step_opens_a_range_when_enabled():
    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    cfg = HybridConfig(vocab_size=4096, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=256, gdn_qk_heads=2,
                       gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=1, init_std=0.05)
    model = HybridForCausalLM(cfg).init_weights(3).cuda()
    eng = RolloutEngine(model, EngineConfig(num_blocks=64, max_num_seqs=2), device="cuda")
    nvtx.enable(True)
    try:
        before = nvtx.ranges_opened
        eng.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=3, temperature=1.0))
        assert nvtx.ranges_opened > before
    finally:
        nvtx.enable(False)

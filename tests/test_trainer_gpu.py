"""The training loop on one B200 with the tiny model: rollout, GRPO step through the CUDA kernels, weight sync."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(900)
def test_one_training_step_on_gpu(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from pear_b200.ops import lib as kl
    from test_trainer_e2e_cpu import _cfg
    from pear_b200.train.main import build_stack

    kl.lib()  # the CUDA library must be present on a GPU box
    before = kl.LAUNCH_COUNT
    trainer, close = build_stack(_cfg(str(tmp_path / "run"), ["trainer.total_training_steps=1", "trainer.save_freq=-1"]), device="cuda")
    trainer.cfg.sample_timeout_s = 180.0  # a broken rollout path fails the test quickly
    try:
        hist = trainer.fit()
        assert len(hist) == 1 and np.isfinite(hist[0]["actor/grad_norm"]) and trainer.engine.policy_version == 1
        assert kl.LAUNCH_COUNT > before, "the step must run this library's kernels, not a fallback"
    finally:
        close()


def test_retained_attention_outputs_give_the_same_gradients():
    """A checkpointed attention layer that replays the first pass's attention output in its recompute pass has the
    gradients of one that recomputes it, and launches one attention kernel less."""
    import torch

    from pear_b200.models.config import HybridConfig
    from pear_b200.ops import lib as kl
    from pear_b200.train.engine import synthetic_batch
    from pear_b200.train.engine import EngineConfig, TrainEngine

    cfg = HybridConfig(vocab_size=2048, hidden_size=512, num_layers=4, num_attention_heads=4, num_kv_heads=1, head_dim=256, rotary_dim=64,
                       gdn_qk_heads=2, gdn_v_heads=4, gdn_head_dim=128, intermediate_size=1024, num_mtp_layers=0)
    grads, launches = {}, {}
    for retain in (False, True):
        eng = TrainEngine(cfg, EngineConfig(lr=1e-6, param_dtype="bf16", enable_gradient_checkpointing=True, topk_log_probs=0,
                                            gradient_checkpointing_retain_attention=retain), device="cuda", seed=0)
        batch = synthetic_batch(cfg, 512, 2, 0, 0).to("cuda")
        before = kl.LAUNCH_COUNT
        eng.forward_backward_batch([batch])
        launches[retain] = kl.LAUNCH_COUNT - before
        grads[retain] = torch.cat([p.grad.float().flatten() for p in eng.sharded.parameters() if p.grad is not None])
    assert launches[True] == launches[False] - 1  # one attention layer: its recompute pass skipped the forward kernel
    # not bit-equal: the library attention backward and the norm weight gradients accumulate with atomics (bf16-level noise)
    assert ((grads[True] - grads[False]).norm() / grads[False].norm()).item() < 2e-2

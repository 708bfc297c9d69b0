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

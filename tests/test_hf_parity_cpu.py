"""The model against the Hugging Face implementation of the family it is written for (``transformers``' Qwen3.5 text model, fp32
on CPU, its torch fallback for the linear-attention layers): a checkpoint saved by ``transformers`` loads here without a missing
or an unexpected tensor and gives the same logits; a model exported here loads there; the rollout engine's greedy continuation
(prefill, paged KV, recurrent state, decode steps) equals ``generate``."""

import pytest
import torch

transformers = pytest.importorskip("transformers")
if not hasattr(transformers, "Qwen3_5ForCausalLM"):
    pytest.skip("this transformers has no Qwen3.5 text model", allow_module_level=True)

from pear_b200.models import io as model_io  # noqa: E402
from pear_b200.models.hybrid import HybridForCausalLM  # noqa: E402


def _hf_model(seed: int = 0):
    from transformers import Qwen3_5ForCausalLM, Qwen3_5TextConfig

    cfg = Qwen3_5TextConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                            linear_num_value_heads=4, layer_types=["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                            max_position_embeddings=512)
    torch.manual_seed(seed)
    m = Qwen3_5ForCausalLM(cfg).eval().float()
    with torch.no_grad():  # norms away from their initial values, larger projections: differences would show
        for n, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
            else:
                p.mul_(3.0)
    return m


def test_transformers_checkpoint_loads_and_gives_the_same_logits(tmp_path):
    hf = _hf_model()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    cfg = model_io.load_config(str(tmp_path / "hf"))
    assert cfg.layer_types == ["linear_attention"] * 3 + ["full_attention"] and cfg.rotary_dim == 8 and cfg.attn_output_gate
    mine = HybridForCausalLM(cfg, with_mtp=False)
    missing, unexpected = model_io.load_model_dir(str(tmp_path / "hf"), mine)
    assert not missing and not unexpected
    g = torch.Generator().manual_seed(1)
    a, b = torch.randint(0, 512, (41,), generator=g), torch.randint(0, 512, (23,), generator=g)
    with torch.no_grad():
        want_a, want_b = hf(a[None]).logits[0], hf(b[None]).logits[0]
        got_a = mine.logits(mine(a, torch.arange(41), [0, 41]))
        # two sequences packed into one call: neither sees the other (attention mask, conv window, recurrent state)
        packed = mine.logits(mine(torch.cat([a, b]), torch.cat([torch.arange(41), torch.arange(23)]), [0, 41, 64]))
    scale = float(want_a.abs().max())
    assert float((got_a - want_a).abs().max()) < 1e-5 * max(1.0, scale)
    assert float((packed[:41] - want_a).abs().max()) < 1e-5 * max(1.0, scale) and float((packed[41:] - want_b).abs().max()) < 1e-5 * max(1.0, scale)


def test_exported_model_loads_in_transformers_with_the_same_logits(tmp_path):
    from transformers import Qwen3_5ForCausalLM

    hf = _hf_model(2)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    cfg = model_io.load_config(str(tmp_path / "hf"))
    mine = HybridForCausalLM(cfg, with_mtp=False).init_weights(7)  # this framework's own weights, exported
    model_io.save_model_dir(str(tmp_path / "out"), cfg, mine.state_dict(), dtype=torch.float32)
    back = Qwen3_5ForCausalLM.from_pretrained(str(tmp_path / "out")).eval().float()
    ids = torch.randint(0, 512, (29,), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want = mine.logits(mine(ids, torch.arange(29), [0, 29]))
        got = back(ids[None]).logits[0]
    assert float((got - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))


def test_rollout_engine_greedy_continuation_equals_generate(tmp_path):
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    hf = _hf_model(4)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    mine = HybridForCausalLM(model_io.load_config(str(tmp_path / "hf")), with_mtp=False)
    model_io.load_model_dir(str(tmp_path / "hf"), mine)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 33)]
    eng = RolloutEngine(mine, EngineConfig(num_blocks=64, max_num_seqs=4))
    outs = eng.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0))
    for p, r in zip(prompts, outs):
        with torch.no_grad():
            want = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, pad_token_id=0)[0, len(p):].tolist()
        assert r.output == want

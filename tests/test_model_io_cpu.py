"""Model directories in the Hugging Face layout: key names, config translation, strict loading."""

import json
import os

import pytest
import torch

from pear_b200.models import io as model_io
from pear_b200.models.config import HybridConfig
from pear_b200.models.hybrid import HybridForCausalLM


def test_export_uses_hf_names_and_round_trips(tmp_path):
    cfg = HybridConfig.tiny()
    model = HybridForCausalLM(cfg).init_weights(2)
    out = str(tmp_path / "export")
    model_io.save_model_dir(out, cfg, model.state_dict(), dtype=torch.float32, drop_mtp=False)
    keys = set(model_io.load_safetensors(os.path.join(out, "model.safetensors")))
    assert "model.language_model.layers.0.linear_attn.in_proj_qkv.weight" in keys
    assert "model.language_model.embed_tokens.weight" in keys and "lm_head.weight" in keys and "mtp.fc.weight" in keys
    assert not any(k.startswith("model.layers.") for k in keys)
    hf = json.load(open(os.path.join(out, "config.json")))
    t = hf["text_config"]
    assert (t["num_hidden_layers"], t["num_key_value_heads"], t["linear_num_value_heads"]) == (cfg.num_layers, cfg.num_kv_heads, cfg.gdn_v_heads)
    back = HybridForCausalLM(model_io.load_config(out))
    missing, unexpected = model_io.load_model_dir(out, back)
    assert not missing and not unexpected
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), back.state_dict().values()))


def test_plain_hf_config_is_translated(tmp_path):
    """A config.json with only the transformers field names (no field of this framework) yields the same model shape."""
    cfg = HybridConfig.tiny()
    d = cfg.to_hf_dict()
    path = str(tmp_path / "config.json")
    json.dump(d, open(path, "w"))
    got = HybridConfig.load(path)
    assert got.to_dict() == cfg.to_dict()
    with pytest.raises(KeyError):
        json.dump({"hidden_size": 8}, open(path, "w"))
        HybridConfig.load(path)


def test_loading_a_directory_that_does_not_match_raises(tmp_path):
    cfg = HybridConfig.tiny()
    model = HybridForCausalLM(cfg, with_mtp=False).init_weights(2)
    state = model.state_dict()
    out = str(tmp_path / "partial")
    model_io.save_model_dir(out, cfg, {k: v for k, v in state.items() if "layers.2." not in k}, dtype=torch.float32)
    fresh = HybridForCausalLM(cfg, with_mtp=False)
    with pytest.raises(KeyError, match="parameters missing"):
        model_io.load_model_dir(out, fresh)
    missing, _ = model_io.load_model_dir(out, fresh, strict=False)
    assert missing and all("layers.2." in k for k in missing)
    # a checkpoint that also carries the drafter and a vision tower loads into a text-only model without complaint
    full = HybridForCausalLM(cfg).init_weights(2).state_dict()
    full["visual.patch_embed.weight"] = torch.zeros(4, 4)
    out2 = str(tmp_path / "full")
    model_io.save_model_dir(out2, cfg, full, dtype=torch.float32, drop_mtp=False)
    assert "model.visual.patch_embed.weight" in model_io.load_safetensors(os.path.join(out2, "model.safetensors"))
    missing, unexpected = model_io.load_model_dir(out2, fresh)
    assert not missing and all(k.startswith(("mtp.", "visual.")) for k in unexpected)


def test_replica_takes_its_frozen_drafter_from_the_base_model_directory(tmp_path):
    """A trained checkpoint is exported without the drafter; the replica reads the base directory's ``mtp.*`` tensors for it,
    the rest strictly from the trained directory, and a weight sync without drafter tensors leaves the drafter as loaded."""
    import torch

    from pear_b200.models import io as model_io
    from pear_b200.models.config import HybridConfig
    from pear_b200.models.hybrid import HybridForCausalLM
    from pear_b200.rollout.engine import EngineConfig, SamplingParams
    from pear_b200.rollout.server import build_server, load_rollout_model

    cfg = HybridConfig.tiny()
    base = HybridForCausalLM(cfg, with_mtp=True).init_weights(1)
    trained = HybridForCausalLM(cfg, with_mtp=False).init_weights(2)
    model_io.save_model_dir(str(tmp_path / "base"), cfg, base.state_dict(), dtype=torch.float32, drop_mtp=False)
    model_io.save_model_dir(str(tmp_path / "trained"), cfg, trained.state_dict(), dtype=torch.float32)  # no drafter inside
    assert any(n.startswith("mtp.") for n in map(model_io.from_hf_name, model_io.model_tensor_names(str(tmp_path / "base"))))
    assert not any(n.startswith("mtp.") for n in map(model_io.from_hf_name, model_io.model_tensor_names(str(tmp_path / "trained"))))
    m = load_rollout_model(str(tmp_path / "trained"), drafter_path=str(tmp_path / "base"))
    got, want_body, want_mtp = m.state_dict(), trained.state_dict(), base.state_dict()
    assert m.mtp is not None and all(torch.equal(got[k], want_body[k]) for k in want_body)
    assert all(torch.equal(got[k], want_mtp[k]) for k in want_mtp if k.startswith("mtp."))
    assert load_rollout_model(str(tmp_path / "trained")).mtp is None          # no drafter anywhere: none built
    assert load_rollout_model(str(tmp_path / "base")).mtp is not None         # a directory that carries its own
    with pytest.raises(KeyError, match="holds no mtp"):
        load_rollout_model(str(tmp_path / "trained"), drafter_path=str(tmp_path / "trained"))
    # speculative decoding runs with it, and a sync of the trainer's (drafter-less) state leaves it frozen
    srv = build_server(m, EngineConfig(num_blocks=64, max_num_seqs=2, num_speculative_tokens=2))
    try:
        r = srv.generate(list(range(3, 20)), SamplingParams(max_tokens=6, temperature=0.0))
        assert len(r.output) == 6 and srv.engine.metrics["spec_drafted"] > 0
        srv.pause(abort=True)
        srv.update_weights({k: v * 0.5 for k, v in trained.state_dict().items()}, version=1)
        srv.resume()
        after = srv.engine.model.state_dict()
        assert all(torch.equal(after[k].float(), want_mtp[k]) for k in want_mtp if k.startswith("mtp."))
    finally:
        srv.close()


def test_model_directory_tokenizer_is_read_and_renders_the_chat_template(tmp_path):
    """A directory with a ``tokenizer.json`` gets the reader over the ``tokenizers`` package (same interface as the byte
    tokenizer); one without, or a preset, gets the byte tokenizer; a vocabulary without the chat specials is refused."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    from pear_b200.utils.tokenizer import ByteTokenizer, HFTokenizer, load_tokenizer

    words = ["user", "assistant", "system", "pick", "the", "cube", "front", "[", "]", "\n", "Ċ"]
    vocab = {w: i for i, w in enumerate(words)}
    vocab["[UNK]"] = len(vocab)
    tk = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tk.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split("\n", "isolated"), pre_tokenizers.WhitespaceSplit(), pre_tokenizers.Punctuation()])
    tk.add_special_tokens(["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>"])
    d = tmp_path / "model"
    d.mkdir()
    tk.save(str(d / "tokenizer.json"))
    (d / "generation_config.json").write_text('{"eos_token_id": [%d, %d]}' % (tk.token_to_id("<|im_end|>"), tk.token_to_id("<|endoftext|>")))
    tok = load_tokenizer(str(d))
    assert isinstance(tok, HFTokenizer) and tok.eos_id == tk.token_to_id("<|im_end|>") and tok.extra_stop_ids == (tk.token_to_id("<|endoftext|>"),)
    ids = tok.render_turn("user", "pick the cube", images=1, image_tokens=3, labels=["front"]) + tok.generation_prompt()
    assert ids[0] == tok.special_ids["<|im_start|>"] and ids.count(tok.image_pad_id) == 3
    text = tok.decode(ids)
    assert text.startswith("<|im_start|>") and "pick the cube" in text and "<|vision_start|>" in text and "assistant" in text
    assert "<|im_start|>" not in tok.decode(ids, skip_special=True)
    assert tok.encode("pick the cube") == [vocab["pick"], vocab["the"], vocab["cube"]]
    assert isinstance(load_tokenizer("preset:tiny"), ByteTokenizer) and isinstance(load_tokenizer(str(tmp_path)), ByteTokenizer)
    bad = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    (tmp_path / "bad").mkdir()
    bad.save(str(tmp_path / "bad" / "tokenizer.json"))
    with pytest.raises(KeyError, match="im_start"):
        load_tokenizer(str(tmp_path / "bad"))

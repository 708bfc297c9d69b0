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


def test_family_vision_tower_equals_the_transformers_tower():
    """The family's vision tower with transformers' weights: same rows for pictures of two sizes (position table interpolation,
    row / column rotary, window-major patch order, merger), through the state dict as it is (same tensor names)."""
    from transformers import Qwen3_5Config, Qwen3_5VisionModel

    from pear_b200.models.vision import FamilyVisionConfig, FamilyVisionTower

    v = Qwen3_5Config().vision_config
    v.depth, v.hidden_size, v.intermediate_size, v.num_heads, v.out_hidden_size, v.num_position_embeddings, v.patch_size = 2, 64, 128, 4, 48, 64, 4
    torch.manual_seed(0)
    hf = Qwen3_5VisionModel(v).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            p.copy_(torch.randn_like(p) * (0.05 if p.dim() > 1 else 0.3) + (1.0 if p.dim() == 1 else 0.0))
    mine = FamilyVisionTower(FamilyVisionConfig.from_hf_dict(v.to_dict())).eval()
    missing, unexpected = mine.load_state_dict(hf.state_dict(), strict=True)
    assert not missing and not unexpected
    g = torch.Generator().manual_seed(1)
    pics = [torch.rand(3, 16, 24, generator=g) * 2 - 1, torch.rand(3, 32, 8, generator=g) * 2 - 1, torch.rand(3, 16, 24, generator=g) * 2 - 1]
    with torch.no_grad():
        got = mine(pics)
        for img, rows in zip(pics, got):
            vec, gh, gw = mine.patches(img)
            want = hf(vec, grid_thw=torch.tensor([[1, gh, gw]])).pooler_output
            assert rows.shape == want.shape == (mine.tokens_per_image(*img.shape[1:]), 48)
            assert float((rows - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max()))


def test_multimodal_checkpoint_with_a_picture_gives_the_same_logits(tmp_path):
    """A transformers conditional-generation model (text + vision) written out under its state-dict names: everything loads
    (``model.language_model.*`` into the decoder, ``model.visual.*`` into the family's tower, sizes from ``vision_config``), the
    (temporal, row, column) positions of a prompt with pictures equal transformers', and so do the logits."""
    import json

    from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration

    from pear_b200.models.hybrid import mrope_positions

    c = Qwen3_5Config()
    t, v = c.text_config, c.vision_config
    t.vocab_size, t.hidden_size, t.intermediate_size, t.num_hidden_layers, t.num_attention_heads, t.num_key_value_heads, t.head_dim = 512, 64, 128, 4, 4, 2, 32
    t.linear_key_head_dim = t.linear_value_head_dim = 16
    t.linear_num_key_heads, t.linear_num_value_heads = 2, 4
    t.layer_types = ["linear_attention"] * 3 + ["full_attention"]
    v.depth, v.hidden_size, v.intermediate_size, v.num_heads, v.out_hidden_size, v.num_position_embeddings, v.patch_size = 2, 64, 128, 4, 64, 64, 4
    c.image_token_id, c.vision_start_token_id, c.vision_end_token_id, c.video_token_id = 500, 501, 502, 503
    torch.manual_seed(0)
    hf = Qwen3_5ForConditionalGeneration(c).eval().float()
    d = tmp_path / "mm"
    d.mkdir()
    model_io.save_safetensors(str(d / "model.safetensors"), {k: p.contiguous() for k, p in hf.state_dict().items()})
    (d / "config.json").write_text(json.dumps(c.to_dict(), default=str))
    cfg, vcfg = model_io.load_config(str(d)), model_io.load_vision_config(str(d))
    mine = HybridForCausalLM(cfg, with_mtp=False, vision=vcfg)
    assert model_io.load_model_dir(str(d), mine, ignore_unexpected=()) == ([], [])
    g = torch.Generator().manual_seed(1)
    pics = [torch.rand(3, 16, 24, generator=g) * 2 - 1, torch.rand(3, 24, 8, generator=g) * 2 - 1]
    grids, vecs = [], []
    for img in pics:
        vec, gh, gw = mine.visual.patches(img)
        grids.append((gh, gw))
        vecs.append(vec)
    text = lambda n: torch.randint(0, 400, (n,), generator=g)  # noqa: E731
    run = lambda k: torch.tensor([501] + [500] * (grids[k][0] * grids[k][1] // 4) + [502])  # noqa: E731
    ids = torch.cat([text(7), run(0), text(5), run(1), text(9)])
    mm = (ids == 500).int()[None]
    thw = torch.tensor([[1, gh, gw] for gh, gw in grids])
    with torch.no_grad():
        want = hf(input_ids=ids[None], pixel_values=torch.cat(vecs), image_grid_thw=thw, mm_token_type_ids=mm).logits[0]
        want_pos, _ = hf.model.get_rope_index(ids[None], mm, image_grid_thw=thw)
        pos = mrope_positions(ids, grids, image_pad_id=500)
        assert torch.equal(pos, want_pos[:, 0])
        rows = torch.cat(mine.visual(pics))
        mask = ids == 500
        emb = torch.zeros(len(ids), cfg.hidden_size)
        emb[mask] = rows
        got = mine.logits(mine(ids, pos, [0, len(ids)], inputs_embeds=emb, embeds_mask=mask))
    assert float((got - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.timeout(600)
def test_training_entry_starts_from_a_multimodal_checkpoint_directory(tmp_path):
    """``model.path`` = a conditional-generation checkpoint, ``vision.preset=checkpoint``: decoder and tower start from the
    directory's tensors, the pixel environment's pictures go through that tower in the agent loop and in the trainer, a step
    trains both."""
    import json

    import numpy as np
    from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration

    from pear_b200.config.loader import compose
    from pear_b200.train.main import RunConfig, build_stack

    c = Qwen3_5Config()
    t, v = c.text_config, c.vision_config
    t.vocab_size, t.hidden_size, t.intermediate_size, t.num_hidden_layers, t.num_attention_heads, t.num_key_value_heads, t.head_dim = 512, 64, 128, 4, 4, 2, 32
    t.linear_key_head_dim = t.linear_value_head_dim = 16
    t.linear_num_key_heads, t.linear_num_value_heads = 2, 4
    t.layer_types = ["linear_attention"] * 3 + ["full_attention"]
    v.depth, v.hidden_size, v.intermediate_size, v.num_heads, v.out_hidden_size, v.num_position_embeddings, v.patch_size = 2, 64, 128, 4, 64, 64, 4
    torch.manual_seed(0)
    hf = Qwen3_5ForConditionalGeneration(c).eval().float()
    d = tmp_path / "mm"
    d.mkdir()
    model_io.save_safetensors(str(d / "model.safetensors"), {k: p.contiguous() for k, p in hf.state_dict().items()})
    (d / "config.json").write_text(json.dumps(c.to_dict(), default=str))
    cfg = RunConfig(compose("training", [f"run_dir={tmp_path / 'run'}", f"actor_rollout_ref.model.path={d}", "data.train_batch_size=3", "actor_rollout_ref.rollout.n=4",
                                         "data.max_response_length=16", "actor_rollout_ref.rollout.max_model_len=2048", "actor_rollout_ref.rollout.max_num_seqs=8",
                                         "actor_rollout_ref.rollout.agent.num_workers=2", "actor_rollout_ref.rollout.topk_log_probs=4", "algorithm.filter_groups.enable=false",
                                         "trainer.total_training_steps=1", "trainer.save_freq=0", "transfer_queue.num_data_storage_units=4",
                                         "actor_rollout_ref.actor.optim.lr=1e-3", "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=4096", "trainer.logger=[file]",
                                         "actor_rollout_ref.model.vision.enable=true", "actor_rollout_ref.model.vision.preset=checkpoint",
                                         "actor_rollout_ref.model.vision.train=true", "actor_rollout_ref.rollout.multi_turn.synthetic_turns=1",
                                         "actor_rollout_ref.rollout.multi_turn.synthetic_reward=hash"])).prepare()
    fam = {"synthetic": {"env_path": "pear_b200.envs.synthetic.SyntheticEnv", "num_processes": 1, "env_kwargs": {"pixels": 16}}}
    trainer, close = build_stack(cfg, env_families=fam)
    try:
        start = trainer.engine.full_state_dict()
        sd = hf.state_dict()
        assert torch.equal(start["visual.blocks.0.attn.qkv.weight"], sd["model.visual.blocks.0.attn.qkv.weight"])
        assert torch.equal(start["model.layers.3.self_attn.q_proj.weight"], sd["model.language_model.layers.3.self_attn.q_proj.weight"])
        hist = trainer.fit()
        after = trainer.engine.full_state_dict()
        assert np.isfinite(hist[0]["actor/grad_norm"]) and hist[0]["actor/grad_norm"] > 0
        assert not torch.equal(after["visual.blocks.0.attn.qkv.weight"], start["visual.blocks.0.attn.qkv.weight"])
    finally:
        close()


def _picture_case(tmp_path, with_mtp: bool = False):
    """A small multi-modal transformers model saved as a checkpoint directory, this framework's model loaded from it, and one
    prompt with a picture: (hf, mine, cfg, ids, mask, emb, vec, gh, gw)."""
    import json

    from transformers import Qwen3_5Config, Qwen3_5ForConditionalGeneration

    from pear_b200.models.config import HybridConfig

    c = Qwen3_5Config()
    t, v = c.text_config, c.vision_config
    t.vocab_size, t.hidden_size, t.intermediate_size, t.num_hidden_layers, t.num_attention_heads, t.num_key_value_heads, t.head_dim = 512, 64, 128, 4, 4, 2, 32
    t.linear_key_head_dim = t.linear_value_head_dim = 16
    t.linear_num_key_heads, t.linear_num_value_heads = 2, 4
    t.layer_types = ["linear_attention"] * 3 + ["full_attention"]
    v.depth, v.hidden_size, v.intermediate_size, v.num_heads, v.out_hidden_size, v.num_position_embeddings, v.patch_size = 2, 64, 128, 4, 64, 64, 4
    c.image_token_id, c.vision_start_token_id, c.vision_end_token_id, c.video_token_id = 500, 501, 502, 503
    torch.manual_seed(3)
    hf = Qwen3_5ForConditionalGeneration(c).eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            if p.dim() > 1:
                p.mul_(3.0)
    d = tmp_path / "mm"
    d.mkdir()
    model_io.save_safetensors(str(d / "model.safetensors"), {k: p.contiguous() for k, p in hf.state_dict().items()})
    (d / "config.json").write_text(json.dumps(c.to_dict(), default=str))
    cfg, vcfg = model_io.load_config(str(d)), model_io.load_vision_config(str(d))
    if with_mtp:  # the checkpoint has no drafter: a random one proposes, the main model verifies
        cfg = HybridConfig.from_dict({**cfg.to_dict(), "num_mtp_layers": 1})
        mine = HybridForCausalLM(cfg, with_mtp=True, vision=vcfg).init_weights(11)
        model_io.load_model_dir(str(d), mine, allow_missing=("mtp.",), ignore_unexpected=())
    else:
        mine = HybridForCausalLM(cfg, with_mtp=False, vision=vcfg)
        model_io.load_model_dir(str(d), mine, ignore_unexpected=())
    g = torch.Generator().manual_seed(1)
    img = torch.rand(3, 16, 24, generator=g) * 2 - 1
    vec, gh, gw = mine.visual.patches(img)
    ids = torch.cat([torch.randint(0, 400, (6,), generator=g), torch.tensor([501] + [500] * (gh * gw // 4) + [502]), torch.randint(0, 400, (8,), generator=g)])
    mask = ids == 500
    with torch.no_grad():
        emb = torch.zeros(len(ids), cfg.hidden_size)
        emb[mask] = mine.visual([img])[0]
    return hf, mine, cfg, ids, mask, emb, vec, gh, gw


def test_rollout_engine_with_pictures_and_checkpoint_positions_equals_generate(tmp_path):
    """A prompt with a picture through the rollout engine (rows at the placeholders, the checkpoint's (t, h, w) positions, decode
    positions continuing past the picture) gives transformers' greedy continuation of the same multi-modal input."""
    from pear_b200.models.hybrid import mrope_positions
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    hf, mine, cfg, ids, mask, emb, vec, gh, gw = _picture_case(tmp_path)
    with torch.no_grad():
        want = hf.generate(input_ids=ids[None], pixel_values=vec, image_grid_thw=torch.tensor([[1, gh, gw]]), mm_token_type_ids=mask.int()[None],
                           max_new_tokens=8, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    eng = RolloutEngine(mine, EngineConfig(num_blocks=64, max_num_seqs=2, max_num_batched_tokens=16))  # (prefill in chunks: positions per chunk)
    req = eng.add_request(ids.tolist(), SamplingParams(max_tokens=8, temperature=0.0), embeds=emb, embeds_mask=mask,
                          position_ids=mrope_positions(ids, [(gh, gw)], image_pad_id=500))
    while eng.has_work():
        eng.step()
    assert req.output == want
    plain = eng.add_request(ids.tolist(), SamplingParams(max_tokens=8, temperature=0.0), embeds=emb, embeds_mask=mask)  # sequential positions: another model input
    while eng.has_work():
        eng.step()
    assert len(plain.output) == 8


def test_speculative_decoding_of_a_picture_prompt_with_checkpoint_positions_equals_generate(tmp_path):
    """The drafter runs at the request's own positions too: a picture prompt under the checkpoint's position rule, three drafts a
    step from a (random) MTP module, still continues as transformers' ``generate`` does."""
    from pear_b200.models.hybrid import mrope_positions
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    hf, mine, cfg, ids, mask, emb, vec, gh, gw = _picture_case(tmp_path, with_mtp=True)
    with torch.no_grad():
        want = hf.generate(input_ids=ids[None], pixel_values=vec, image_grid_thw=torch.tensor([[1, gh, gw]]), mm_token_type_ids=mask.int()[None],
                           max_new_tokens=12, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    eng = RolloutEngine(mine, EngineConfig(num_blocks=64, max_num_seqs=2, max_num_batched_tokens=16, num_speculative_tokens=3))
    req = eng.add_request(ids.tolist(), SamplingParams(max_tokens=12, temperature=0.0), embeds=emb, embeds_mask=mask,
                          position_ids=mrope_positions(ids, [(gh, gw)], image_pad_id=500))
    while eng.has_work():
        eng.step()
    assert req.output == want and eng.metrics["spec_drafted"] > 0


def test_speculative_decoding_and_a_cached_second_turn_stay_equal_to_generate(tmp_path):
    """Lossless by construction, checked against the outside implementation: with a (random) MTP drafter proposing three tokens a
    step the greedy continuation is still transformers'; a second turn that resumes from the prefix cache (KV pages and the
    recurrent-state snapshot of the first turn) continues as ``generate`` does on the whole conversation."""
    from pear_b200.models.config import HybridConfig
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    hf = _hf_model(6)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    base = model_io.load_config(str(tmp_path / "hf"))
    cfg = HybridConfig.from_dict({**base.to_dict(), "num_mtp_layers": 1})
    mine = HybridForCausalLM(cfg, with_mtp=True).init_weights(11)  # the drafter keeps these random weights
    model_io.load_model_dir(str(tmp_path / "hf"), mine, allow_missing=("mtp.",))
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 512, (37,), generator=g).tolist()
    eng = RolloutEngine(mine, EngineConfig(num_blocks=64, max_num_seqs=2, num_speculative_tokens=3))
    first = eng.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0), sessions=["s"])[0]
    with torch.no_grad():
        want1 = hf.generate(torch.tensor([prompt]), max_new_tokens=12, do_sample=False, pad_token_id=0)[0, len(prompt):].tolist()
    assert first.output == want1 and eng.metrics["spec_drafted"] > 0
    turn2 = prompt + first.output + torch.randint(0, 512, (9,), generator=g).tolist()
    second = eng.generate([turn2], SamplingParams(max_tokens=10, temperature=0.0), sessions=["s"])[0]
    with torch.no_grad():
        want2 = hf.generate(torch.tensor([turn2]), max_new_tokens=10, do_sample=False, pad_token_id=0)[0, len(turn2):].tolist()
    assert second.cached_prefix >= 16 and second.output == want2


def test_picture_patches_and_sizes_equal_the_family_image_processor():
    """What reaches the tower: the window-major patch rows of a picture equal the family's image processor's ``pixel_values`` (same
    normalisation, same order), and the resize rule picks the processor's sizes."""
    import numpy as np
    from transformers import Qwen2VLImageProcessor

    from pear_b200.eval.general import picture_size
    from pear_b200.models.vision import FamilyVisionConfig, FamilyVisionTower

    tower = FamilyVisionTower(FamilyVisionConfig.tiny())  # patch 4, merge 2, temporal patch 2
    rng = np.random.default_rng(0)
    arr = rng.integers(0, 256, (16, 24, 3), dtype=np.uint8)
    proc = Qwen2VLImageProcessor(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=64, max_pixels=4096, image_mean=[0.5] * 3, image_std=[0.5] * 3, do_resize=False)
    out = proc(images=[arr], return_tensors="pt")
    vec, gh, gw = tower.patches(torch.from_numpy(arr).permute(2, 0, 1).float() / 127.5 - 1.0)
    assert out["image_grid_thw"].tolist() == [[1, gh, gw]] and float((vec - out["pixel_values"]).abs().max()) < 1e-6
    resizing = Qwen2VLImageProcessor(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=256, max_pixels=2048, image_mean=[0.5] * 3, image_std=[0.5] * 3)
    for h, w in ((37, 50), (9, 11), (100, 70), (16, 16), (64, 200)):
        grid = resizing(images=[rng.integers(0, 256, (h, w, 3), dtype=np.uint8)], return_tensors="pt")["image_grid_thw"][0].tolist()
        assert picture_size(h, w, 8, 256, 2048) == (grid[1] * 4, grid[2] * 4), (h, w, grid)


def _tp_rank_fn(rank, world, hf_dir, out_dir):
    import torch.distributed as dist

    from pear_b200.models import hybrid
    from pear_b200.parallel.tensor_parallel import shard_state, tp_config
    from pear_b200.rollout.engine import EngineConfig, RolloutEngine, SamplingParams

    cfg = model_io.load_config(hf_dir)
    full = HybridForCausalLM(cfg, with_mtp=False)
    model_io.load_model_dir(hf_dir, full)
    tp = HybridForCausalLM(tp_config(cfg, world), with_mtp=False)
    tp.load_state_dict(shard_state(full.state_dict(), cfg, rank, world), strict=True)
    hybrid.set_tensor_parallel_group(dist.group.WORLD)
    try:
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 33)]
        outs = RolloutEngine(tp, EngineConfig(num_blocks=64, max_num_seqs=4)).generate(prompts, SamplingParams(max_tokens=10, temperature=0.0))
    finally:
        hybrid.set_tensor_parallel_group(None)
    if rank == 0:
        torch.save({"prompts": prompts, "outputs": [r.output for r in outs]}, out_dir + "/tp.pt")


def test_tensor_parallel_shards_of_a_transformers_checkpoint_generate_the_same(tmp_path):
    """The sharding rules on the family's real tensor layouts (per-head [q | gate] rows of q_proj, the q | k | v sections of the
    linear-attention projection and its convolution, vocabulary-parallel head): two ranks with half of every projection each
    continue as transformers does with the whole model."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_ranks

    hf = _hf_model(4)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    run_ranks(_tp_rank_fn, 2, tmp_path, str(tmp_path / "hf"), str(tmp_path))
    got = torch.load(str(tmp_path / "tp.pt"))
    for p, out in zip(got["prompts"], got["outputs"]):
        with torch.no_grad():
            want = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, pad_token_id=0)[0, len(p):].tolist()
        assert out == want


def test_trainer_step_on_a_transformers_checkpoint_equals_autograd_and_adamw_on_the_transformers_model(tmp_path):
    """The training engine (packed sequences, sharded flat parameters, recomputed layers, chunked log-prob head, token-mean REINFORCE,
    gradient clipping, its own AdamW) takes the step that plain autograd and ``torch.optim.AdamW`` take on the ``transformers`` model
    with the loss written out by hand, sequence by sequence."""
    from pear_b200.train.engine import EngineConfig, PackedBatch, TrainEngine
    from pear_b200.train.grpo import LossConfig

    hf = _hf_model(4)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    cfg = model_io.load_config(str(tmp_path / "hf"))
    mine = HybridForCausalLM(cfg, with_mtp=False)
    model_io.load_model_dir(str(tmp_path / "hf"), mine)
    ecfg = EngineConfig(lr=1e-3, eps=1e-6, clip_grad=0.5, weight_decay=0.01, param_dtype="fp32", enable_gradient_checkpointing=True, temperature=0.8,
                        loss=LossConfig(score_centering=False))
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 512, (n,), generator=g) for n in (45, 30, 19)]
    advs = [float(torch.randn((), generator=g)) for _ in seqs]
    masks = []
    for s in seqs:
        m = torch.zeros(len(s))
        m[len(s) // 3 : len(s) - 1] = 1  # the generated part; the last token has no successor
        masks.append(m)

    def batch(idx):
        cu = [0]
        for i in idx:
            cu.append(cu[-1] + len(seqs[i]))
        return PackedBatch(torch.cat([seqs[i] for i in idx]), torch.cat([torch.arange(len(seqs[i])) for i in idx]), cu,
                           torch.cat([torch.cat([seqs[i][1:], seqs[i][:1]]) for i in idx]), torch.cat([masks[i] for i in idx]),
                           torch.cat([torch.full((len(seqs[i]),), advs[i]) for i in idx]))

    eng = TrainEngine(cfg, ecfg, seed=0, state_dict=mine.state_dict())
    eng.forward_backward_batch([batch([0, 1]), batch([2])])  # two micro-batches of one step
    stats = eng.optimizer_step()

    hf.train()
    opt = torch.optim.AdamW(hf.parameters(), lr=ecfg.lr, betas=ecfg.betas, eps=ecfg.eps, weight_decay=ecfg.weight_decay, foreach=False, fused=False)
    denom = sum(float(m.sum()) for m in masks)
    for s, a, m in zip(seqs, advs, masks):
        lp = torch.log_softmax(hf(s[None]).logits[0, :-1].float() / ecfg.temperature, -1).gather(1, s[1:, None])[:, 0]
        (-(a * lp * m[:-1]).sum() / denom).backward()
    norm = float(torch.nn.utils.clip_grad_norm_(hf.parameters(), ecfg.clip_grad))
    opt.step()
    assert abs(stats["actor/grad_norm"] - norm) < 1e-4 * max(1.0, norm)
    hf.save_pretrained(str(tmp_path / "hf_after"), safe_serialization=True)
    after = HybridForCausalLM(cfg, with_mtp=False)
    model_io.load_model_dir(str(tmp_path / "hf_after"), after)
    got, before = eng.full_state_dict(), mine.state_dict()
    moved = 0.0
    for k, v in after.state_dict().items():
        assert torch.allclose(got[k], v, atol=2e-5, rtol=1e-4), k
        moved = max(moved, float((v - before[k]).abs().max()))
    assert moved > 1e-4  # (the step changed something: equal-because-nothing-moved would pass the loop above)

"""Shared helpers of the megakernel tests: a small model of kernel-legal shapes whose weights are exactly NVFP4
representable, and the fp32 torch oracle of a speculative decode step."""

from __future__ import annotations

import torch

from pear_b200.models import nvfp4
from pear_b200.models.config import HybridConfig
from pear_b200.models.drafter import BlockDrafter
from pear_b200.models.hybrid import DenseCache, HybridForCausalLM, forward_cached


def small_configs():
    cfg = HybridConfig(vocab_size=2048, hidden_size=512, num_layers=3, full_attention_interval=3, num_attention_heads=4,
                       num_kv_heads=2, head_dim=256, rotary_dim=64, gdn_qk_heads=2, gdn_v_heads=4, gdn_head_dim=128,
                       intermediate_size=1024, num_mtp_layers=0, init_std=0.05)
    dcfg = HybridConfig(vocab_size=2048, hidden_size=512, num_layers=2, full_attention_interval=1, num_attention_heads=4,
                        num_kv_heads=2, head_dim=128, rotary_dim=64, intermediate_size=1024, num_mtp_layers=0,
                        attn_output_gate=False, init_std=0.05)
    return cfg, dcfg


def _requantize_(mats: list[torch.nn.Parameter]) -> None:
    """Replace a group of matrices (quantised as one row-concatenated matrix) by their NVFP4 dequantisation."""
    with torch.no_grad():
        cat = torch.cat([m.reshape(m.shape[0], -1) for m in mats], dim=0)
        deq = nvfp4.quantize(cat).dequantize()
        o = 0
        for m in mats:
            m.copy_(deq[o : o + m.shape[0]].reshape(m.shape))
            o += m.shape[0]


def build_models(seed: int = 0):
    cfg, dcfg = small_configs()
    model = HybridForCausalLM(cfg, with_mtp=False).init_weights(seed)
    drafter = BlockDrafter(dcfg).init_weights(seed + 1)
    with torch.no_grad():
        for m in (model, drafter):
            for n, p in m.named_parameters():  # non-trivial norm weights so the norms are really exercised
                if p.dim() == 1 and "A_log" not in n and "dt_bias" not in n:
                    p.add_(torch.randn_like(p) * 0.1)
        model.model.embed_tokens.weight.copy_(model.model.embed_tokens.weight.bfloat16().float())
    for layer in list(model.model.layers) + list(drafter.layers):
        if layer.layer_type == "linear_attention":
            g = layer.linear_attn
            _requantize_([g.in_proj_qkv.weight, g.in_proj_z.weight, g.in_proj_b.weight, g.in_proj_a.weight])
            _requantize_([g.out_proj.weight])
        else:
            a = layer.self_attn
            _requantize_([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight])
            _requantize_([a.o_proj.weight])
        _requantize_([layer.mlp.gate_proj.weight, layer.mlp.up_proj.weight])
        _requantize_([layer.mlp.down_proj.weight])
    _requantize_([model.lm_head.weight])
    _requantize_([drafter.fc.weight])
    return model.eval(), drafter.eval()


@torch.no_grad()
def oracle_logits(model: HybridForCausalLM, tokens: list[int]):
    """Logits [len, V] and pre-norm residuals [len, H] of the whole sequence (fp32, CPU)."""
    cache = DenseCache(model.config)
    h, r = forward_cached(model, torch.tensor(tokens), cache, return_prenorm=True)
    return model.logits(h), r


@torch.no_grad()
def oracle_draft_logits(model, drafter, residuals: torch.Tensor, next_tokens: list[int], n_committed_rows_before: int,
                        draft_cache: DenseCache, n_mask: int):
    """Drafter pass over committed rows (residual_j, token_{j+1}) then ``n_mask`` mask rows reading the last committed
    residual. ``draft_cache`` holds the drafter KV of earlier committed rows and is extended by the committed rows only.
    Returns logits of all rows [rows + n_mask, V]."""
    emb = model.model.embed_tokens(torch.tensor(next_tokens)).float()
    x = drafter.project(emb, residuals)
    pos = torch.arange(n_committed_rows_before, n_committed_rows_before + x.shape[0])
    draft_cache.length = n_committed_rows_before
    r = forward_cached(drafter_as_model(model, drafter), torch.zeros(x.shape[0], dtype=torch.long), draft_cache, position_ids=pos,
                       layers=drafter.layers, embeds=x)
    outs = [r]
    if n_mask:
        tmp = draft_cache.clone()
        memb = model.model.embed_tokens(torch.full((n_mask,), drafter.mask_token_id)).float()
        xm = drafter.project(memb, residuals[-1:].expand(n_mask, -1))
        posm = torch.arange(n_committed_rows_before + x.shape[0], n_committed_rows_before + x.shape[0] + n_mask)
        rm = forward_cached(drafter_as_model(model, drafter), torch.zeros(n_mask, dtype=torch.long), tmp, position_ids=posm,
                            layers=drafter.layers, embeds=xm)
        outs.append(rm)
    r_all = torch.cat(outs, dim=0)
    return model.logits(drafter.norm(r_all))


class drafter_as_model:
    """Adapter giving :func:`forward_cached` the attributes it reads (config, rope) for the drafter's layers."""

    def __init__(self, model, drafter):
        self.config = drafter.config
        self._model = model
        self._drafter = drafter

    def rope(self, position_ids):
        from pear_b200.ops import reference as ref

        c = self.config
        return ref.mrope_cos_sin(position_ids, c.rotary_dim, c.rope_theta, c.mrope_sections)

"""Hybrid Gated-DeltaNet + gated-attention decoder with an MTP head.

Parameter names follow the HF checkpoint layout of the family so a state dict is a safetensors model directory as is
(``model.layers.N.linear_attn.in_proj_qkv.weight``, ``model.layers.N.self_attn.q_proj.weight``, ``mtp.fc.weight`` ...).

The layer recipe is the upstream trainer's (``pear/models/qwen3_5/trainer/rms_norm.py:363-423``): an fp32 residual
stream ``r``; ``h = norm(r)``; ``r += mixer(h)``; ``y = norm(r)``; ``r += mlp(y)``. Linear layers take their input in
the weight's dtype and return fp32. The same module is the CPU oracle (fp32 weights) and the GPU training model (bf16
weights, ops routed to the sm_100a kernels by :mod:`pear_b200.ops.api`).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import api as ops
from .config import HybridConfig


def linear_fp32(x: torch.Tensor, weight: torch.Tensor, output_unused: bool = False) -> torch.Tensor:
    """``x @ weight^T`` with the operands in the weight's dtype and an fp32 result."""
    return ops.linear(x, weight, output_unused)


# Set by the layer runner around the recompute pass of a checkpointed layer: the value of the layer's LAST GEMM (the MLP's
# down projection) is never read there (only its backward runs), so its forward is skipped (upstream trainer/mlp.py:132-134).
RECOMPUTE: dict = {"skip_down_proj": False}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, one_plus: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(dim) if one_plus else torch.ones(dim))
        self.eps, self.one_plus = eps, one_plus

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps, self.one_plus)


_TP: dict = {"group": None, "fused": None, "defer": False}
FRONT_KERNEL: dict = {"on": True}  # GDN front end of the training forward through the fused kernel pair on a GPU


def set_tensor_parallel_group(group) -> None:
    """Tensor-parallel mode: the modules hold 1 / world of the heads and of the FFN width
    (``pear_b200/parallel/tensor_parallel.py`` shards the weights); the outputs of the row-parallel projections
    (o_proj, out_proj, down_proj) are partial sums that ``row_linear`` all-reduces over this group."""
    _TP["group"] = group
    if group is None:
        _TP["fused"] = None


def set_tensor_parallel_fused(symm_world, max_rows: int, hidden: int) -> None:
    """Route the reductions that are followed by a residual add and an RMSNorm (every one inside the rollout step)
    through the NVSwitch kernel ``SymmWorld.all_reduce_add_rmsnorm`` instead of an NCCL all-reduce plus a norm kernel
    (upstream ``rollout/blackwell/csrc/ar_norm.cu``). Steps with more than ``max_rows`` rows keep the NCCL path."""
    _TP["fused"] = (symm_world, symm_world.make_ar_workspace(max_rows, hidden), max_rows)


def tensor_parallel_active() -> bool:
    return _TP["group"] is not None


class defer_row_reduce:
    """Inside this context ``row_linear`` returns the rank's partial sum; the caller reduces it with
    ``reduce_add_rms_norm`` / ``reduce_partial``."""

    def __enter__(self):
        self.prev, _TP["defer"] = _TP["defer"], True

    def __exit__(self, *exc):
        _TP["defer"] = self.prev


def reduce_partial(y: torch.Tensor) -> torch.Tensor:
    g = _TP["group"]
    if g is not None:
        import torch.distributed as dist

        dist.all_reduce(y, group=g)
    return y


def reduce_add_rms_norm(partial: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """``residual + sum over ranks(partial)`` and its (1 + w) RMSNorm: returns (normed, new residual), both fp32."""
    fused = _TP["fused"]
    if fused is not None and partial.is_cuda and partial.shape[0] <= fused[2] and residual.dtype == torch.float32 and residual.is_contiguous():
        symm, ws, _ = fused
        y = symm.all_reduce_add_rmsnorm(ws, partial.to(torch.bfloat16), residual, weight.detach().float(), eps)  # residual in place
        return y.float(), residual
    return ops.add_rms_norm(reduce_partial(partial), residual, weight, eps)


def row_linear(x: torch.Tensor, weight: torch.Tensor, output_unused: bool = False) -> torch.Tensor:
    y = linear_fp32(x, weight, output_unused)
    return y if _TP["defer"] else reduce_partial(y)


class SwiGLUMLP(nn.Module):
    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        act = ops.swiglu(linear_fp32(y, self.gate_proj.weight), linear_fp32(y, self.up_proj.weight))
        return row_linear(act, self.down_proj.weight, output_unused=RECOMPUTE["skip_down_proj"] and torch.is_grad_enabled())


@dataclass
class SeqMeta:
    """What a packed micro-batch carries besides tokens. ``cu_seqlens`` are GLOBAL boundaries; under sequence
    parallelism a rank holds tokens [offset, offset + T_local) of the packed stream."""

    cu_seqlens: list[int]
    cos: torch.Tensor
    sin: torch.Tensor
    sp: Optional[object] = None  # parallel.ulysses.SequenceParallel, None on one rank
    offset: int = 0
    extras: dict = field(default_factory=dict)

    def local_bounds(self, t_local: int) -> list[int]:
        """Sequence boundaries clipped to this rank's slice, relative to its first token."""
        lo, hi = self.offset, self.offset + t_local
        cuts = sorted({min(max(c, lo), hi) - lo for c in self.cu_seqlens} | {0, t_local})
        return cuts


class GatedAttention(nn.Module):
    """``q_proj`` yields per head ``[q | gate]``; per-head (1+w) RMSNorm on q and k; interleaved M-RoPE on the first
    ``rotary_dim`` channels; causal GQA attention; ``o_proj(attn * sigmoid(gate))``."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.cfg = cfg
        h = cfg.hidden_size
        self.gated = cfg.attn_output_gate
        self.q_proj = nn.Linear(h, (2 if self.gated else 1) * cfg.q_size, bias=False)
        self.k_proj = nn.Linear(h, cfg.kv_size, bias=False)
        self.v_proj = nn.Linear(h, cfg.kv_size, bias=False)
        self.o_proj = nn.Linear(cfg.q_size, h, bias=False)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_eps)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_eps)

    def project(self, hidden: torch.Tensor, meta: SeqMeta):
        cfg = self.cfg
        t = hidden.shape[0]
        if self.gated:
            qg = linear_fp32(hidden, self.q_proj.weight).view(t, cfg.num_attention_heads, 2 * cfg.head_dim)
            q, gate = qg[..., : cfg.head_dim], qg[..., cfg.head_dim :]
        else:
            q, gate = linear_fp32(hidden, self.q_proj.weight).view(t, cfg.num_attention_heads, cfg.head_dim), None
        k = linear_fp32(hidden, self.k_proj.weight).view(t, cfg.num_kv_heads, cfg.head_dim)
        v = linear_fp32(hidden, self.v_proj.weight).view(t, cfg.num_kv_heads, cfg.head_dim)
        q = ops.apply_rope(self.q_norm(q), meta.cos, meta.sin)
        k = ops.apply_rope(self.k_norm(k), meta.cos, meta.sin)
        return q, k, v, gate

    def forward(self, hidden: torch.Tensor, meta: SeqMeta) -> torch.Tensor:
        cfg = self.cfg
        t = hidden.shape[0]
        q, k, v, gate = self.project(hidden, meta)
        if meta.sp is not None and meta.sp.size > 1:
            attn = meta.sp.attention(q, k, v, meta.cu_seqlens, cfg.head_dim ** -0.5)
        else:
            attn = ops.causal_attention(q, k, v, meta.cu_seqlens, cfg.head_dim ** -0.5)
        gated = (ops.sigmoid_gate(attn, gate) if gate is not None else attn).reshape(t, cfg.q_size)
        return row_linear(gated, self.o_proj.weight)


class GatedDeltaNet(nn.Module):
    """Gated DeltaNet mixer (upstream ``pear/models/qwen3_5/trainer/gdn.py:550-651``)."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.cfg = cfg
        h, c = cfg.hidden_size, cfg.gdn_conv_dim
        self.in_proj_qkv = nn.Linear(h, c, bias=False)
        self.in_proj_z = nn.Linear(h, cfg.gdn_value_dim, bias=False)
        self.in_proj_b = nn.Linear(h, cfg.gdn_v_heads, bias=False)
        self.in_proj_a = nn.Linear(h, cfg.gdn_v_heads, bias=False)
        self.conv1d = nn.Conv1d(c, c, cfg.conv_kernel, groups=c, bias=False)
        self.A_log = nn.Parameter(torch.zeros(cfg.gdn_v_heads))
        self.dt_bias = nn.Parameter(torch.zeros(cfg.gdn_v_heads))
        self.norm = RMSNorm(cfg.gdn_head_dim, cfg.rms_eps, one_plus=False)
        self.out_proj = nn.Linear(cfg.gdn_value_dim, h, bias=False)

    def conv_weight(self) -> torch.Tensor:
        return self.conv1d.weight.view(self.cfg.gdn_conv_dim, self.cfg.conv_kernel)

    def front(self, mixed: torch.Tensor, bounds: list[int], init_conv: Optional[torch.Tensor], need_conv_state: bool = True):
        """conv + SiLU + split + L2 norms. Returns q [T,Hk,K], k, v [T,Hv,V] and the final conv rows."""
        cfg = self.cfg
        t = mixed.shape[0]
        if (not need_conv_state and mixed.is_cuda and init_conv is None and mixed.dtype == torch.float32 and cfg.gdn_head_dim == 128 and cfg.conv_kernel == 4
                and FRONT_KERNEL["on"]):
            # one kernel forward (conv + SiLU + both L2 norms), two backward; the final conv rows are the last raw rows
            from ..ops import rollout_ops

            u = rollout_ops.gdn_front_autograd(mixed, self.conv_weight(), bounds, 2 * cfg.gdn_key_dim, cfg.l2_eps)
            kd = cfg.gdn_key_dim
            q = u[:, :kd].reshape(t, cfg.gdn_qk_heads, cfg.gdn_head_dim)
            k = u[:, kd : 2 * kd].reshape(t, cfg.gdn_qk_heads, cfg.gdn_head_dim)
            v = u[:, 2 * kd :].reshape(t, cfg.gdn_v_heads, cfg.gdn_head_dim)
            return q, k, v, None
        u, conv_final = ops.causal_conv_silu(mixed, self.conv_weight(), bounds, init_conv)
        kd = cfg.gdn_key_dim
        q = u[:, :kd].reshape(t, cfg.gdn_qk_heads, cfg.gdn_head_dim)
        k = u[:, kd : 2 * kd].reshape(t, cfg.gdn_qk_heads, cfg.gdn_head_dim)
        v = u[:, 2 * kd :].reshape(t, cfg.gdn_v_heads, cfg.gdn_head_dim)
        q = ops.l2norm(q, cfg.l2_eps) * (cfg.gdn_head_dim ** -0.5)
        k = ops.l2norm(k, cfg.l2_eps)
        return q, k, v, conv_final

    def forward(self, hidden: torch.Tensor, meta: SeqMeta) -> torch.Tensor:
        cfg = self.cfg
        t = hidden.shape[0]
        mixed = linear_fp32(hidden, self.in_proj_qkv.weight)
        sp_on = meta.sp is not None and meta.sp.size > 1
        halo = meta.sp.start_conv_halo(mixed, cfg.conv_kernel) if sp_on else None  # in flight under the three projections below
        z = linear_fp32(hidden, self.in_proj_z.weight).view(t, cfg.gdn_v_heads, cfg.gdn_head_dim)
        b = linear_fp32(hidden, self.in_proj_b.weight)
        a = linear_fp32(hidden, self.in_proj_a.weight)
        g, beta = ops.gdn_gates(a, b, self.A_log, self.dt_bias)
        bounds = meta.local_bounds(t)
        if sp_on:
            o = meta.sp.gdn(self, mixed, g, beta, meta, bounds, halo=halo)
        else:
            q, k, v, _ = self.front(mixed, bounds, None, need_conv_state=False)
            o = ops.gdn_scan_packed(q, k, v, g, beta, bounds)
        y = ops.gated_rms_norm(o, z, self.norm.weight, cfg.rms_eps).reshape(t, cfg.gdn_value_dim)
        return row_linear(y, self.out_proj.weight)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: HybridConfig, layer_type: str):
        super().__init__()
        self.layer_type = layer_type
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        if layer_type == "full_attention":
            self.self_attn = GatedAttention(cfg)
        else:
            self.linear_attn = GatedDeltaNet(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.mlp = SwiGLUMLP(cfg)

    @property
    def mixer(self) -> nn.Module:
        return self.self_attn if self.layer_type == "full_attention" else self.linear_attn

    def forward(self, residual: torch.Tensor, meta: SeqMeta) -> torch.Tensor:
        h = self.input_layernorm(residual)
        mixed = self.mixer(h, meta)
        y, residual = ops.add_rms_norm(mixed, residual, self.post_attention_layernorm.weight,
                                       self.post_attention_layernorm.eps)
        return residual + self.mlp(y)


class Backbone(nn.Module):
    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(cfg, t) for t in cfg.layer_types])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)


class MTPHead(nn.Module):
    """``x = fc([norm_e(embed(tok_{t+1})) | norm_h(hidden_t)])`` then one full-attention decoder layer and a final
    norm; logits come from the shared ``lm_head`` (upstream ``rollout/blackwell/mtp.py:191-234``)."""

    def __init__(self, cfg: HybridConfig):
        super().__init__()
        self.pre_fc_norm_embedding = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.pre_fc_norm_hidden = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.fc = nn.Linear(2 * cfg.hidden_size, cfg.hidden_size, bias=False)
        self.layers = nn.ModuleList([DecoderLayer(cfg, "full_attention") for _ in range(cfg.num_mtp_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)

    def forward(self, next_embeds: torch.Tensor, hidden: torch.Tensor, meta: SeqMeta) -> torch.Tensor:
        x = torch.cat([self.pre_fc_norm_embedding(next_embeds), self.pre_fc_norm_hidden(hidden)], dim=-1)
        r = linear_fp32(x, self.fc.weight)
        for layer in self.layers:
            r = layer(r, meta)
        return self.norm(r)


class HybridForCausalLM(nn.Module):
    def __init__(self, cfg: HybridConfig, with_mtp: bool = True, vision=None):
        """``vision``: a ``models.vision.VisionConfig``: the model then owns a vision tower (``visual``) whose rows the trainer
        computes from the trajectories' pictures with gradients (rollout replicas get finished rows and build without it)."""
        super().__init__()
        self.config = cfg
        self.model = Backbone(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.mtp = MTPHead(cfg) if (with_mtp and cfg.num_mtp_layers > 0) else None
        self.visual = None
        if vision is not None:
            from .vision import FamilyVisionConfig, FamilyVisionTower, VisionTower

            # the family's own tower (what its checkpoints carry under model.visual.*) or this framework's small ViT
            self.visual = FamilyVisionTower(vision) if isinstance(vision, FamilyVisionConfig) else VisionTower(vision)
        self.gradient_checkpointing = False
        self.activation_offload = None  # train.offload.CheckpointInputOffload when enabled

    # ---------------------------------------------------------------------------------------------------------------
    def init_weights(self, seed: int = 0) -> "HybridForCausalLM":
        """normal(0, init_std) for matrices and embeddings; zeros for (1+w) norm weights; ones for the plain gated
        norm; ``A_log`` = log of uniform(1, 16) decay rates and ``dt_bias`` from a softplus-inverse of small steps."""
        gen = torch.Generator().manual_seed(seed)
        std = self.config.init_std
        for name, p in self.named_parameters():
            with torch.no_grad():
                if name.endswith("A_log"):
                    p.copy_(torch.log(torch.empty(p.shape).uniform_(1.0, 16.0, generator=gen)))
                elif name.endswith("dt_bias"):
                    dt = torch.exp(torch.empty(p.shape).uniform_(0.0, 1.0, generator=gen) * (
                        torch.log(torch.tensor(0.1)) - torch.log(torch.tensor(0.001))) + torch.log(torch.tensor(0.001)))
                    p.copy_(dt + torch.log(-torch.expm1(-dt)))
                elif p.dim() >= 2:
                    p.copy_((torch.randn(p.shape, generator=gen) * std).to(p.dtype))
                elif "linear_attn.norm" in name:
                    p.fill_(1.0)
                else:
                    p.zero_()
        if self.visual is not None:
            self.visual.init_weights(seed)  # its own rule (LayerNorm weights are ones)
        return self

    def init_weights_device(self, seed: int = 0) -> "HybridForCausalLM":
        """The rule of :meth:`init_weights` drawn on the parameters' own device (a 27B-shape model is initialised on the
        GPU in seconds; the CPU generator of ``init_weights`` would take minutes and the host memory of the whole model)."""
        std = self.config.init_std
        dev = next(self.parameters()).device
        gen = torch.Generator(device=dev).manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("A_log"):
                    p.copy_(torch.log(torch.empty(p.shape, device=dev, dtype=torch.float32).uniform_(1.0, 16.0, generator=gen)))
                elif name.endswith("dt_bias"):
                    u = torch.empty(p.shape, device=dev, dtype=torch.float32).uniform_(0.0, 1.0, generator=gen)
                    dt = torch.exp(u * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
                    p.copy_(dt + torch.log(-torch.expm1(-dt)))
                elif p.dim() >= 2:
                    p.normal_(0.0, std, generator=gen)
                elif "linear_attn.norm" in name:
                    p.fill_(1.0)
                else:
                    p.zero_()
        if self.visual is not None:
            self.visual.init_weights(seed)
        return self

    def rope(self, position_ids: torch.Tensor):
        cfg = self.config
        return ops.mrope_cos_sin(position_ids, cfg.rotary_dim, cfg.rope_theta, cfg.mrope_sections)

    def make_meta(self, position_ids: torch.Tensor, cu_seqlens, sp=None, offset: int = 0) -> SeqMeta:
        cos, sin = self.rope(position_ids)
        cs = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
        return SeqMeta(cu_seqlens=cs, cos=cos, sin=sin, sp=sp, offset=offset)

    def embed(self, input_ids: torch.Tensor, inputs_embeds: Optional[torch.Tensor] = None,
              embeds_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Token embeddings on the fp32 stream; rows where ``embeds_mask`` is set take ``inputs_embeds`` (vision
        placeholder blocks) instead."""
        r = self.model.embed_tokens(input_ids).float()
        if inputs_embeds is not None:
            r = torch.where(embeds_mask[:, None], inputs_embeds.float(), r) if embeds_mask is not None \
                else inputs_embeds.float()
        return r

    def run_layers(self, r: torch.Tensor, meta: SeqMeta) -> torch.Tensor:
        runner = getattr(self, "layer_runner", None)
        for i, layer in enumerate(self.model.layers):
            r = runner(i, layer, r, meta) if runner is not None else layer(r, meta)
        return r

    def forward(self, input_ids: torch.Tensor, position_ids: Optional[torch.Tensor] = None, cu_seqlens=None,
                inputs_embeds: Optional[torch.Tensor] = None, embeds_mask: Optional[torch.Tensor] = None,
                sp=None, offset: int = 0, return_prenorm: bool = False):
        """Packed forward. ``input_ids`` [T]; returns the final-norm hidden states fp32 [T, H] (and the pre-norm
        residual for the MTP head when asked)."""
        t = input_ids.shape[0]
        if position_ids is None:
            position_ids = _positions_from_cu(cu_seqlens if cu_seqlens is not None else [0, t], t, input_ids.device)
        if cu_seqlens is None:
            cu_seqlens = [0, t]
        meta = self.make_meta(position_ids, cu_seqlens, sp, offset)
        r = self.run_layers(self.embed(input_ids, inputs_embeds, embeds_mask), meta)
        h = self.model.norm(r)
        return (h, r) if return_prenorm else h

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return linear_fp32(hidden, self.lm_head.weight)

    def mtp_hidden(self, next_ids: torch.Tensor, prenorm_hidden: torch.Tensor, position_ids, cu_seqlens) -> torch.Tensor:
        """Hidden states of the MTP layer predicting token t+2 from the backbone state at t and token t+1."""
        meta = self.make_meta(position_ids, cu_seqlens)
        return self.mtp(self.model.embed_tokens(next_ids).float(), prenorm_hidden, meta)


def mrope_positions(input_ids: torch.Tensor, image_grids: list[tuple[int, int]], image_pad_id: int, merge: int = 2) -> torch.Tensor:
    """(temporal, row, column) positions ``[3, T]`` of one sequence with pictures, as the family's checkpoints were trained: text
    tokens advance all three together; the rows of a picture (a run of ``image_pad_id`` tokens, ``gh / merge x gw / merge`` of them
    for a patch grid ``gh x gw``) share the temporal position where the picture starts and count rows and columns from it; the
    text after a picture continues from the largest position the picture used plus one. The rollout and training paths of this
    framework give pictures sequential positions instead (consistent with each other, not with a pretrained checkpoint's
    pictures); this function is the checkpoint's rule, checked against ``transformers`` in ``tests/test_hf_parity_cpu.py``."""
    ids = input_ids.tolist()
    pos = torch.zeros(3, len(ids), dtype=torch.long)
    nxt, i, k = 0, 0, 0
    while i < len(ids):
        if ids[i] == image_pad_id:
            gh, gw = image_grids[k]
            k += 1
            rows, cols = gh // merge, gw // merge
            n = rows * cols
            if ids[i:i + n] != [image_pad_id] * n:
                raise ValueError(f"picture {k - 1} needs {n} image-pad tokens at position {i}")
            r = torch.arange(rows).repeat_interleave(cols)
            c = torch.arange(cols).repeat(rows)
            pos[0, i:i + n], pos[1, i:i + n], pos[2, i:i + n] = nxt, nxt + r, nxt + c
            nxt += max(rows, cols)
            i += n
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    if k != len(image_grids):
        raise ValueError(f"{len(image_grids)} pictures given, {k} found in the tokens")
    return pos


def _positions_from_cu(cu_seqlens, t: int, device) -> torch.Tensor:
    cs = cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else list(cu_seqlens)
    pos = torch.empty(t, dtype=torch.long, device=device)
    for s, e in zip(cs[:-1], cs[1:]):
        pos[s:e] = torch.arange(e - s, device=device)
    return pos


# ---------------------------------------------------------------------------------------------------------------------
# incremental (cached) reference for one sequence: the oracle of the rollout engine and of the decode megakernel
# ---------------------------------------------------------------------------------------------------------------------
class DenseCache:
    """Per-layer state of one sequence: attention K/V rows, GDN conv rows and recurrent state."""

    def __init__(self, cfg: HybridConfig):
        self.cfg = cfg
        self.k: dict[int, torch.Tensor] = {}
        self.v: dict[int, torch.Tensor] = {}
        self.conv: dict[int, torch.Tensor] = {}
        self.state: dict[int, torch.Tensor] = {}
        self.length = 0

    def clone(self) -> "DenseCache":
        c = DenseCache(self.cfg)
        c.k = {i: t.clone() for i, t in self.k.items()}
        c.v = {i: t.clone() for i, t in self.v.items()}
        c.conv = {i: t.clone() for i, t in self.conv.items()}
        c.state = {i: t.clone() for i, t in self.state.items()}
        c.length = self.length
        return c


@torch.no_grad()
def forward_cached(model: HybridForCausalLM, input_ids: torch.Tensor, cache: DenseCache,
                   position_ids: Optional[torch.Tensor] = None, layers=None, key_offset: int = 0,
                   embeds: Optional[torch.Tensor] = None, return_prenorm: bool = False):
    """Append ``input_ids`` [T] to one sequence's cache; returns final-norm hidden [T, H] fp32."""
    cfg = model.config
    t = input_ids.shape[0]
    start = cache.length
    if position_ids is None:
        position_ids = torch.arange(start, start + t, device=input_ids.device)
    cos, sin = model.rope(position_ids)
    meta = SeqMeta(cu_seqlens=[0, t], cos=cos, sin=sin)
    r = embeds if embeds is not None else model.embed(input_ids)
    layer_list = layers if layers is not None else model.model.layers
    for i, layer in enumerate(layer_list):
        li = i + key_offset
        h = layer.input_layernorm(r)
        if layer.layer_type == "full_attention":
            att = layer.self_attn
            q, k, v, gate = att.project(h, meta)
            kc = torch.cat([cache.k[li], k], dim=0) if li in cache.k else k
            vc = torch.cat([cache.v[li], v], dim=0) if li in cache.v else v
            cache.k[li], cache.v[li] = kc, vc
            from ..ops import reference as ref

            o = ref.attention_with_cache(q, kc, vc, kc.shape[0] - t, cfg.head_dim ** -0.5)
            mixed = row_linear((ops.sigmoid_gate(o, gate) if gate is not None else o).reshape(t, cfg.q_size), att.o_proj.weight)
        else:
            gdn = layer.linear_attn
            x = linear_fp32(h, gdn.in_proj_qkv.weight)
            z = linear_fp32(h, gdn.in_proj_z.weight).view(t, cfg.gdn_v_heads, cfg.gdn_head_dim)
            g, beta = ops.gdn_gates(linear_fp32(h, gdn.in_proj_a.weight), linear_fp32(h, gdn.in_proj_b.weight),
                                    gdn.A_log, gdn.dt_bias)
            init = cache.conv[li].unsqueeze(0) if li in cache.conv else None
            q, k, v, conv_final = gdn.front(x, [0, t], init)
            cache.conv[li] = conv_final[0]
            from ..ops import reference as ref

            o, s = ref.gdn_recurrent(q, k, v, g, beta, cache.state.get(li))
            cache.state[li] = s
            y = ops.gated_rms_norm(o, z, gdn.norm.weight, cfg.rms_eps).reshape(t, cfg.gdn_value_dim)
            mixed = row_linear(y, gdn.out_proj.weight)
        y, r = ops.add_rms_norm(mixed, r, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
        r = r + layer.mlp(y)
    if layers is None:
        cache.length += t
        h = model.model.norm(r)
        return (h, r) if return_prenorm else h
    return r

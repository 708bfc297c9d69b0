"""Trainer engine: sharded hybrid model + GRPO forward/backward over packed micro-batches + optimizer step.

The role of upstream ``pear/trainer/engine.py`` (``PearFSDPEngine``): kernels are installed in a fixed order before the
model is sharded (``kernels.install`` -> ``check_model`` -> ``install_gpu_backend`` -> ``install_checkpointing``,
``engine.py:71-98``), garbage collection is frozen after init (``:55-62``), a batch whose fast path reports an overflow
is re-run on the safe path (``forward_backward_batch`` ``:100-112``), and the sampler's top-k head ids are passed into
the fused head whose log-probs become the score-centering term (``:114-137``). The optimizer update is clip -> skip on a
non-finite norm -> step (``3rdparty/verl/patches/0017-*``); a resumed run trains at the CONFIGURED learning rate at the
restored schedule position (``0003-*``).
"""

from __future__ import annotations

import gc
import math
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from ..models.config import HybridConfig
from ..models.hybrid import HybridForCausalLM
from ..models.kernels import TrainingKernels
from ..ops import api as ops
from ..parallel.fsdp import ShardedModel
from ..parallel.ulysses import SequenceParallel
from . import grpo
from .checkpointing import LayerRunner, install as install_runner
from .offload import CheckpointInputOffload
from .fused_adamw import FusedAdamW
from .streamed_adamw import StreamedAdamW


@dataclass
class PackedBatch:
    """Packed (padding-free) trajectories. All per-token tensors have T entries; ``labels[t]`` is the token following
    ``input_ids[t]`` inside its sequence (anything where ``loss_mask`` is 0)."""

    input_ids: torch.Tensor
    position_ids: torch.Tensor
    cu_seqlens: list[int]
    labels: torch.Tensor
    loss_mask: torch.Tensor
    advantages: torch.Tensor
    sampler_log_probs: Optional[torch.Tensor] = None
    head_ids: Optional[torch.Tensor] = None
    head_log_probs: Optional[torch.Tensor] = None
    inputs_embeds: Optional[torch.Tensor] = None
    embeds_mask: Optional[torch.Tensor] = None
    # pictures whose rows the trainer computes itself (a vision tower in the training graph): (position of the first row in the
    # packed batch, uint8 [H, W, 3] picture); positions are global to the batch and survive padding and slicing unchanged
    images: Optional[list] = None

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0])

    def to(self, device) -> "PackedBatch":
        kw = {}
        for k, v in self.__dict__.items():
            kw[k] = v.to(device, non_blocking=True) if torch.is_tensor(v) else v
        return PackedBatch(**kw)

    def pad_to_multiple(self, m: int) -> "PackedBatch":
        """Append a dummy masked sequence so that T is a multiple of ``m`` (equal sequence-parallel slices)."""
        pad = (-self.num_tokens) % m
        if pad == 0:
            return self
        def ext(t, fill=0):
            if t is None:
                return None
            shape = (pad,) + tuple(t.shape[1:])
            return torch.cat([t, torch.full(shape, fill, dtype=t.dtype, device=t.device)], dim=0)
        pos = self.position_ids
        if pos.dim() == 2:
            pos = torch.cat([pos, torch.arange(pad, device=pos.device).expand(pos.shape[0], pad)], dim=1)
        else:
            pos = torch.cat([pos, torch.arange(pad, device=pos.device)])
        return PackedBatch(
            input_ids=ext(self.input_ids), position_ids=pos, cu_seqlens=self.cu_seqlens + [self.cu_seqlens[-1] + pad],
            labels=ext(self.labels), loss_mask=ext(self.loss_mask), advantages=ext(self.advantages),
            sampler_log_probs=ext(self.sampler_log_probs), head_ids=ext(self.head_ids),
            head_log_probs=ext(self.head_log_probs, -math.log(max(1, self.head_ids.shape[1])) if self.head_ids is not None else 0),
            inputs_embeds=ext(self.inputs_embeds), embeds_mask=ext(self.embeds_mask, False) if self.embeds_mask is not None else None,
            images=self.images)

    def slice(self, lo: int, hi: int) -> "PackedBatch":
        def cut(t):
            return None if t is None else t[lo:hi]
        pos = self.position_ids[..., lo:hi]
        return PackedBatch(cut(self.input_ids), pos, self.cu_seqlens, cut(self.labels), cut(self.loss_mask), cut(self.advantages),
                           cut(self.sampler_log_probs), cut(self.head_ids), cut(self.head_log_probs), cut(self.inputs_embeds),
                           cut(self.embeds_mask), self.images)


@dataclass
class EngineConfig:
    lr: float = 1e-6
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_grad: float = 1.0
    lr_warmup_steps: int = 0
    param_dtype: str = "bf16"
    fp32_modules: list = field(default_factory=list)
    ulysses_sequence_parallel_size: int = 1
    # ranks per sharding group: -1 (or the world size) shards over the whole world (FSDP); a divisor S of the world size
    # gives world / S replicas of an S-way sharded model (HSDP): reduce-scatter inside a shard group, all-reduce of the
    # shard gradients across replicas on the last micro-batch
    fsdp_size: int = -1
    enable_gradient_checkpointing: bool = True
    gradient_checkpointing_retain_attention: bool = False
    enable_activation_offload: bool = False
    streamed_adamw: bool = False
    streamed_chunk_bytes: int = 2 << 30
    temperature: float = 1.0
    topk_log_probs: int = 0
    head_chunk: int = 4096
    loss: grpo.LossConfig = field(default_factory=grpo.LossConfig)
    kernels: Optional[str] = None
    use_gpu_backend: bool = False
    hsdp_all_reduce_on_last_micro_batch: bool = True
    # fp32 matrix products left to the library on a GPU (the chunked delta-rule scan, attention with gradients) run on
    # the TF32 tensor cores instead of SIMT fp32; the head's logits do not (split-bf16 GEMM, close to fp32)
    tf32_matmul: bool = True
    fused_adamw: bool = True  # on a GPU: one kernel pass per parameter tensor instead of torch's AdamW statements
    # multi-rank runs: only rank 0 builds (or loads) real weights, the other ranks build the model on the meta device and
    # receive their shards unit by unit (no rank but 0 ever holds the whole model; rank 0 holds it on the host only)
    sharded_construction: bool = True

    @classmethod
    def from_config(cls, cfg) -> "EngineConfig":
        """From a composed recipe (``actor_rollout_ref`` / ``algorithm`` sections with the upstream key names)."""
        actor, model, rollout = cfg.actor_rollout_ref.actor, cfg.actor_rollout_ref.model, cfg.actor_rollout_ref.rollout
        fs = actor.fsdp_config
        rc = cfg.algorithm.rollout_correction
        return cls(
            lr=float(actor.optim.lr), betas=tuple(actor.optim.get("betas", (0.9, 0.999))), eps=float(actor.optim.get("eps", 1e-8)),
            weight_decay=float(actor.optim.get("weight_decay", 0.01)), clip_grad=float(actor.get("clip_grad", 1.0)),
            lr_warmup_steps=int(actor.optim.get("lr_warmup_steps", 0)), param_dtype=fs.mixed_precision.get("param_dtype", "bf16"),
            fp32_modules=list(fs.mixed_precision.get("fp32_modules", [])),
            ulysses_sequence_parallel_size=int(fs.ulysses_sequence_parallel_size), fsdp_size=int(fs.get("fsdp_size", -1)),
            enable_gradient_checkpointing=bool(model.enable_gradient_checkpointing),
            enable_activation_offload=bool(model.get("enable_activation_offload", False)),
            gradient_checkpointing_retain_attention=bool(model.get("gradient_checkpointing_retain_attention", False)),
            streamed_adamw=bool(fs.get("streamed_adamw", False) or fs.get("optimizer_offload", False) or fs.get("optimizer_offload_step", False)),
            temperature=float(rollout.temperature), topk_log_probs=int(rollout.get("topk_log_probs", 0)),
            loss=grpo.LossConfig(loss_agg_mode=actor.loss_agg_mode, score_centering=bool(rc.score_centering),
                                 rollout_is=rc.get("rollout_is"), rollout_is_threshold=rc.get("rollout_is_threshold", 2.0),
                                 entropy_coeff=float(actor.entropy_coeff)),
            kernels=fs.get("kernels"), use_gpu_backend=bool(fs.get("use_gpu_backend", False)),
            hsdp_all_reduce_on_last_micro_batch=bool(fs.get("hsdp_all_reduce_on_last_micro_batch", True)))


class TrainEngine:
    def __init__(self, model_cfg: HybridConfig, cfg: EngineConfig, device="cpu", world_group=None, replicate_group=None,
                 kernels: Optional[type[TrainingKernels]] = None, seed: int = 0, state_dict: Optional[dict] = None,
                 with_mtp: bool = False, vision=None):
        """``vision``: a ``VisionConfig``: the model gets a vision tower, kept in fp32 units of its own, and batches may carry
        pictures (``PackedBatch.images``) whose rows are computed here, sharded over the sequence-parallel ranks."""
        self.model_cfg, self.cfg, self.device = model_cfg, cfg, torch.device(device)
        self.group = world_group
        self.world = dist.get_world_size(world_group) if world_group is not None else 1
        self.rank = dist.get_rank(world_group) if world_group is not None else 0
        sp = cfg.ulysses_sequence_parallel_size
        if self.world % sp:
            raise ValueError(f"world size {self.world} is not a multiple of the sequence-parallel size {sp}")
        self.sp_size, self.dp_size = sp, self.world // sp
        self.dp_rank, self.sp_rank = self.rank // sp, self.rank % sp
        self.sp_group = None
        if sp > 1:
            for d in range(self.dp_size):  # every rank creates every group (collective call)
                g = dist.new_group(list(range(d * sp, (d + 1) * sp)))
                if d == self.dp_rank:
                    self.sp_group = g
        self.sp = SequenceParallel(self.sp_group) if sp > 1 else None
        # ---- sharding groups. `group` / `world` / `rank` stay the whole job's (data distribution, checkpoints, the driver rank);
        # the sharder and the gradient norm work inside `shard_group`
        self.shard_group, self.shard_world, self.shard_rank = world_group, self.world, self.rank
        S = cfg.fsdp_size
        if replicate_group is None and self.world > 1 and 0 < S < self.world:
            if self.world % S or S % sp:
                raise ValueError(f"fsdp_size {S} must divide the world size {self.world} and be a multiple of the sequence-parallel size {sp}")
            ranks = [dist.get_global_rank(world_group, r) for r in range(self.world)]
            for i in range(self.world // S):  # every rank creates every group (collective calls), in the same order
                g = dist.new_group(ranks[i * S:(i + 1) * S])
                if i == self.rank // S:
                    self.shard_group = g
            for j in range(S):
                g = dist.new_group(ranks[j::S])
                if j == self.rank % S:
                    replicate_group = g
            self.shard_world, self.shard_rank = S, self.rank % S
        self.replicate_group = replicate_group
        self.vision_min_pixels, self.vision_max_pixels = 0, 1 << 22  # (the agent loop's encoder must be given the same bounds)
        if kernels is None and cfg.kernels:  # the recipe names the family's training kernels by class path (`fsdp_config.kernels`)
            import importlib

            module_path, _, name = str(cfg.kernels).rpartition(".")
            kernels = getattr(importlib.import_module(module_path), name)
        self.kernels = kernels
        if kernels is not None:
            kernels.check_config(cfg)

        # ---- build: one rank builds the seeded model (or takes the given weights) on the host, the others on the meta device
        self.src_rank = 0 if (self.shard_world > 1 and cfg.sharded_construction) else None  # (rank 0 of every shard group)
        on_meta = self.src_rank is not None and self.shard_rank != self.src_rank
        if on_meta:
            with torch.device("meta"):
                model = HybridForCausalLM(model_cfg, with_mtp=with_mtp, vision=vision)
        else:
            model = HybridForCausalLM(model_cfg, with_mtp=with_mtp, vision=vision)
            if state_dict is not None:
                model.load_state_dict(state_dict, strict=False)
            else:
                model.init_weights(seed)
        if kernels is not None:  # the install order the GPU backend relies on
            kernels.install(model, fp32_residual=True, use_fused_kernels=True, fused_kernels_backend=None)
            kernels.check_model(model, use_remove_padding=True, use_fused_kernels=True, fused_kernels_backend=None)
            if cfg.use_gpu_backend:
                kernels.install_gpu_backend(model)
            kernels.install_checkpointing(model)
        if self.src_rank is None:
            model.to(self.device)  # (with a source rank the parameters go to the device unit by unit while they are sharded)
        dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[cfg.param_dtype]
        if self.device.type == "cpu" and dtype != torch.float32:
            dtype = torch.float32  # CPU plumbing runs in fp32
        self.model = model
        fp32_modules = list(cfg.fp32_modules) + (["visual."] if vision is not None and "visual." not in cfg.fp32_modules else [])
        self.sharded = ShardedModel(model, self.shard_group if self.shard_world > 1 else None, replicate_group, dtype, fp32_modules,
                                    self.device, src_rank=self.src_rank)
        for mod in model.modules():  # buffers (none hold weights) follow the parameters' device
            for bname, buf in list(mod._buffers.items()):
                if buf is not None and buf.device != self.device:
                    mod._buffers[bname] = torch.zeros_like(buf, device=self.device) if buf.is_meta else buf.to(self.device)
        self.offload = CheckpointInputOffload(True) if cfg.enable_activation_offload else None
        self.runner = LayerRunner(self.sharded, self.offload, cfg.enable_gradient_checkpointing,
                                  retain_attention=cfg.gradient_checkpointing_retain_attention,
                                  skip_down_proj=bool(getattr(model, "recompute_skips_down_proj", False)))
        install_runner(model, self.runner)
        self.fused_adamw = (not cfg.streamed_adamw) and self.device.type == "cuda" and cfg.fused_adamw
        opt_cls = StreamedAdamW if cfg.streamed_adamw else (FusedAdamW if self.fused_adamw else torch.optim.AdamW)
        kw = dict(lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay)
        if cfg.streamed_adamw:
            kw["chunk_bytes"] = cfg.streamed_chunk_bytes
        elif not self.fused_adamw:
            kw.update(foreach=False, fused=False)
        self.optimizer = opt_cls(self.sharded.parameters(), **kw)
        self.step_count = 0
        self.policy_version = 0
        gc.collect()
        gc.freeze()  # the long-lived model objects leave the collector's working set

    # -- learning rate ------------------------------------------------------------------------------------------------
    def _lr_at(self, step: int) -> float:
        w = self.cfg.lr_warmup_steps
        return self.cfg.lr * min(1.0, (step + 1) / w) if w > 0 else self.cfg.lr

    # -- micro-batch forward/backward -----------------------------------------------------------------------------------
    def _forward_loss(self, mb: PackedBatch, denom: torch.Tensor):
        """Loss of this rank's slice of one packed micro-batch."""
        cfg = self.cfg
        mb = mb.pad_to_multiple(self.sp_size)
        t = mb.num_tokens
        t_local = t // self.sp_size
        lo = self.sp_rank * t_local
        loc = mb.slice(lo, lo + t_local) if self.sp_size > 1 else mb
        inputs_embeds, embeds_mask = loc.inputs_embeds, loc.embeds_mask
        if mb.images and self.model.visual is not None:
            inputs_embeds, embeds_mask = self._image_rows(mb.images, lo, t_local, inputs_embeds, embeds_mask)
        hidden = self.model(loc.input_ids, loc.position_ids, mb.cu_seqlens, inputs_embeds=inputs_embeds,
                            embeds_mask=embeds_mask, sp=self.sp, offset=lo)
        ids = loc.labels[:, None].long()
        use_sc = cfg.loss.score_centering and loc.head_ids is not None
        if use_sc:
            ids = torch.cat([ids, loc.head_ids.long()], dim=1)
        if getattr(self.model, "use_fused_head", True):  # chunked: the [tokens, vocabulary] logits never exist whole
            lp, ent = ops.logprob_entropy(hidden, self.model.lm_head.weight, ids, cfg.temperature, cfg.head_chunk)
        else:
            lp, ent = ops.ref.logprob_entropy_dense(hidden, self.model.lm_head.weight, ids, cfg.temperature)
        loss, metrics = grpo.policy_loss(
            lp[:, 0], loc.advantages, loc.loss_mask, cfg.loss, head_log_probs=lp[:, 1:] if use_sc else None,
            sampler_head_log_probs=loc.head_log_probs if use_sc else None, sampler_log_probs=loc.sampler_log_probs,
            entropy=ent, denominator=denom)
        return loss, metrics

    def _image_rows(self, images: list, lo: int, t_local: int, inputs_embeds, embeds_mask):
        """The vision tower's rows for a micro-batch's pictures, placed at their positions inside this rank's slice
        ``[lo, lo + t_local)``. Every picture is encoded once, by the sequence-parallel rank it is dealt to (by patch count);
        the rows are all-gathered with gradients (``parallel/vision_sp.py``), so the tower trains under the policy loss."""
        from ..models.vision import prepare_picture, tower_cell
        from ..parallel.vision_sp import encode_sharded

        dev = self.device
        cell = tower_cell(self.model.visual.cfg)
        pics = [prepare_picture(img, cell, self.vision_min_pixels, self.vision_max_pixels, dev) for _, img in images]  # as the agent loop's encoder does
        rows = encode_sharded(self.model.visual, pics, self.sp_group)
        h = self.model_cfg.hidden_size
        base = inputs_embeds.float() if inputs_embeds is not None else torch.zeros(t_local, h, device=dev)
        mask = embeds_mask.clone() if embeds_mask is not None else torch.zeros(t_local, dtype=torch.bool, device=dev)
        idx, parts = [], []
        for (pos, _), block in zip(images, rows):
            a, b = max(pos, lo), min(pos + block.shape[0], lo + t_local)
            if a < b:
                idx.append(torch.arange(a - lo, b - lo, device=dev))
                parts.append(block[a - pos:b - pos])
        keep = sum(r.sum() for r in rows) * 0.0  # every rank's graph reaches the gathered rows: the backward collectives stay matched
        if idx:
            where = torch.cat(idx)
            base = base.index_copy(0, where, torch.cat(parts).to(base.dtype))
            mask[where] = True
        return base + keep, mask

    def forward_backward_batch(self, micro_batches: list[PackedBatch], total_loss_tokens: Optional[int] = None) -> dict:
        """Accumulate gradients over this DP rank's micro-batches. ``total_loss_tokens``: loss tokens of the GLOBAL
        batch (token-mean over everything the step trains on); computed by an all-reduce when omitted."""
        local = sum(int(mb.loss_mask.sum()) for mb in micro_batches)
        if total_loss_tokens is None:
            tot = torch.tensor([float(local)], device=self.device)
            if self.world > 1:
                if self.sp_rank != 0:
                    tot.zero_()
                dist.all_reduce(tot, group=self.group)
            total_loss_tokens = int(tot.item())
        denom = torch.tensor(float(max(1, total_loss_tokens)), device=self.device)

        def run():
            agg: dict[str, float] = {}
            self.sharded.gather_static()
            for i, mb in enumerate(micro_batches):
                self.runner.last_micro_batch = (i == len(micro_batches) - 1) or not self.cfg.hsdp_all_reduce_on_last_micro_batch
                loss, metrics = self._forward_loss(mb.to(self.device), denom)
                loss.backward()
                w = float(mb.loss_mask.sum()) / max(1, local)
                for k, v in metrics.items():
                    agg[k] = agg.get(k, 0.0) + (v if k == "actor/pg_loss" else v * w)
                if self.offload is not None:
                    self.offload.clear()
            self.sharded.reduce_static_grads(True)
            self.sharded.release_static()
            self.sharded.wait_grads()
            return agg

        def before_rerun():
            self.optimizer.zero_grad(set_to_none=True)

        # fp32 library products of the step (delta-rule scan, attention with gradients) on the TF32 tensor cores; the
        # process-wide switch is put back afterwards so that nothing else in the process changes precision
        tf32 = self.device.type == "cuda" and self.cfg.tf32_matmul
        prev = torch.backends.cuda.matmul.allow_tf32
        if tf32:
            torch.backends.cuda.matmul.allow_tf32 = True
        try:
            if self.kernels is not None:
                return self.kernels.run_checked(run, before_rerun)
            return run()
        finally:
            if tf32:
                torch.backends.cuda.matmul.allow_tf32 = prev

    # -- optimizer ----------------------------------------------------------------------------------------------------
    def _grad_norm(self) -> torch.Tensor:
        sq = torch.zeros((), device=self.device)
        for p in self.sharded.parameters():
            if p.grad is not None:
                sq = sq + p.grad.float().pow(2).sum()
        if self.shard_world > 1:  # (replicas of a shard hold the same gradient after the cross-replica all-reduce)
            dist.all_reduce(sq, group=self.shard_group)
        return sq.sqrt()

    def optimizer_step(self) -> dict:
        """Clip by the global norm, skip the update when the norm is not finite, step."""
        for g in self.optimizer.param_groups:
            g["lr"] = self._lr_at(self.step_count)
        norm = self._grad_norm()
        metrics = {"actor/grad_norm": float(norm), "actor/lr": self.optimizer.param_groups[0]["lr"]}
        if not torch.isfinite(norm):
            self.optimizer.zero_grad(set_to_none=True)
            metrics["actor/skipped_update"] = 1.0
            return metrics
        scale = min(1.0, self.cfg.clip_grad / (float(norm) + 1e-6)) if self.cfg.clip_grad > 0 else 1.0
        if self.fused_adamw:
            self.optimizer.step(grad_scale=scale)  # the clip coefficient rides in the update's single pass
        else:
            if scale < 1.0:
                for p in self.sharded.parameters():
                    if p.grad is not None:
                        p.grad.mul_(scale)
            self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.step_count += 1
        self.policy_version += 1
        return metrics

    # -- state --------------------------------------------------------------------------------------------------------
    def full_state_dict(self, dtype=torch.float32) -> dict[str, torch.Tensor]:
        return self.sharded.full_state_dict(dtype)

    def train_state(self) -> dict:
        return {"shards": self.sharded.shard_state(), "optimizer": self.optimizer.state_dict(), "step": self.step_count,
                "policy_version": self.policy_version, "world_size": self.world, "shard_world_size": self.shard_world}

    def load_train_state(self, st: dict) -> None:
        if st["world_size"] != self.world:
            raise ValueError(f"checkpoint was written by world size {st['world_size']}, this run has {self.world}")
        if st.get("shard_world_size", st["world_size"]) != self.shard_world:
            raise ValueError(f"checkpoint was sharded over {st.get('shard_world_size')} ranks, this run shards over {self.shard_world}")
        self.sharded.load_shard_state(st["shards"])
        self.optimizer.load_state_dict(st["optimizer"])
        self.step_count, self.policy_version = st["step"], st["policy_version"]
        for g in self.optimizer.param_groups:  # the configured LR, at the restored schedule position
            g["lr"] = self._lr_at(self.step_count)


def synthetic_batch(cfg: HybridConfig, tokens: int, seqs: int, topk: int, seed: int) -> PackedBatch:
    """A packed micro-batch of uniform-random token ids in ``seqs`` equal sequences, N(0, 1) advantages on the second half of
    each sequence (the "response"): the synthetic data of the trainer benchmarks and GPU tests."""
    g = torch.Generator().manual_seed(seed)
    per = tokens // seqs
    cu = [i * per for i in range(seqs)] + [tokens]
    ids = torch.randint(0, cfg.vocab_size, (tokens,), generator=g)
    pos = torch.cat([torch.arange(e - s) for s, e in zip(cu[:-1], cu[1:])])
    mask = torch.ones(tokens)
    for s, e in zip(cu[:-1], cu[1:]):
        mask[s: s + (e - s) // 2] = 0
        mask[e - 1] = 0
    return PackedBatch(ids, pos, cu, torch.roll(ids, -1), mask, torch.randn(tokens, generator=g) * mask,
                       sampler_log_probs=-torch.rand(tokens, generator=g) * 3,
                       head_ids=torch.randint(0, cfg.vocab_size, (tokens, topk), generator=g, dtype=torch.int32) if topk else None,
                       head_log_probs=torch.log_softmax(torch.randn(tokens, topk + 2, generator=g), -1)[:, :topk] if topk else None)

"""Batch-1 NVFP4 decode engine on the persistent megakernel: weights, buffers, programs and the step loop.

The counterpart of upstream ``pear/models/qwen3_5/deploy/blackwell/nvfp4/step.py`` (``DecodeStep.build`` lays out a
whole verify step) and ``runner.py`` (``DecodeLaunch``: one request's decode/verify step is one launch). Here the engine
owns its memory instead of patching a serving runtime: packed NVFP4 weight stages, fp32 activation buffers, paged KV
cache (identity block table at batch 1), Gated-DeltaNet state/conv slots with per-block replay records, the step
records on the device and a ring of step outputs that is copied to pinned host memory after every launch.
"""

from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..models import nvfp4
from ..models.config import HybridConfig
from ..ops import lib as _lib
from . import schedule as S


class _Params(ctypes.Structure):
    _fields_ = [
        ("instrs", ctypes.c_void_p), ("descs", ctypes.c_void_p), ("rec", ctypes.c_void_p), ("out_ring", ctypes.c_void_p),
        ("barrier", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("max_instrs", ctypes.c_int32), ("ring", ctypes.c_int32), ("step_parity", ctypes.c_int32),
        ("seed", ctypes.c_uint32), ("temperature", ctypes.c_float), ("vocab", ctypes.c_int32),
        ("barrier_base", ctypes.c_uint32), ("pad", ctypes.c_int32), ("ctrl", ctypes.c_void_p),
        ("trace", ctypes.c_void_p), ("trace_ctas", ctypes.c_int32), ("trace_cap", ctypes.c_int32),
        ("l2_ahead", ctypes.c_int32), ("pad2", ctypes.c_int32),
        ("tile_cnt", ctypes.c_void_p), ("tile_expect", ctypes.c_void_p),
    ]


# ---------------------------------------------------------------------------------------------------------------------
# weight sources
# ---------------------------------------------------------------------------------------------------------------------
class RandomWeights:
    """Seeded random-init weights generated matrix by matrix on the device (a 27B model never exists unquantised)."""

    def __init__(self, device, seed: int = 0, std: float = 0.02):
        self.device, self.std = device, std
        self.gen = torch.Generator(device=device).manual_seed(seed)

    def matrix(self, name: str, rows: int, cols: int) -> torch.Tensor:
        return torch.randn(rows, cols, device=self.device, generator=self.gen, dtype=torch.float32) * self.std

    def vector(self, name: str, n: int) -> torch.Tensor:
        if name.endswith("A_log"):
            return torch.log(torch.empty(n, device=self.device).uniform_(1.0, 16.0, generator=self.gen))
        if name.endswith("dt_bias"):
            dt = torch.exp(torch.empty(n, device=self.device).uniform_(0.0, 1.0, generator=self.gen)
                           * (math.log(0.1) - math.log(0.001)) + math.log(0.001))
            return dt + torch.log(-torch.expm1(-dt))
        if name.endswith("linear_attn.norm.weight"):
            return torch.ones(n, device=self.device)
        return torch.zeros(n, device=self.device)


class ModuleWeights:
    """Weights of a :class:`HybridForCausalLM` (keys as in its state dict) and a :class:`BlockDrafter` (``draft.*``)."""

    def __init__(self, model, drafter, device):
        self.device = device
        self.sd = {k: v for k, v in model.state_dict().items()}
        if drafter is not None:
            self.sd.update({"draft." + k: v for k, v in drafter.state_dict().items()})

    def matrix(self, name: str, rows: int, cols: int) -> torch.Tensor:
        w = self.sd[name].to(self.device, torch.float32).reshape(rows, cols)
        return w

    def vector(self, name: str, n: int) -> torch.Tensor:
        return self.sd[name].to(self.device, torch.float32).reshape(n)


@dataclass
class GenerationResult:
    tokens: list[int]
    steps: int
    accepted: int
    prefill_steps: int


# ---------------------------------------------------------------------------------------------------------------------
# engine
# ---------------------------------------------------------------------------------------------------------------------
class MegakernelEngine:
    """One sequence, one GPU. ``prefill`` then ``decode_steps``/``generate``."""

    RING = 64
    # (weight ring stages, rows of the activation operand) per program: decode steps have <= 4 rows (4 FP4 terms per row in
    # a 16-row operand); prefill blocks have 8 rows (4 terms in a 32-row operand and a shorter ring)
    LAUNCH_SHAPE = {"decode": (8, 16), "prefill": (5, 32)}
    L2_AHEAD = 0  # weight stages per CTA requested into L2 beyond the ring (148 x 16 x 18 KB = 44 MB of the 126 MB L2)
    CHUNK = 1024  # vocab entries per sampler partial

    def __init__(self, cfg: HybridConfig, draft_cfg: Optional[HybridConfig], weights, device="cuda", max_len: int = 8192,
                 n_draft: int = 3, seed: int = 0, temperature: float = 1.0, num_ctas: Optional[int] = None,
                 mask_token_id: int = 0, attn_splits: Optional[int] = None):
        assert cfg.gdn_head_dim == 128 and cfg.rotary_dim == 64 and cfg.head_dim in (128, 256)
        assert cfg.hidden_size % 256 == 0 and cfg.intermediate_size % 256 == 0 and cfg.hidden_size <= 5120
        assert 0 <= n_draft <= 3 or draft_cfg is None
        self.cfg, self.draft_cfg, self.device = cfg, draft_cfg, torch.device(device)
        self.n_draft = n_draft if draft_cfg is not None else 0
        self.max_len, self.seed, self.temperature, self.mask_token_id = max_len, seed, temperature, mask_token_id
        props = torch.cuda.get_device_properties(self.device)
        self.num_ctas = num_ctas or props.multi_processor_count
        self.attn_splits = attn_splits
        self._keep: list[torch.Tensor] = []  # owns every device allocation the descriptors point into
        self.weight_bytes = 0
        self._build(weights)
        self.launches = 0
        self._use_ctrl = True
        self.l2_ahead = int(os.environ.get("PEAR_MK_L2_AHEAD", self.L2_AHEAD))
        self._trace, self._trace_ctas, self._trace_cap = None, 0, 0
        self.barrier_base = 0
        self.reset()

    # -- allocation helpers ------------------------------------------------------------------------------------------
    def _zeros(self, *shape, dtype=torch.float32) -> torch.Tensor:
        t = torch.zeros(*shape, dtype=dtype, device=self.device)
        self._keep.append(t)
        return t

    def _dev(self, t: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
        t = t.to(self.device, dtype).contiguous()
        self._keep.append(t)
        return t

    def _pack(self, w: torch.Tensor) -> tuple[torch.Tensor, float]:
        packed, gs = nvfp4.quantize_packed(w)
        self._keep.append(packed)
        self.weight_bytes += packed.numel()
        return packed, gs

    # -- build -------------------------------------------------------------------------------------------------------
    def _build(self, W) -> None:
        cfg, dc = self.cfg, self.draft_cfg
        H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
        T8 = 8
        C, VD, HV, HK = cfg.gdn_conv_dim, cfg.gdn_value_dim, cfg.gdn_v_heads, cfg.gdn_qk_heads
        self.rec_stride = ((C + VD + 2 * HV + 127) // 128) * 128
        qw = (2 if cfg.attn_output_gate else 1) * cfg.head_dim
        self.qkv_stride = cfg.num_attention_heads * qw + 2 * cfg.kv_size
        nchunks = (V + self.CHUNK - 1) // self.CHUNK
        self.nchunks = nchunks

        # buffers
        self.r = self._zeros(T8, H)
        self.gu = self._zeros(T8, 2 * I)
        self.gdn_o = self._zeros(T8, VD)
        self.attn_out = self._zeros(T8, cfg.q_size)
        self.qkv = self._zeros(T8, self.qkv_stride)
        self.logits = self._zeros(T8, V)
        self.sample_part = self._zeros(T8, nchunks, 4)
        self.rec = torch.zeros(2, S.STEPREC_INTS, dtype=torch.int32, device=self.device)
        self.out_ring = torch.zeros(self.RING, S.STEPOUT_DTYPE.itemsize // 4, dtype=torch.int32, device=self.device)
        self.out_host = torch.zeros(self.RING, S.STEPOUT_DTYPE.itemsize // 4, dtype=torch.int32).pin_memory()
        self.barrier = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        # per-step control records: pinned host ring -> device ring, one 32-byte record copied before every launch
        self.ctrl_dev = torch.zeros(self.RING, 8, dtype=torch.int32, device=self.device)
        self.ctrl_host = torch.zeros(self.RING, 8, dtype=torch.int32).pin_memory()
        self.prompt_dev = torch.zeros(self.max_len + 16, dtype=torch.int32, device=self.device)
        self.prompt_host = torch.zeros(self.max_len + 16, dtype=torch.int32).pin_memory()
        inv_freq = cfg.rope_theta ** (-torch.arange(cfg.rotary_dim // 2, dtype=torch.float64) * 2.0 / cfg.rotary_dim)
        self.inv_freq = self._dev(inv_freq)
        nsplit_max = self.num_ctas
        self.attn_part = self._zeros(T8 * cfg.num_attention_heads, nsplit_max, cfg.head_dim + 2)
        self.embed = self._dev(W.matrix("model.embed_tokens.weight", V, H), torch.bfloat16)

        # activation-operand images built by the QUANT phases (largest K = the FFN width, 32-row operand) and the per-GEMV
        # row statistics (sum of squares for the deferred RMS), zeroed at the start of every step
        kmax = max(I, 2 * H, VD, cfg.q_size, *((dc.intermediate_size, dc.q_size) if dc is not None else ()))
        # (two of each: the finishers of GEMV n build GEMV n + 1's operand while other CTAs still read GEMV n's)
        self._b_bytes, self._sfb_bytes = (kmax // 32) * 4 * 128 + 1024, (kmax // 64) * 32 * 16 + 1024
        self.b_image = self._zeros(2 * self._b_bytes, dtype=torch.uint8)
        self.sfb_image = self._zeros(2 * self._sfb_bytes, dtype=torch.uint8)
        self._gemv_count = 0
        self.link_gdn = os.environ.get("PEAR_MK_LINK_GDN", "1") != "0"  # GDN items build the out_proj operand
        self.link_gemvs = os.environ.get("PEAR_MK_LINK", "0") != "0"  # finishers build the next operand (measured: no faster)
        self._links: dict[int, int] = {}  # producer GEMV descriptor -> first tile counter
        self._num_counters = 0
        self.gemv_stats = self._zeros(4096 * 8)
        progs = {"decode": S.Program(self.num_ctas), "prefill": S.Program(self.num_ctas)}
        self.programs = progs
        self._descs: list[dict] = []

        def desc(**f) -> int:
            self._descs.append(f)
            return len(self._descs) - 1

        def both(fn) -> None:
            for p in progs.values():
                p.rotate_save = p.rotate
                fn(p)

        def P(t: torch.Tensor, offset_elems: int = 0) -> int:
            return t.data_ptr() + offset_elems * t.element_size()

        def gemv_desc(packed, gs, K, rows, inp, in_stride, out, out_stride, pro, epi, flags=0, p2=0, p3=0, i8=0, i9=0,
                      eps=cfg.rms_eps):
            img = self._gemv_count & 1
            self._gemv_count += 1
            return desc(p0=P(packed), p1=inp, p2=p2, p3=p3, p4=out, p5=P(self.b_image, img * self._b_bytes),
                        p6=P(self.sfb_image, img * self._sfb_bytes), p7=P(self.gemv_stats, 8 * len(self._descs)), i0=K, i1=K // S.STAGE_K, i2=rows, i3=in_stride,
                        i4=out_stride, i5=pro, i6=epi, i7=flags, i8=i8, i9=i9, f0=1.0 / gs, f1=eps)

        def zero_desc(t: torch.Tensor, flags=0, i8=0) -> int:
            return desc(p4=P(t), i7=flags, i8=i8)

        def add_zero(p: S.Program, zd: int, count: int) -> None:
            p.ranged(S.OP_ZERO, zd, count, granule=4096)

        # ---- embed + zeroing that only depends on the previous step
        d_embed = desc(p0=P(self.embed), p4=P(self.r), i0=H, i4=H)
        z_gu = zero_desc(self.gu)
        z_qkv = zero_desc(self.qkv)
        z_stats = zero_desc(self.gemv_stats)
        both(lambda p: (p.ranged(S.OP_EMBED, d_embed, H, granule=256), add_zero(p, z_stats, 4096 * 8)))

        def G(p: S.Program, d: int, rows: int, K: int, aligned: bool = False, producer: Optional[int] = None) -> None:
            """A GEMV op. Its activation operand is built either by a phase of its own (followed by a grid barrier) or,
            when the input is the output of GEMV ``producer`` (the previous GEMV op), by that op's finishers: the warps
            that deliver the last stream-K contribution to a row tile quantise it in place of a separate phase."""
            if producer is None or not self.link_gemvs:
                p.quant(d, K)
                p.barrier()
            else:
                units = K // 128
                if producer not in self._links:
                    self._links[producer] = self._num_counters
                    self._num_counters += units
                    assert self._descs[d]["p5"] != self._descs[producer]["p5"], "linked GEMVs must use different images"
                    self._descs[producer]["pad"] = (d + 1, self._links[producer])
                base = self._links[producer]
                counts = [0] * units
                for l in p.lists:
                    for ins in l:
                        if ins[0] == S.OP_GEMV and ins[1] == producer:
                            counts[ins[2] % units] += 1
                assert min(counts) > 0
                p.expect.extend([0] * (base + units - len(p.expect)))
                p.expect[base:base + units] = counts
            p.gemv(d, rows, K, aligned)

        # drafter buffers (zeroed during the target's first phase)
        if dc is not None:
            DH, DI = dc.hidden_size, dc.intermediate_size
            assert DH == H
            self.d_qkv_stride = dc.q_size + 2 * dc.kv_size
            self.fc_in = self._zeros(T8, 2 * H)
            self.rd = self._zeros(T8, H)
            self.dgu = self._zeros(T8, 2 * DI)
            self.dqkv = self._zeros(T8, self.d_qkv_stride)
            self.dattn_out = self._zeros(T8, dc.q_size)
            self.dlogits = self._zeros(T8, V)
            self.argmax_part = self._zeros(4, nchunks, 2)
            self.dattn_part = self._zeros(T8 * dc.num_attention_heads, nsplit_max, dc.head_dim + 2)
            z_rd, z_dgu, z_dqkv = zero_desc(self.rd), zero_desc(self.dgu), zero_desc(self.dqkv)
            both(lambda p: (add_zero(p, z_rd, T8 * H), add_zero(p, z_dgu, T8 * 2 * DI),
                            add_zero(p, z_dqkv, T8 * self.d_qkv_stride)))
        both(lambda p: p.barrier())

        # ---- layers
        self.gdn_state, self.gdn_conv, self.gdn_rec, self.kcache, self.vcache = {}, {}, {}, {}, {}

        def mlp_block(prefix: str, r_buf, gu_buf, z_gu_desc, icfg: HybridConfig, flags: int, lname: str):
            Hh, Ii = icfg.hidden_size, icfg.intermediate_size
            post_w = self._dev(W.vector(f"{prefix}.post_attention_layernorm.weight", Hh))
            wg = W.matrix(f"{prefix}.mlp.gate_proj.weight", Ii, Hh)
            wu = W.matrix(f"{prefix}.mlp.up_proj.weight", Ii, Hh)
            pk, gs = self._pack(torch.cat([wg, wu], dim=0))
            del wg, wu
            d_gu = gemv_desc(pk, gs, Hh, 2 * Ii, P(r_buf), Hh, P(gu_buf), 2 * Ii, S.PRO_NORM, S.EPI_RED, flags, p2=P(post_w))
            pk2, gs2 = self._pack(W.matrix(f"{prefix}.mlp.down_proj.weight", Hh, Ii))
            d_dn = gemv_desc(pk2, gs2, Ii, Hh, P(gu_buf), 2 * Ii, P(r_buf), Hh, S.PRO_SWIGLU, S.EPI_RED, flags)
            return d_gu, d_dn, 2 * Ii, Ii

        def attn_block(prefix: str, li, icfg: HybridConfig, r_buf, qkv_buf, qkv_stride, aout_buf, part_buf, flags: int):
            Hh, D, Hq, Hkv = icfg.hidden_size, icfg.head_dim, icfg.num_attention_heads, icfg.num_kv_heads
            in_w = self._dev(W.vector(f"{prefix}.input_layernorm.weight", Hh))
            qrows = (2 if icfg.attn_output_gate else 1) * icfg.q_size
            wq = W.matrix(f"{prefix}.self_attn.q_proj.weight", qrows, Hh)
            wk = W.matrix(f"{prefix}.self_attn.k_proj.weight", icfg.kv_size, Hh)
            wv = W.matrix(f"{prefix}.self_attn.v_proj.weight", icfg.kv_size, Hh)
            pk, gs = self._pack(torch.cat([wq, wk, wv], dim=0))
            del wq, wk, wv
            rows = qrows + 2 * icfg.kv_size
            d_in = gemv_desc(pk, gs, Hh, rows, P(r_buf), Hh, P(qkv_buf), qkv_stride, S.PRO_NORM, S.EPI_RED, flags, p2=P(in_w))
            qk_norm = self._dev(torch.cat([W.vector(f"{prefix}.self_attn.q_norm.weight", D),
                                           W.vector(f"{prefix}.self_attn.k_norm.weight", D)]))
            kc = self._zeros(self.max_len + 16, Hkv, D, dtype=torch.bfloat16)
            vc = self._zeros(self.max_len + 16, Hkv, D, dtype=torch.bfloat16)
            self.kcache[li], self.vcache[li] = kc, vc
            d_at = desc(p0=P(qkv_buf), p1=P(kc), p2=P(vc), p3=P(qk_norm), p4=P(part_buf), p5=P(self.inv_freq), p6=P(aout_buf),
                        i0=qkv_stride, i1=Hkv, i2=Hq, i3=D, i4=nsplit_max, i5=icfg.rotary_dim, i6=16, i7=flags,
                        i9=1 if icfg.attn_output_gate else 0, f0=D ** -0.5, f1=icfg.rms_eps)
            pk2, gs2 = self._pack(W.matrix(f"{prefix}.self_attn.o_proj.weight", Hh, icfg.q_size))
            d_out = gemv_desc(pk2, gs2, icfg.q_size, Hh, P(aout_buf), icfg.q_size, P(r_buf), Hh, S.PRO_PLAIN, S.EPI_RED, flags)
            return d_in, rows, d_at, d_out

        def emit_attn(p: S.Program, icfg, d_in, rows, d_at, d_out, z_qkv_desc, qkv_elems, pre=None, producer=None):
            Hq, Hkv = icfg.num_attention_heads, icfg.num_kv_heads
            nsplit = self.attn_splits or max(1, self.num_ctas // Hkv)
            if pre is not None:
                pre(p)
            G(p, d_in, rows, icfg.hidden_size, producer=producer)
            p.barrier()
            p.spread(S.OP_ATTN, d_at, [(h, s, nsplit) for s in range(nsplit) for h in range(Hkv)])
            p.barrier()
            npairs = T8 * Hq
            per = max(1, (npairs + p.num_ctas - 1) // p.num_ctas)
            p.spread(S.OP_ATTN_COMBINE, d_at, [(a, min(per, npairs - a), nsplit) for a in range(0, npairs, per)])
            p.barrier()
            G(p, d_out, icfg.hidden_size, icfg.q_size)
            add_zero(p, z_qkv_desc, qkv_elems)
            p.barrier()

        def emit_mlp(p: S.Program, d_out, d_gu, d_dn, gu_rows, ii, hh):
            G(p, d_gu, gu_rows, hh, producer=d_out)
            p.barrier()
            G(p, d_dn, hh, ii, producer=d_gu)
            p.barrier()

        prev_dn = None  # the previous layer's down projection: its finishers build this layer's first operand
        for li, lt in enumerate(cfg.layer_types):
            prefix = f"model.layers.{li}"
            if lt == "linear_attention":
                in_w = self._dev(W.vector(f"{prefix}.input_layernorm.weight", H))
                wcat = torch.cat([W.matrix(f"{prefix}.linear_attn.in_proj_qkv.weight", C, H),
                                  W.matrix(f"{prefix}.linear_attn.in_proj_z.weight", VD, H),
                                  W.matrix(f"{prefix}.linear_attn.in_proj_b.weight", HV, H),
                                  W.matrix(f"{prefix}.linear_attn.in_proj_a.weight", HV, H)], dim=0)
                pk, gs = self._pack(wcat)
                del wcat
                recbuf = self._zeros(2, T8, self.rec_stride)
                par_stride = T8 * self.rec_stride
                self.gdn_rec[li] = recbuf
                d_in = gemv_desc(pk, gs, H, C + VD + 2 * HV, P(self.r), H, P(recbuf), self.rec_stride, S.PRO_NORM, S.EPI_RED,
                                 S.F_OUT_PARITY, p2=P(in_w), i8=par_stride)
                conv_w = self._dev(W.matrix(f"{prefix}.linear_attn.conv1d.weight", C, cfg.conv_kernel))
                gates = self._dev(torch.cat([W.vector(f"{prefix}.linear_attn.A_log", HV),
                                             W.vector(f"{prefix}.linear_attn.dt_bias", HV)]))
                state = self._zeros(HV, 128, 128)
                conv = self._zeros(2, 3, C)
                self.gdn_state[li], self.gdn_conv[li] = state, conv
                d_core = desc(p0=P(recbuf), p2=P(conv_w), p3=P(gates), p4=P(state), p5=P(conv), p6=P(self.gdn_o),
                              i0=self.rec_stride, i1=HV, i2=HK, i3=C, i4=VD, i8=par_stride, f1=cfg.l2_eps)
                norm_w = self._dev(W.vector(f"{prefix}.linear_attn.norm.weight", 128))
                pk2, gs2 = self._pack(W.matrix(f"{prefix}.linear_attn.out_proj.weight", H, VD))
                d_out = gemv_desc(pk2, gs2, VD, H, P(self.gdn_o), VD, P(self.r), H, S.PRO_GDN_NORM, S.EPI_RED, S.F_IN_PARITY,
                                  p2=P(recbuf, C), p3=P(norm_w), i8=par_stride, i9=self.rec_stride)
                z_rec = zero_desc(recbuf, S.F_OUT_OTHER_PARITY, par_stride)
                # value-head rows split so that Hv * parts covers the CTAs (144 items of 42-43 rows at 48 heads)
                parts = max(1, min(4, self.num_ctas // HV))
                items = []
                for hv in range(HV):
                    for k in range(parts):
                        lo, hi = 128 * k // parts, 128 * (k + 1) // parts
                        items.append((hv, lo, hi - lo))
                d_gu, d_dn, gu_rows, ii = mlp_block(prefix, self.r, self.gu, z_gu, cfg, 0, lt)

                def emit(p: S.Program, d_in=d_in, d_core=d_core, d_out=d_out, z_rec=z_rec, items=items, d_gu=d_gu, d_dn=d_dn,
                         gu_rows=gu_rows, ii=ii, prev_dn=prev_dn):
                    G(p, d_in, C + VD + 2 * HV, H, producer=prev_dn)
                    add_zero(p, z_gu, T8 * 2 * I)
                    p.barrier()
                    p.spread(S.OP_GDN, d_core, items)
                    p.barrier()
                    if self.link_gdn:
                        # the GDN item that completes a value head builds that head's unit of the out_proj operand
                        if d_core not in self._links:
                            self._links[d_core] = self._num_counters
                            self._num_counters += HV
                            self._descs[d_core]["pad"] = (d_out + 1, self._links[d_core])
                        base = self._links[d_core]
                        p.expect.extend([0] * (base + HV - len(p.expect)))
                        p.expect[base:base + HV] = [sum(1 for it in items if it[0] == hv) for hv in range(HV)]
                        p.gemv(d_out, H, VD)
                    else:
                        G(p, d_out, H, VD)
                    add_zero(p, z_rec, T8 * self.rec_stride)
                    p.barrier()
                    emit_mlp(p, d_out, d_gu, d_dn, gu_rows, ii, H)

                both(emit)
            else:
                d_in, rows, d_at, d_out = attn_block(prefix, li, cfg, self.r, self.qkv, self.qkv_stride, self.attn_out,
                                                     self.attn_part, 0)
                d_gu, d_dn, gu_rows, ii = mlp_block(prefix, self.r, self.gu, z_gu, cfg, 0, lt)

                def emit(p: S.Program, d_in=d_in, rows=rows, d_at=d_at, d_out=d_out, d_gu=d_gu, d_dn=d_dn, gu_rows=gu_rows, ii=ii,
                         prev_dn=prev_dn):
                    emit_attn(p, cfg, d_in, rows, d_at, d_out, z_qkv, T8 * self.qkv_stride,
                              pre=lambda q: add_zero(q, z_gu, T8 * 2 * I), producer=prev_dn)
                    emit_mlp(p, d_out, d_gu, d_dn, gu_rows, ii, H)

                both(emit)
            prev_dn = d_dn

        # ---- head + sampler (decode) / bookkeeping (prefill)
        fin_w = self._dev(W.vector("model.norm.weight", H))
        pk, gs = self._pack(W.matrix("lm_head.weight", V, H))
        self._lm_head = (pk, gs)
        d_head = gemv_desc(pk, gs, H, V, P(self.r), H, P(self.logits), V, S.PRO_NORM, S.EPI_STORE, 0, p2=P(fin_w))
        d_samp = desc(p0=P(self.logits), p1=P(self.prompt_dev), p4=P(self.sample_part), i0=V, i1=V, i2=self.CHUNK, i3=nchunks,
                      i4=self.n_draft, i5=0, i6=0, i9=self.mask_token_id)
        d_book = desc(p1=P(self.prompt_dev), i4=self.n_draft, i5=0, i6=1, i9=self.mask_token_id)
        self._d_samp, self._d_book = d_samp, d_book
        dp, pp = progs["decode"], progs["prefill"]
        G(dp, d_head, V, H, aligned=True, producer=prev_dn)
        dp.barrier()
        dp.ranged(S.OP_SAMPLE_PART, d_samp, nchunks)
        dp.barrier()
        dp.emit(0, S.OP_SAMPLE_FIN, d_samp)
        pp.emit(0, S.OP_SAMPLE_FIN, d_book)
        both(lambda p: p.barrier())

        # ---- drafter
        if dc is not None:
            nw = self._dev(torch.cat([W.vector("draft.pre_fc_norm_embedding.weight", H),
                                      W.vector("draft.pre_fc_norm_hidden.weight", H)]))
            d_din = desc(p0=P(self.embed), p1=P(self.r), p2=P(nw), p4=P(self.fc_in), p5=P(self.prompt_dev), i0=H, i3=H,
                         i5=self.mask_token_id, i6=0, f1=dc.rms_eps)
            d_din_pre = desc(p0=P(self.embed), p1=P(self.r), p2=P(nw), p4=P(self.fc_in), p5=P(self.prompt_dev), i0=H, i3=H,
                             i5=self.mask_token_id, i6=1, f1=dc.rms_eps)
            pk, gs = self._pack(W.matrix("draft.fc.weight", H, 2 * H))
            d_fc = gemv_desc(pk, gs, 2 * H, H, P(self.fc_in), 2 * H, P(self.rd), H, S.PRO_PLAIN, S.EPI_RED, S.F_DRAFT_ROWS)
            dp.spread(S.OP_DRAFT_IN, d_din, [(j,) for j in range(T8)])
            pp.spread(S.OP_DRAFT_IN, d_din_pre, [(j,) for j in range(T8)])
            both(lambda p: p.barrier())
            both(lambda p: (G(p, d_fc, H, 2 * H), p.barrier()))
            prev_dn = d_fc
            for li in range(dc.num_layers):
                prefix = f"draft.layers.{li}"
                d_in, rows, d_at, d_out = attn_block(prefix, ("draft", li), dc, self.rd, self.dqkv, self.d_qkv_stride,
                                                     self.dattn_out, self.dattn_part, S.F_DRAFT_ROWS)
                d_gu, d_dn, gu_rows, ii = mlp_block(prefix, self.rd, self.dgu, None, dc, S.F_DRAFT_ROWS, "draft")
                z_dgu2 = zero_desc(self.dgu)

                def emit(p: S.Program, d_in=d_in, rows=rows, d_at=d_at, d_out=d_out, d_gu=d_gu, d_dn=d_dn, gu_rows=gu_rows,
                         ii=ii, li=li, z_dgu2=z_dgu2, prev_dn=prev_dn):
                    emit_attn(p, dc, d_in, rows, d_at, d_out, z_dqkv, T8 * self.d_qkv_stride,
                              pre=(lambda q: add_zero(q, z_dgu2, T8 * 2 * dc.intermediate_size)) if li > 0 else None,
                              producer=prev_dn)
                    emit_mlp(p, d_out, d_gu, d_dn, gu_rows, ii, dc.hidden_size)

                both(emit)
                prev_dn = d_dn
            dfin_w = self._dev(W.vector("draft.norm.weight", H))
            pk, gs = self._lm_head
            d_dhead = gemv_desc(pk, gs, H, V, P(self.rd), H, P(self.dlogits), V, S.PRO_NORM, S.EPI_STORE, S.F_DRAFT_ROWS,
                                p2=P(dfin_w))
            d_arg = desc(p0=P(self.dlogits), p4=P(self.argmax_part), i0=V, i1=V, i2=self.CHUNK, i3=nchunks, i4=self.n_draft)
            if self.n_draft > 0:
                G(dp, d_dhead, V, H, aligned=True, producer=prev_dn)
                dp.barrier()
                dp.ranged(S.OP_ARGMAX_PART, d_arg, nchunks)
                dp.barrier()
                dp.emit(0, S.OP_ARGMAX_FIN, d_arg)

        # ---- finalise: one descriptor table, two instruction arrays
        self._prog_dev = {}
        for name, p in progs.items():
            p.descs = self._descs
            instrs, descs, max_len = p.finalize()
            self._prog_dev[name] = (torch.from_numpy(instrs.view(np.int32).reshape(self.num_ctas, max_len * 8).copy()).to(self.device),
                                    max_len, p.stats())
        self.tile_cnt = torch.zeros(max(1, self._num_counters), dtype=torch.int32, device=self.device)
        self._expect_dev = {}
        for name, p in progs.items():
            e = list(p.expect) + [0] * (max(1, self._num_counters) - len(p.expect))
            self._expect_dev[name] = torch.tensor(e, dtype=torch.int32, device=self.device)
        self._descs_np = descs
        self.descs_dev = torch.from_numpy(descs.view(np.uint8).reshape(-1).copy()).to(self.device)
        self.smem_bytes = {k: _lib.lib().pear_mk_smem_bytes(*v) for k, v in self.LAUNCH_SHAPE.items()}

    # -- descriptor patching (prompt length lives in the sampler/bookkeeping descriptors) -------------------------------
    def _set_prompt_len(self, n: int) -> None:
        for d in (self._d_samp, self._d_book):
            self._descs_np[d]["i5"] = n
        self.descs_dev.copy_(torch.from_numpy(self._descs_np.view(np.uint8).reshape(-1).copy()))

    # -- sequence state ----------------------------------------------------------------------------------------------
    def reset(self) -> None:
        for group in (self.gdn_state, self.gdn_conv, self.gdn_rec):
            for t in group.values():
                t.zero_()
        for t in (self.qkv, self.gu, self.rec, self.out_ring, self.status):
            t.zero_()
        if self.draft_cfg is not None:
            for t in (self.rd, self.dgu, self.dqkv):
                t.zero_()
        self.step = 0
        self.prompt_len = 0

    def start(self, prompt: list[int] | torch.Tensor) -> None:
        """Copy the prompt from pinned host memory and write the first step record."""
        self.reset()
        p = torch.as_tensor(prompt, dtype=torch.int32).flatten()
        n = int(p.numel())
        assert 1 <= n <= self.max_len - 16 * (1 + self.n_draft)
        self.prompt_len = n
        self.prompt_host[:n].copy_(p)
        self.prompt_dev[:n].copy_(self.prompt_host[:n], non_blocking=True)
        self._set_prompt_len(n)
        rec = np.zeros((2, S.STEPREC_INTS), dtype=np.int32)
        if n > 1:
            t0 = min(8, n - 1)
            rec[0, 0], rec[0, 5] = t0, 1
            rec[0, 8 : 8 + t0] = p[:t0].numpy()
        else:
            rec[0, 0], rec[0, 5] = 1, 0
            rec[0, 8] = int(p[0])
        self.rec.copy_(torch.from_numpy(rec))
        self.prefill_steps = (n - 1 + 7) // 8

    def _launch(self, program: str) -> None:
        instrs, max_len, stats = self._prog_dev[program]
        prm = _Params(
            instrs=instrs.data_ptr(), descs=self.descs_dev.data_ptr(), rec=self.rec.data_ptr(), out_ring=self.out_ring.data_ptr(),
            barrier=self.barrier.data_ptr(), status=self.status.data_ptr(), max_instrs=max_len, ring=self.RING,
            step_parity=self.step & 1, seed=self.seed, temperature=self.temperature, vocab=self.cfg.vocab_size,
            barrier_base=self.barrier_base & 0xFFFFFFFF, pad=int(os.environ.get("PEAR_MK_DEBUG", "0")), l2_ahead=self.l2_ahead, tile_cnt=self.tile_cnt.data_ptr(),
            tile_expect=self._expect_dev[program].data_ptr(),
            ctrl=self.ctrl_dev[self.step % self.RING].data_ptr() if self._use_ctrl else 0,
            trace=self._trace.data_ptr() if self._trace is not None else 0, trace_ctas=self._trace_ctas, trace_cap=self._trace_cap)
        ns, nb = self.LAUNCH_SHAPE[program]
        code = _lib.lib().pear_mk_launch(ctypes.byref(prm), self.num_ctas, ns, nb, _lib.stream())
        _lib.check(code, "megakernel launch")
        _lib.count_launch()
        self.barrier_base += stats["barriers"] * self.num_ctas
        self.step += 1
        self.launches += 1

    # -- in-kernel tracing ------------------------------------------------------------------------------------------------
    def enable_trace(self, ctas: int = 2, cap: int = 8192) -> None:
        """Timeline of the next launches: thread 0 of the first ``ctas`` CTAs records (mark, instruction, globaltimer)."""
        self._trace = torch.zeros(3 * ctas * cap * 2, dtype=torch.int64, device=self.device)
        self._trace_ctas, self._trace_cap = ctas, cap

    def read_trace(self, program: str = "decode", issuer: int = 0, clear: bool = True) -> list[list[tuple[int, int, int, int]]]:
        """Per traced CTA: (mark id, instruction index, opcode, nanoseconds since the earliest record of any CTA)."""
        full = self._trace.cpu().numpy().reshape(self._trace_ctas, 3, self._trace_cap, 2)
        t0 = min(int(full[c, w, 1, 1]) for c in range(self._trace_ctas) for w in range(3) if int(full[c, w, 0, 0]) > 0)
        t = full[:, int(issuer)]
        instrs = self._prog_dev[program][0].cpu().numpy().reshape(self.num_ctas, -1, 8)
        out = []
        for c in range(self._trace_ctas):
            n = int(t[c, 0, 0])
            recs = []
            for i in range(1, n + 1):
                word, ts = int(t[c, i, 0]), int(t[c, i, 1])
                ip = word & 0xFFFFFFFF
                op = int(instrs[c, ip, 0]) if ip < instrs.shape[1] else -1
                recs.append((word >> 32, ip, op, ts - t0))
            out.append(recs)
        if clear:
            self._trace.zero_()
        return out

    def prefill(self) -> None:
        for _ in range(self.prefill_steps):
            self._launch("prefill")

    def decode_step(self, copy_out: bool = True, temperature: Optional[float] = None, seed: Optional[int] = None) -> int:
        """Launch one decode/verify step; returns the ring slot its output lands in. The step's sampling controls
        travel host -> device in a 32-byte record copied from pinned memory ahead of the launch."""
        slot = (self.step) % self.RING
        if self._use_ctrl:
            rec = self.ctrl_host[slot]
            rec[0] = int(np.float32(self.temperature if temperature is None else temperature).view(np.int32))
            rec[1] = int(np.uint32(self.seed if seed is None else seed).view(np.int32))
            rec[2] = -1
            self.ctrl_dev[slot].copy_(rec, non_blocking=True)
        self._launch("decode")
        if copy_out:
            self.out_host[slot].copy_(self.out_ring[slot], non_blocking=True)
        return slot

    def check_status(self) -> None:
        st = int(self.status[0].item())
        if st != 0:
            raise RuntimeError(f"megakernel reported status {st} (1 mbarrier timeout, 2 grid barrier, 3 flag, 4 bad instr)")

    def read_slot(self, slot: int) -> dict:
        a = self.out_host[slot].numpy().view(S.STEPOUT_DTYPE)[0]
        return {"step": int(a["step"]), "n_out": int(a["n_out"]), "n_accept": int(a["n_accept"]), "pos0": int(a["pos0"]),
                "tokens": [int(x) for x in a["tokens"][: int(a["n_out"])]], "logprob": float(a["logprobs"][0])}

    def generate(self, prompt, max_new_tokens: int, lookahead: int = 2) -> GenerationResult:
        """Public entry: prefill ``prompt`` then decode until ``max_new_tokens`` tokens were emitted. The host reads
        each step's output from pinned memory, ``lookahead`` launches behind the device."""
        self.start(prompt)
        self.prefill()
        budget = self.max_len - 16 * (1 + self.n_draft) - self.prompt_len
        res = self.decode(min(max_new_tokens, budget), lookahead=lookahead)
        self.check_status()
        return res

    def decode(self, count: int, by_steps: bool = False, lookahead: int = 2) -> GenerationResult:
        """Continue the current sequence until ``count`` tokens were emitted (or for exactly ``count`` launches with
        ``by_steps``). Per step: a control record goes pinned host -> device, the step is launched, its output slot
        is copied device -> pinned host, and the host reads the emitted tokens ``lookahead`` launches behind."""
        tokens: list[int] = []
        pending: list[tuple[int, torch.cuda.Event]] = []
        steps = launched = accepted = 0
        while (steps < count) if by_steps else (len(tokens) < count):
            while len(pending) < lookahead and launched < count:
                slot = self.decode_step()
                ev = torch.cuda.Event()
                ev.record()
                pending.append((slot, ev))
                launched += 1
            slot, ev = pending.pop(0)
            ev.synchronize()
            out = self.read_slot(slot)
            tokens.extend(out["tokens"])
            accepted += out["n_accept"]
            steps += 1
        for slot, ev in pending:
            ev.synchronize()
        return GenerationResult(tokens if by_steps else tokens[:count], steps, accepted, getattr(self, "prefill_steps", 0))

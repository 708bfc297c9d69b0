"""The batched, GPU-resident decode / speculative-verify step of the rollout engine.

One step advances every sequence of the batch by ``1 + accepted drafts`` tokens with a fixed sequence of kernel launches
over fixed buffers: embedding, per layer [RMSNorm -> weight-streaming GEMM -> (paged tensor-core attention | GDN verify
core under the replay scheme) -> row-parallel GEMM -> (all-reduce +) residual add + RMSNorm -> SwiGLU GEMM -> down GEMM],
vocabulary-sharded lm_head, the sharded rejection sampler with in-kernel Philox, and the MTP drafter's passes that write
the next step's draft tokens. Context lengths, replay counts, record parities and input tokens live on the device and are
updated by the step itself, so after warm-up the step is replayed as ONE CUDA graph and the host only reads the small
result record (tokens, accepted counts) when it wants to.

Upstream reaches the same shape through vLLM's V2 runner with per-size CUDA graphs, its Blackwell kernels and a Python
speculator (``pear/models/qwen3_5/rollout/blackwell/{model,cudagraph,mtp}.py``, ``rollout/speculator.py``); here it is one
object owning its buffers. Tensor parallelism: heads / FFN columns / vocabulary are sharded over the ranks of a
``SymmWorld``; row-parallel partials are reduced by the fused NVSwitch all-reduce + add + RMSNorm kernel with its epoch in
device memory (graph-replayable), the sampler exchanges 32-byte records instead of logits.

The recurrent state follows the replay scheme (``ops/csrc/decode_step.cu: ds_gdn_verify_kernel``): ``rec_state`` is shared
with the prefill runner, the conv window travels in the block record.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..models.hybrid import HybridForCausalLM
from ..ops import decode_ops as K
from ..ops import lib as _lib
from ..ops import rollout_ops
from ..utils import nvtx

SLOT_STEP_AR, SLOT_STEP_SYNC = 8, 10  # flag slots of the SymmWorld signal region used by the step (the two-shot reduction also uses 9)


@dataclass
class StepResult:
    tokens: torch.Tensor  # [B, T] int32 on the host, -1 after the last emitted token of a sequence
    accepted: torch.Tensor  # [B] int32
    logprobs: torch.Tensor  # [B, T] fp32
    nonfinite: torch.Tensor  # [B] int32
    topk_ids: Optional[torch.Tensor] = None  # [B, T, 32] int32 when the decoder was built with ``topk_logprobs``
    topk_logprobs: Optional[torch.Tensor] = None  # [B, T, 32] fp32, descending


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.bfloat16).contiguous()


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().float().contiguous()


class _Mixer:
    pass


class FastDecoder:
    """``model``: this rank's (tensor-parallel shard of the) hybrid model on the GPU. ``k_cache`` / ``v_cache`` (dict layer ->
    [pages, 16, Hkv, D] bf16), ``rec_state`` (dict layer -> [slots, Hv, 128, 128] fp32) and the drafter's caches are the
    prefill runner's tensors. ``vocab_shard``: (first row, rows) of lm_head this rank owns."""

    def __init__(self, model: HybridForCausalLM, k_cache: dict, v_cache: dict, rec_state: dict, mtp_k: list, mtp_v: list, num_slots: int,
                 max_batch: int, n_draft: int, max_blocks_per_seq: int, temperature: float = 1.0, seed: int = 0, symm=None,
                 share_weights: bool = True, use_graph: bool = True, tensor_core_attention: Optional[bool] = None, ar_mode: str = "auto",
                 topk_logprobs: bool = False):
        cfg = model.config
        self.model, self.cfg = model, cfg
        dev = next(model.parameters()).device
        self.dev = dev
        self.B, self.T, self.n_draft = max_batch, 1 + n_draft, n_draft
        self.M = self.B * self.T
        self.symm = symm
        self.world = symm.world if symm is not None else 1
        self.rank = symm.rank if symm is not None else 0
        self.temperature, self.seed = float(temperature), int(seed) & 0xFFFFFFFF
        self.use_graph, self.graph, self._warm = use_graph, None, 0
        self.tc_attn = tensor_core_attention
        # "one": one-shot pull, "two": two-shot (reduce-scatter + all-gather) over peer loads / stores, "nvls": the two-shot form
        # with the sum and the broadcast done by the switch (multimem), "auto": by rows and ranks
        self.ar_mode = ar_mode
        self.nvls_auto = False
        self.topk = bool(topk_logprobs)  # every step also produces the 32 largest log-probs of every row (what score centering reads)
        if cfg.gdn_head_dim != 128 and cfg.gdn_layers:
            raise ValueError("the GDN verify kernel is built for head dimension 128")
        if model.mtp is None and n_draft > 0:
            raise ValueError("speculative drafts need the MTP head")
        self.k_cache, self.v_cache, self.rec_state, self.mtp_k, self.mtp_v = k_cache, v_cache, rec_state, mtp_k, mtp_v
        H, M, B, T = cfg.hidden_size, self.M, self.B, self.T
        self.H = H
        self.sms = K.num_sms(dev)
        self.status = K.status_word(dev)
        self.share_weights = share_weights
        V = cfg.vocab_size
        if V % self.world or (V // self.world) % 4:
            raise ValueError("vocabulary size must split into shards that are multiples of 4")
        self.Vs, self.v0 = V // self.world, self.rank * (V // self.world)
        self.repack()
        half = cfg.rotary_dim // 2
        self.inv_freq = (cfg.rope_theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / cfg.rotary_dim)).to(dev)
        # ---- device-resident step state
        i32 = dict(dtype=torch.int32, device=dev)
        self.ctx = torch.full((B,), -1, **i32)
        self.slots = torch.zeros(B, **i32)
        self.parity = torch.zeros(B, **i32)
        self.ncommit = torch.zeros(B, **i32)
        self.rope_off = torch.zeros(B, **i32)
        self.tok_in = torch.zeros(M, **i32)
        self.block_table = torch.zeros(B, max_blocks_per_seq, **i32)
        self.step_ctr = torch.zeros(1, **i32)
        self.out_tok = torch.full((B, T), -1, **i32)
        self.out_lp = torch.zeros(B, T, dtype=torch.float32, device=dev)
        self.n_accept = torch.zeros(B, **i32)
        self.nonfinite = torch.zeros(B, **i32)
        self.sel_row = torch.zeros(B, **i32)
        self.mtp_tok = torch.zeros(M, **i32)
        self.mtp_ctx = torch.full((T, B), -1, **i32)
        self.draft_tok = torch.zeros(B, **i32)
        # GDN block records (conv window + block rows, (a, b) rows), two copies per slot
        self.conv_rec, self.ab_rec = {}, {}
        for li in cfg.gdn_layers:
            self.conv_rec[li] = torch.zeros(num_slots, 2, 3 + T, self._gdn_dims()[2], dtype=torch.float32, device=dev)
            self.ab_rec[li] = torch.zeros(num_slots, 2, T, 2 * cfg.gdn_v_heads, dtype=torch.float32, device=dev)
        # ---- workspaces
        f32, b16 = dict(dtype=torch.float32, device=dev), dict(dtype=torch.bfloat16, device=dev)
        if self.world > 1:  # symmetric: the two-shot reduction stores rows into every rank's copies
            self.h_sym, self.x_sym = symm.alloc((M, H), torch.bfloat16), symm.alloc((M, H), torch.float32)
            self.h, self.x_res = self.h_sym.tensor, self.x_sym.tensor
            self.h.zero_()
            self.x_res.zero_()
        else:
            self.x_res = torch.zeros(M, H, **f32)
            self.h = torch.zeros(M, H, **b16)
        n_in = 0
        for lw in self.layers + (self.mtp.layers if self.mtp else []):
            n_in = max(n_in, lw.w_in.shape[0])
        self.proj = torch.zeros(M, (n_in + 3) // 4 * 4, **f32)
        self.q = torch.zeros(M, max(1, cfg.num_attention_heads) * cfg.head_dim, **b16)
        self.mix_out = torch.zeros(M, max(cfg.q_size, cfg.gdn_value_dim), **b16)
        self.act = torch.zeros(M, cfg.intermediate_size, **b16)
        self.max_split = 8
        self.parts = torch.zeros(self.max_split, M, H, **f32)
        self.logits = torch.zeros(M, (self.Vs + 3) // 4 * 4, **f32)
        self.chunks = max(1, min(16, (2 * self.sms) // max(1, M)))
        self.achunks = max(1, min(32, (2 * self.sms) // max(1, B)))
        rec_elems = self.world * M * self.chunks
        key_elems = self.world * B * self.achunks
        self.rec_buf_elems, self.key_buf_elems = rec_elems, key_elems
        if self.topk:
            if self.world * self.chunks * K.TOPK > 1024:
                self.chunks = max(1, 1024 // (self.world * K.TOPK))  # the merge sorts world x chunks lists of 32 in one CTA
                rec_elems = self.world * M * self.chunks
                self.rec_buf_elems = rec_elems
            self.top_ids = torch.zeros(M, K.TOPK, **i32)
            self.top_lp = torch.zeros(M, K.TOPK, **f32)
        if self.mtp:
            self.xcat = torch.zeros(M, 2 * H, **b16)
            if self.world > 1:
                self.r_sym = symm.alloc((M, H), torch.float32)
                self.r_mtp = self.r_sym.tensor
                self.r_mtp.zero_()
            else:
                self.r_mtp = torch.zeros(M, H, **f32)
            self.r_sel = torch.zeros(B, H, **f32)
            self.r_sel2 = torch.zeros(B, H, **f32)
            self.h_sel = torch.zeros(B, H, **b16)
        if self.world > 1:
            s = symm
            self.ar_ws = s.alloc((3, M, H), torch.bfloat16)  # two buffers by epoch parity + one the GEMMs write straight into
            if self.ar_mode == "nvls" and not self.nvls_available():
                raise RuntimeError("ar_mode 'nvls': the symmetric buffers have no multicast address on this platform")
            # measured at 128 rows per step: switch-side sum and broadcast 24.7 ms against 25.1 ms per step at 8 ranks, no
            # difference at 4, slightly behind at 2 (the two flag exchanges of a reduction, not its bytes, are most of its cost)
            self.nvls_auto = self.ar_mode == "auto" and self.world >= 8 and self.nvls_available()
            self.recs = s.alloc((2 * rec_elems * K.rec_bytes(),), torch.uint8)
            self.keys = s.alloc((2 * key_elems,), torch.int64)
            self.ar_ctr = s.device_counter(SLOT_STEP_AR)  # shared by every decoder on this SymmWorld: one epoch sequence per slot
            self.ar_ticket = torch.zeros(1, **i32)
            self.sync_ctr = s.device_counter(SLOT_STEP_SYNC)
            self.recs_ptrs, self.keys_ptrs = self.recs.c_ptrs, self.keys.c_ptrs
            self.recs_t, self.keys_t = self.recs.tensor, self.keys.tensor
            self.recs_t.zero_()
            self.keys_t.zero_()
            if self.topk:
                self.tops = s.alloc((2 * rec_elems * K.top_bytes(),), torch.uint8)
                self.tops_ptrs, self.tops_t = self.tops.c_ptrs, self.tops.tensor
                self.tops_t.zero_()
            torch.cuda.synchronize(dev)
            import torch.distributed as dist

            dist.barrier(s.group)
        else:
            self.recs_t = torch.zeros(rec_elems * K.rec_bytes(), dtype=torch.uint8, device=dev)
            self.keys_t = torch.zeros(key_elems, dtype=torch.int64, device=dev)
            self.recs_ptrs = K._ptr_array([self.recs_t.data_ptr()])
            self.keys_ptrs = K._ptr_array([self.keys_t.data_ptr()])
            self.ar_ctr = self.sync_ctr = None
            if self.topk:
                self.tops_t = torch.zeros(rec_elems * K.top_bytes(), dtype=torch.uint8, device=dev)
                self.tops_ptrs = K._ptr_array([self.tops_t.data_ptr()])
        # work table of the tensor-core paged attention: per sequence one item over the keys it does not share, per group
        # of sequences with a common prefix a few items over the shared keys (set_shared_prefixes)
        self.pa_items = None
        if cfg.attention_layers or self.mtp:
            hq, hkv = cfg.num_attention_heads, cfg.num_kv_heads
            if tensor_core_attention is not False and K.tc_attention_ok(cfg.head_dim, hq, hkv, T):
                self.pa_splits = 8  # most items a shared prefix is cut into
                self.pa_nparts = 1 + self.pa_splits
                self.pa_group = max(1, min(K.PA_ITEM_SEQS, 128 // ((hq // hkv) * T)))
                self.pa_items = torch.zeros(B + (B // 2 + 1) * self.pa_splits, K.PA_ITEM_INTS, **i32)
                self.pa_part_o = torch.zeros(self.pa_nparts, M, hq, cfg.head_dim, **f32)
                self.pa_part_ml = torch.zeros(self.pa_nparts, M, hq, 2, **f32)
                self.set_shared_prefixes([])
        # pinned result record
        self._host = torch.zeros(B * (2 * T + 2), dtype=torch.int32).pin_memory()
        if self.topk:
            self._host_top_ids = torch.zeros(M, K.TOPK, dtype=torch.int32).pin_memory()
            self._host_top_lp = torch.zeros(M, K.TOPK, dtype=torch.float32).pin_memory()
        self._dev_rec = torch.zeros(B * (2 * T + 2), **i32)
        self.steps = 0
        self.debug_logits = None  # tests: a [M, Vs] tensor that receives the verify rows' logits before the drafter reuses the buffer

    # -- weights ------------------------------------------------------------------------------------------------------
    def _gdn_dims(self):
        cfg = self.cfg
        c = 2 * cfg.gdn_qk_heads * cfg.gdn_head_dim + cfg.gdn_v_heads * cfg.gdn_head_dim
        return cfg.gdn_qk_heads, cfg.gdn_v_heads, c

    def _merge(self, mods: list, share: bool) -> torch.Tensor:
        ws = [m.weight.detach() for m in mods]
        merged = torch.cat([_bf16(w) for w in ws], dim=0).contiguous()
        if share and all(w.dtype == torch.bfloat16 for w in ws):
            o = 0
            for m in mods:  # the module keeps working (prefill path) on views of the merged tensor: one copy in memory
                n = m.weight.shape[0]
                m.weight.data = merged[o:o + n]
                o += n
        return merged

    def _pack_layer(self, layer, share: bool):
        lw = _Mixer()
        lw.kind = layer.layer_type
        lw.ln_in, lw.ln_post = _f32(layer.input_layernorm.weight), _f32(layer.post_attention_layernorm.weight)
        lw.eps = layer.input_layernorm.eps
        if layer.layer_type == "full_attention":
            a = layer.self_attn
            lw.w_in = self._merge([a.q_proj, a.k_proj, a.v_proj], share)
            lw.w_out = a.o_proj.weight.detach() if a.o_proj.weight.dtype == torch.bfloat16 else _bf16(a.o_proj.weight)
            lw.qn, lw.kn = _f32(a.q_norm.weight), _f32(a.k_norm.weight)
            lw.gated = a.gated
            lw.hq, lw.hkv, lw.d = a.cfg.num_attention_heads, a.cfg.num_kv_heads, a.cfg.head_dim
        else:
            g = layer.linear_attn
            lw.w_in = self._merge([g.in_proj_qkv, g.in_proj_z, g.in_proj_b, g.in_proj_a], share)
            lw.w_out = g.out_proj.weight.detach() if g.out_proj.weight.dtype == torch.bfloat16 else _bf16(g.out_proj.weight)
            lw.conv_w = _f32(g.conv_weight())
            lw.a_log, lw.dt_bias, lw.norm_w = _f32(g.A_log), _f32(g.dt_bias), _f32(g.norm.weight)
        m = layer.mlp
        lw.w_gu = self._merge([m.gate_proj, m.up_proj], share)
        lw.ffn = m.gate_proj.weight.shape[0]
        lw.w_down = m.down_proj.weight.detach() if m.down_proj.weight.dtype == torch.bfloat16 else _bf16(m.down_proj.weight)
        return lw

    def repack(self) -> None:
        """(Re)build the merged bf16 weights from the module. With ``share_weights`` and a bf16 module the parameters become
        views of the merged tensors (one copy in memory; an in-place weight update needs no repack); otherwise call this
        after the module's weights changed."""
        model, cfg, share = self.model, self.cfg, self.share_weights
        H = cfg.hidden_size
        self.layers = [self._pack_layer(layer, share) for layer in model.model.layers]
        self.final_norm = _f32(model.model.norm.weight)
        ew = model.model.embed_tokens.weight.detach()
        self.embed = ew if ew.dtype == torch.bfloat16 else _bf16(ew)
        lm = model.lm_head.weight.detach()
        self.lm_head = (lm if lm.dtype == torch.bfloat16 else _bf16(lm))[self.v0:self.v0 + self.Vs]
        self.mtp = None
        if self.n_draft > 0:
            mtp = model.mtp
            self.mtp = _Mixer()
            self.mtp.we, self.mtp.wh = _f32(mtp.pre_fc_norm_embedding.weight), _f32(mtp.pre_fc_norm_hidden.weight)
            fc = mtp.fc.weight.detach()  # [H, 2H]; row-parallel over K under tensor parallelism
            kk = 2 * H // self.world
            self.mtp.fc = _bf16(fc[:, self.rank * kk:(self.rank + 1) * kk])
            self.mtp.kshard = (self.rank * kk, kk)
            self.mtp.layers = [self._pack_layer(layer, share) for layer in mtp.layers]
            self.mtp.norm = _f32(mtp.norm.weight)
        self.graph = None  # pointers may have changed
        self._warm = 0

    # -- batch membership ---------------------------------------------------------------------------------------------
    def assign(self, b: int, slot: int, ctx: int, block_table: list[int], last_token: int, conv_state: Optional[dict] = None,
               rope_off: int = 0, drafts: Optional[list[int]] = None) -> None:
        """Put a sequence whose first ``ctx`` tokens are cached (KV pages, recurrent state in ``slot``) into batch slot
        ``b``; ``last_token`` is the token at position ``ctx`` (sampled, not yet run). ``conv_state``: layer -> [3, C] rows
        before position ``ctx``. Draft slots start as ``drafts`` or as copies of the token (they are verified, never trusted)."""
        self.graph_sync()
        self.ctx[b] = ctx
        self.slots[b] = slot
        self.parity[b] = 0
        self.ncommit[b] = 0
        self.rope_off[b] = rope_off
        toks = [last_token] + list(drafts or [])
        toks += [last_token] * (self.T - len(toks))
        self.tok_in[b * self.T:(b + 1) * self.T] = torch.tensor(toks[: self.T], dtype=torch.int32)
        self.set_block_table(b, block_table)
        for li in self.cfg.gdn_layers:
            self.conv_rec[li][slot, 0, :3] = conv_state[li].float() if conv_state is not None else 0.0

    def set_shared_prefixes(self, groups: list, tiles_per_item: int = 8) -> None:
        """``groups``: (batch slots, tokens) — sequences whose first ``tokens`` tokens live in the SAME pages (the samples of
        one prompt; a prefix-cache hit). Their query rows are stacked in one CTA over the shared keys, so those pages are
        read once per group instead of once per sequence; every sequence keeps an item of its own for the rest of its
        context. Shared lengths are cut to multiples of 128 keys and must not exceed any member's context."""
        if self.pa_items is None:
            return
        self.graph_sync()
        rows = []
        shared_of = {}
        for members, tokens in groups:
            tiles = int(tokens) // 128
            if tiles < 2 or len(members) < 2 or self.pa_group < 2:
                continue
            nsplit = min(self.pa_splits, (tiles + tiles_per_item - 1) // tiles_per_item)
            for i in range(0, len(members), self.pa_group):
                sub = list(members[i:i + self.pa_group])
                if len(sub) < 2:
                    continue
                for m in sub:
                    shared_of[m] = (tiles * 128, nsplit)
                for sp in range(nsplit):
                    lo, hi = tiles * sp // nsplit, tiles * (sp + 1) // nsplit
                    rows.append([len(sub), lo * 128, hi * 128, 1 + sp, 0, 0, 0, 0] + sub + [0] * (K.PA_ITEM_SEQS - len(sub)))
        own = []
        for b in range(self.B):
            begin, nsplit = shared_of.get(b, (0, 0))
            own.append([1, begin, -1, 0, 1 + nsplit, self.pa_nparts, 0, 0, b] + [0] * (K.PA_ITEM_SEQS - 1))
        table = own + rows  # the per-sequence items first: they are the longest
        if len(table) > self.pa_items.shape[0]:
            raise ValueError("more attention work items than the table holds")
        host = torch.zeros(self.pa_items.shape, dtype=torch.int32)
        host[: len(table)] = torch.tensor(table, dtype=torch.int32)
        self.pa_items.copy_(host)

    def set_block_table(self, b: int, block_table: list[int]) -> None:
        n = len(block_table)
        if n > self.block_table.shape[1]:
            raise ValueError("sequence needs more pages than max_blocks_per_seq")
        self.block_table[b, :n] = torch.tensor(block_table, dtype=torch.int32)

    def release(self, b: int, commit: Optional[int] = None) -> dict:
        """Take the sequence out of the batch: replay its committed rows (``commit`` overrides how many rows of the last
        block count) into the recurrent state and return its conv windows (layer -> [3, C]) so the prefill runner / a
        state snapshot can continue from them."""
        self.graph_sync()
        if commit is not None:
            self.ncommit[b] = commit
        keep = self.ctx.clone()
        only = torch.full_like(self.ctx, -1)
        only[b] = keep[b]
        out = {}
        cfg = self.cfg
        slot = int(self.slots[b])
        par = int(self.parity[b]) & 1
        for li, lw in zip(range(len(self.layers)), self.layers):
            if lw.kind == "full_attention":
                continue
            hk, hv, _ = self._gdn_dims()
            K.gdn_verify(None, lw.conv_w, lw.a_log, lw.dt_bias, lw.norm_w, self.rec_state[li], self.conv_rec[li], self.ab_rec[li], self.slots, only,
                         self.parity, self.ncommit, self.B, 0, self.T, hk, hv, cfg.l2_eps, cfg.rms_eps, None)
            out[li] = self.conv_rec[li][slot, par ^ 1, :3].clone()
        self.ctx[b] = -1
        self.ncommit[b] = 0
        return out

    def set_temperature(self, temperature: float) -> None:
        """The temperature is a launch argument: a captured graph is dropped and re-captured."""
        self.graph_sync()
        self.temperature = float(temperature)
        self.graph, self._warm = None, 0

    def graph_sync(self) -> None:
        torch.cuda.current_stream().synchronize()

    # -- the step -----------------------------------------------------------------------------------------------------
    def _gemm(self, x, w, rows, epi=0, out=None, n=None, up_row0=0):
        """Row-parallel / column GEMM of the step's rows. Returns (tensor, nsplit)."""
        if epi == 0 and out is None:
            ns = min(self.max_split, K.pick_splits(rows, w.shape[0], w.shape[1], self.sms))
            if self.world > 1 and ns == 1 and self._two_shot(rows):
                # bf16 partial rows straight into the reduction's staging buffer: no separate staging kernel
                K.stream_gemm(x[:rows], w, self.ar_ws.tensor[2, :rows], 1, 1)
                return None, -1
            K.stream_gemm(x[:rows], w, self.parts[:, :rows], ns, 0)
            return self.parts, ns
        K.stream_gemm(x[:rows], w, out[:rows], 1, epi, up_row0, n)
        return out, 1

    def _two_shot(self, rows: int) -> bool:
        if self.ar_mode != "auto":
            return self.ar_mode in ("two", "nvls")
        return rows * (self.world - 1) >= 256  # rows every rank would pull in the one-shot form

    def nvls_available(self) -> bool:
        """Multicast addresses exist for every buffer the switch-side reduction touches."""
        bufs = [self.ar_ws, self.h_sym, self.x_sym] + ([self.r_sym] if getattr(self, "r_sym", None) is not None else [])
        return self.world > 1 and all(getattr(b, "mc_ptr", 0) for b in bufs)

    def _reduce_norm(self, parts, ns, residual, weight, out, rows, eps, mode=0, bcast=False):
        """residual (+)= sum over splits and ranks of the partial rows; out = RMSNorm(residual). Under the two-shot form a
        row's residual is current only on its owner unless ``bcast`` (the callers that read the residual itself ask for it)."""
        if self.world == 1:
            K.add_rmsnorm(parts, ns, residual, weight, out, eps, mode, True, rows)
            return
        buf = self.ar_ws.tensor.shape[1] * self.ar_ws.tensor.shape[2]
        if ns >= 0:
            K.reduce_parts_bf16(parts, ns, self.ar_ws.tensor, rows, self.H, buf, self.ar_ctr)
        if self._two_shot(rows):
            res_sym = self.x_sym if residual is self.x_res else self.r_sym
            mc = (self.ar_ws.mc_ptr, self.h_sym.mc_ptr, res_sym.mc_ptr) if (self.ar_mode == "nvls" or self.nvls_auto) else (0, 0, 0)
            K.ar2_add_rmsnorm(self.ar_ws.c_ptrs, self.symm.flags.c_ptrs, self.h_sym.c_ptrs, res_sym.c_ptrs, self.rank, self.world, SLOT_STEP_AR,
                              self.ar_ctr, self.ar_ticket, mode, bcast, weight, rows, self.H, buf, eps, 1 << 22, self.status, 2 * self.sms,
                              fixed_buf=2 if ns < 0 else -1, mc_partials=mc[0], mc_outs=mc[1], mc_residuals=mc[2])
            return
        K.ar_add_rmsnorm(self.ar_ws.c_ptrs, self.symm.flags.c_ptrs, self.rank, self.world, SLOT_STEP_AR, self.ar_ctr, self.ar_ticket, residual, mode,
                         weight, out, rows, self.H, buf, eps, 1 << 22, self.status, 2 * self.sms)

    def _attention(self, lw, kc, vc, ctx, batch, t):
        cfg = self.cfg
        rows = batch * t
        K.stream_gemm(self.h[:rows], lw.w_in, self.proj[:rows], 1, 0)
        K.attn_prep(self.proj, lw.qn, lw.kn, self.inv_freq, cfg.rotary_dim, ctx, self.rope_off, self.block_table, rows, t, lw.hq, lw.hkv, lw.d,
                    lw.gated, cfg.rms_eps, self.q, kc, vc)
        if self.pa_items is not None:
            K.paged_attention(self.q, kc, vc, self.block_table, ctx, batch, t, lw.hq, lw.hkv, lw.d, lw.d ** -0.5, self.proj, lw.gated, self.mix_out,
                              True, self.pa_items, self.pa_nparts, self.pa_part_o, self.pa_part_ml)
        else:
            K.paged_attention(self.q, kc, vc, self.block_table, ctx, batch, t, lw.hq, lw.hkv, lw.d, lw.d ** -0.5, self.proj, lw.gated, self.mix_out,
                              self.tc_attn)
        return self._gemm(self.mix_out.view(-1)[: self.M * lw.hq * lw.d].view(self.M, lw.hq * lw.d), lw.w_out, rows)

    def _layer(self, li, lw, rows, batch, t, ctx, kc, vc, next_norm, residual, bcast_last=False):
        cfg = self.cfg
        if lw.kind == "full_attention":
            parts, ns = self._attention(lw, kc, vc, ctx, batch, t)
        else:
            hk, hv, _ = self._gdn_dims()
            K.stream_gemm(self.h[:rows], lw.w_in, self.proj[:rows], 1, 0)
            out = self.mix_out.view(-1)[: self.M * hv * 128].view(self.M, hv * 128)
            K.gdn_verify(self.proj, lw.conv_w, lw.a_log, lw.dt_bias, lw.norm_w, self.rec_state[li], self.conv_rec[li], self.ab_rec[li], self.slots, ctx,
                         self.parity, self.ncommit, batch, t, self.T, hk, hv, cfg.l2_eps, cfg.rms_eps, out)
            parts, ns = self._gemm(out, lw.w_out, rows)
        self._reduce_norm(parts, ns, residual, lw.ln_post, self.h, rows, lw.eps)
        act = self.act.view(-1)[: self.M * lw.ffn].view(self.M, lw.ffn)
        K.stream_gemm(self.h[:rows], lw.w_gu, act[:rows], 1, 2, lw.ffn, lw.ffn)
        parts, ns = self._gemm(act, lw.w_down, rows)
        self._reduce_norm(parts, ns, residual, next_norm, self.h, rows, lw.eps, bcast=bcast_last)

    def _sync(self):
        if self.world > 1:
            K.symm_barrier(self.symm.flags.c_ptrs, self.rank, self.world, SLOT_STEP_SYNC, self.sync_ctr, 1 << 22, self.status)

    def _launch_step(self) -> None:
        cfg, M, B, T = self.cfg, self.M, self.B, self.T
        lib = _lib.lib()
        _lib.check(lib.pear_embed_merge(_lib.ptr(self.tok_in), _lib.ptr(self.embed), _lib.ptr(None), _lib.ptr(None), _lib.ptr(self.x_res), M, self.H,
                                        cfg.vocab_size, _lib.stream()), "embed")
        _lib.count_launch()
        K.add_rmsnorm(None, 0, self.x_res, self.layers[0].ln_in, self.h, cfg.rms_eps, 0, True, M)
        for li, lw in enumerate(self.layers):
            nxt = self.layers[li + 1].ln_in if li + 1 < len(self.layers) else self.final_norm
            self._layer(li, lw, M, B, T, self.ctx, self.k_cache.get(li), self.v_cache.get(li), nxt, self.x_res,
                        bcast_last=(li + 1 == len(self.layers) and self.mtp is not None))
        K.stream_gemm(self.h, self.lm_head, self.logits, 1, 0)
        K.verify_chunks(self.logits, self.Vs, self.v0, self.temperature, self.tok_in, self.ctx, B, T, self.chunks, self.seed, self.step_ctr,
                        self.recs_ptrs, self.rank, self.world, self.sync_ctr, self.rec_buf_elems)
        if self.topk:
            K.topk_chunks(self.logits, self.Vs, self.v0, self.temperature, self.ctx, B, T, self.chunks, self.tops_ptrs, self.rank, self.world,
                          self.sync_ctr, self.rec_buf_elems)
        self._sync()
        if self.topk:  # (before verify_finish: it advances the contexts, inactive slots are told by ctx < 0 either way)
            K.topk_finish(self.tops_t, self.rec_buf_elems, self.recs_t, self.rec_buf_elems, self.sync_ctr, self.world, self.chunks, B, T, self.ctx,
                          self.top_ids, self.top_lp)
        K.verify_finish(self.recs_t, self.rec_buf_elems, self.sync_ctr, self.world, self.chunks, B, T, self.seed, self.step_ctr, self.tok_in, self.ctx,
                        self.ncommit, self.parity, self.out_tok, self.out_lp, self.n_accept, self.nonfinite, self.sel_row, self.mtp_tok, self.mtp_ctx)
        if self.debug_logits is not None:
            self.debug_logits.copy_(self.logits)
        if self.mtp is not None:
            self._launch_drafter()
        # result record for the host: tokens | accepted | nonfinite | log-prob bits
        r = self._dev_rec
        r[: B * T].copy_(self.out_tok.view(-1))
        r[B * T: B * T + B].copy_(self.n_accept)
        r[B * T + B: B * T + 2 * B].copy_(self.nonfinite)
        r[B * T + 2 * B:].copy_(self.out_lp.view(-1).view(torch.int32))

    def _launch_drafter(self) -> None:
        cfg, M, B, T, mtp = self.cfg, self.M, self.B, self.T, self.mtp
        k0, kk = mtp.kshard
        for p in range(self.n_draft):
            rows, batch, t = (M, B, T) if p == 0 else (B, B, 1)
            if p == 0:  # over the step's rows: fills the drafter's KV pages; the accepted row's output is the first draft
                K.mtp_input(self.mtp_tok, self.embed, self.x_res, None, mtp.we, mtp.wh, rows, self.H, cfg.rms_eps, self.xcat)
            else:
                K.mtp_input(self.draft_tok, self.embed, self.r_sel if p % 2 == 1 else self.r_sel2, None, mtp.we, mtp.wh, rows, self.H, cfg.rms_eps, self.xcat)
            parts, ns = self._gemm(self.xcat[:, k0:k0 + kk], mtp.fc, rows)
            lw0 = mtp.layers[0]
            self._reduce_norm(parts, ns, self.r_mtp, lw0.ln_in, self.h, rows, lw0.eps, mode=1)
            ctx = self.mtp_ctx[p]
            for j, lw in enumerate(mtp.layers):
                nxt = mtp.layers[j + 1].ln_in if j + 1 < len(mtp.layers) else mtp.norm
                self._layer(-1, lw, rows, batch, t, ctx, self.mtp_k[j], self.mtp_v[j], nxt, self.r_mtp, bcast_last=(j + 1 == len(mtp.layers)))
            nxt_r = self.r_sel if p % 2 == 0 else self.r_sel2
            if p == 0:
                K.gather_rows(self.h, self.sel_row, self.h_sel, B)
                K.gather_rows(self.r_mtp, self.sel_row, nxt_r, B)
                hsel = self.h_sel
            else:
                nxt_r.copy_(self.r_mtp[:B])
                hsel = self.h
            K.stream_gemm(hsel[:B], self.lm_head, self.logits[:B], 1, 0)
            K.argmax_chunks(self.logits, self.Vs, self.v0, B, self.achunks, self.keys_ptrs, self.rank, self.world, self.sync_ctr, self.key_buf_elems)
            self._sync()
            K.argmax_finish(self.keys_t, self.key_buf_elems, self.sync_ctr, self.world, self.achunks, B, self.tok_in, T, 1 + p, self.draft_tok)

    def step(self) -> None:
        """Launch one step on the current stream (graph replay after two eager warm-up steps)."""
        with nvtx.annotate("rollout/decode_step"):
            self._step()

    def _step(self) -> None:
        _lib.on_device(self.h)  # a thread on another current device would launch the step's kernels on the wrong GPU
        if not self.use_graph:
            self._launch_step()
        elif self.graph is not None:
            self.graph.replay()
        elif self._warm < 2:
            self._launch_step()
            self._warm += 1
        else:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._launch_step()
            self.graph = g  # capture does not run the step: replay it once for this call
            g.replay()
        self.steps += 1

    def results(self) -> StepResult:
        """Copy the last step's result record to pinned host memory and wait for it."""
        B, T = self.B, self.T
        self._host.copy_(self._dev_rec, non_blocking=True)
        if self.topk:
            self._host_top_ids.copy_(self.top_ids, non_blocking=True)
            self._host_top_lp.copy_(self.top_lp, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h = self._host
        res = StepResult(h[: B * T].view(B, T).clone(), h[B * T: B * T + B].clone(), h[B * T + 2 * B:].view(torch.float32).view(B, T).clone(),
                         h[B * T + B: B * T + 2 * B].clone())
        if self.topk:
            res.topk_ids = self._host_top_ids.view(B, T, K.TOPK).clone()
            res.topk_logprobs = self._host_top_lp.view(B, T, K.TOPK).clone()
        return res

    def check(self) -> None:
        K.check_status(self.dev)
        if self.symm is not None:
            self.symm.check()

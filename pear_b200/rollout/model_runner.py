"""Model runner of the rollout engine: one scheduler step = one packed forward over every scheduled row.

All rows of all sequences of a step are packed, so every linear layer is one GEMM over the step; attention reads each
sequence's paged KV through its block table; Gated-DeltaNet layers advance each sequence's running state. The recurrent
state under speculative decoding follows the replay scheme (upstream ``rollout/blackwell/gdn/replay.py:15-35``): a
sequence keeps the state at the START of its last verify block plus that block's record of conv inputs and gate rows;
the next step first replays the rows that were committed. The MTP drafter (upstream ``rollout/speculator.py``,
``rollout/blackwell/mtp.py``) shares the embedding and the head and keeps its own KV pages in the same block tables.

Tensor-parallel execution shards heads / FFN columns over the TP group with the collectives of
:mod:`pear_b200.parallel.tp` (fused all-reduce + residual + norm kernel on NVSwitch peers, NCCL otherwise).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..models.config import HybridConfig
from ..models import hybrid
from ..models.hybrid import HybridForCausalLM, linear_fp32, row_linear
from ..ops import api as ops
from ..ops import reference as ref


@dataclass
class SeqState:
    """Per-sequence device state owned by the runner."""

    seq_id: int
    slot: int  # running recurrent-state slot
    pending: dict = field(default_factory=dict)  # layer -> (mixed rows, a rows, b rows) of the uncommitted block
    pending_rows: int = 0
    commit_rows: int = 0  # rows of the pending block to replay at the next step
    mtp_hidden: Optional[torch.Tensor] = None  # pre-norm residual of the last committed row (drafter input)


@dataclass
class StepRow:
    seq: SeqState
    tokens: torch.Tensor  # [n] token ids of this chunk
    start: int  # absolute position of tokens[0]
    block_table: list[int]
    need_logits: int  # number of trailing rows whose logits are needed (0 for a non-final prefill chunk)
    embeds: Optional[torch.Tensor] = None  # [n, H] rows replacing the token embedding where `embeds_mask`
    embeds_mask: Optional[torch.Tensor] = None
    positions: Optional[torch.Tensor] = None  # [3, n] M-RoPE positions (default: start + arange on all axes)


class ModelRunner:
    def __init__(self, model: HybridForCausalLM, num_blocks: int, block_size: int, num_state_slots: int, device="cpu",
                 kv_dtype: Optional[torch.dtype] = None):
        self.model, self.cfg = model, model.config
        cfg = self.cfg
        self.device = torch.device(device)
        self.block_size = block_size
        kv_dtype = kv_dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.attn_layers = cfg.attention_layers
        self.gdn_layers = cfg.gdn_layers
        self.k_cache = {l: torch.zeros(num_blocks, block_size, cfg.num_kv_heads, cfg.head_dim, dtype=kv_dtype, device=self.device)
                        for l in self.attn_layers}
        self.v_cache = {l: torch.zeros_like(self.k_cache[l]) for l in self.attn_layers}
        self.has_mtp = model.mtp is not None
        if self.has_mtp:
            n = len(model.mtp.layers)
            self.mtp_k = [torch.zeros(num_blocks, block_size, cfg.num_kv_heads, cfg.head_dim, dtype=kv_dtype, device=self.device)
                          for _ in range(n)]
            self.mtp_v = [torch.zeros_like(t) for t in self.mtp_k]
        kw = cfg.conv_kernel - 1
        self.conv_state = {l: torch.zeros(num_state_slots, kw, cfg.gdn_conv_dim, dtype=torch.float32, device=self.device)
                           for l in self.gdn_layers}
        self.rec_state = {l: torch.zeros(num_state_slots, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_head_dim, dtype=torch.float32,
                                         device=self.device) for l in self.gdn_layers}
        # On a GPU the decode / verify rows go through the CUDA kernels of ops/csrc/rollout_kernels.cu (split-KV paged
        # attention straight from the block table, the fused GDN decode step); long prefill chunks and shapes the kernels
        # are not built for take the PyTorch statements.
        group = cfg.num_attention_heads // max(1, cfg.num_kv_heads)
        self.use_kernels = self.device.type == "cuda"
        self._attn_kernel_ok = cfg.head_dim in (128, 256) and group <= 8 and block_size == 16 and kv_dtype == torch.bfloat16
        self._gdn_kernel_ok = cfg.gdn_head_dim == 128 and cfg.conv_kernel == 4

    # -- cache plumbing for the block manager / host tier -----------------------------------------------------------------
    def kv_tensors(self) -> list[torch.Tensor]:
        out = []
        for l in self.attn_layers:
            out += [self.k_cache[l], self.v_cache[l]]
        if self.has_mtp:
            out += self.mtp_k + self.mtp_v
        return out

    def state_tensors(self) -> list[torch.Tensor]:
        out = []
        for l in self.gdn_layers:
            out += [self.conv_state[l], self.rec_state[l]]
        return out

    def copy_state(self, src_slot: int, dst_slot: int) -> None:
        for t in self.state_tensors():
            t[dst_slot].copy_(t[src_slot])

    def zero_state(self, slot: int) -> None:
        for t in self.state_tensors():
            t[slot].zero_()

    # -- helpers ------------------------------------------------------------------------------------------------------
    def _write_kv(self, kc, vc, row: StepRow, k: torch.Tensor, v: torch.Tensor) -> None:
        bs = self.block_size
        pos = torch.arange(row.start, row.start + k.shape[0], device=self.device)
        blk = torch.tensor(row.block_table, device=self.device)[pos // bs]
        kc[blk, pos % bs] = k.to(kc.dtype)
        vc[blk, pos % bs] = v.to(vc.dtype)

    def _read_kv(self, kc, vc, row: StepRow, upto: int):
        bs = self.block_size
        nblk = (upto + bs - 1) // bs
        blk = torch.tensor(row.block_table[:nblk], device=self.device)
        k = kc[blk].reshape(nblk * bs, *kc.shape[2:])[:upto]
        v = vc[blk].reshape(nblk * bs, *vc.shape[2:])[:upto]
        return k, v

    def _attention(self, att, hidden: torch.Tensor, rows: list[StepRow], bounds: list[int], cos, sin, kc, vc) -> torch.Tensor:
        cfg = att.cfg
        from ..models.hybrid import SeqMeta

        meta = SeqMeta(cu_seqlens=bounds, cos=cos, sin=sin)
        q, k, v, gate = att.project(hidden, meta)
        outs: list = [None] * len(rows)
        short = []  # rows of at most 8 query tokens: decode and verify blocks
        for i, row in enumerate(rows):
            s, e = bounds[i], bounds[i + 1]
            self._write_kv(kc, vc, row, k[s:e], v[s:e])
            if self.use_kernels and self._attn_kernel_ok and e - s <= 8:
                short.append(i)
                continue
            kk, vv = self._read_kv(kc, vc, row, row.start + (e - s))
            if self.use_kernels and self._attn_kernel_ok and cfg.head_dim == 256:  # prefill chunk: tcgen05 kernel
                from ..ops import kernels as ops_k

                outs[i] = ops_k.prefill_attention(q[s:e], kk, vv, cfg.head_dim ** -0.5)
                continue
            outs[i] = ref.attention_with_cache(q[s:e], kk, vv, row.start, cfg.head_dim ** -0.5)
        if short:
            from ..ops import rollout_ops

            idx, ctx, tabs = [], [], []
            maxb = max(len(rows[i].block_table) for i in short)
            for i in short:
                s, e = bounds[i], bounds[i + 1]
                for j in range(e - s):
                    idx.append(s + j)
                    ctx.append(rows[i].start + j + 1)  # causal inside the block: row j sees the context up to itself
                    tabs.append(rows[i].block_table + [0] * (maxb - len(rows[i].block_table)))
            sel = torch.tensor(idx, device=self.device)
            o_short = rollout_ops.paged_attention(q[sel].float().contiguous(), kc, vc, torch.tensor(tabs, dtype=torch.int32, device=self.device),
                                                  torch.tensor(ctx, dtype=torch.int32, device=self.device), cfg.head_dim ** -0.5)
            off = 0
            for i in short:
                n = bounds[i + 1] - bounds[i]
                outs[i] = o_short[off:off + n]
                off += n
        o = torch.cat(outs, dim=0)
        o = (ops.sigmoid_gate(o, gate) if gate is not None else o).reshape(hidden.shape[0], cfg.q_size)
        return row_linear(o, att.o_proj.weight)

    def _gdn(self, li: int, gdn, hidden: torch.Tensor, rows: list[StepRow], bounds: list[int], speculative: bool) -> torch.Tensor:
        cfg = self.cfg
        t = hidden.shape[0]
        mixed = linear_fp32(hidden, gdn.in_proj_qkv.weight)
        z = linear_fp32(hidden, gdn.in_proj_z.weight).view(t, cfg.gdn_v_heads, cfg.gdn_head_dim)
        b = linear_fp32(hidden, gdn.in_proj_b.weight)
        a = linear_fp32(hidden, gdn.in_proj_a.weight)
        if (self.use_kernels and self._gdn_kernel_ok and not speculative and all(bounds[i + 1] - bounds[i] == 1 for i in range(len(rows)))
                and all(not (r.seq.commit_rows > 0 and li in r.seq.pending) for r in rows)):
            # plain decode step: one token per sequence -> the fused kernel (conv update, gates, L2 norm, delta rule, gated norm)
            from ..ops import rollout_ops

            slots = torch.tensor([r.seq.slot for r in rows], dtype=torch.int32, device=self.device)
            y = rollout_ops.gdn_decode(mixed.float().contiguous(), z.reshape(t, -1).float().contiguous(), a.float().contiguous(), b.float().contiguous(),
                                       gdn.conv_weight().float().contiguous(), gdn.A_log.float(), gdn.dt_bias.float(), gdn.norm.weight.float(),
                                       self.conv_state[li], self.rec_state[li], slots, cfg.gdn_qk_heads, cfg.gdn_v_heads, cfg.l2_eps, cfg.rms_eps)
            for r in rows:
                r.seq.pending.pop(li, None)
            return row_linear(y, gdn.out_proj.weight)
        outs = []
        for i, row in enumerate(rows):
            s, e = bounds[i], bounds[i + 1]
            st = row.seq
            conv, rec = self.conv_state[li][st.slot], self.rec_state[li][st.slot]
            # replay the committed rows of the previous (speculative) block
            if st.commit_rows > 0 and li in st.pending:
                pm, pa, pb = st.pending[li]
                n = st.commit_rows
                conv, rec = self._advance(gdn, pm[:n], pa[:n], pb[:n], conv, rec)[1:]
                self.conv_state[li][st.slot].copy_(conv)
                self.rec_state[li][st.slot].copy_(rec)
            o, conv2, rec2 = self._advance(gdn, mixed[s:e], a[s:e], b[s:e], conv, rec)
            if speculative:
                st.pending[li] = (mixed[s:e].clone(), a[s:e].clone(), b[s:e].clone())  # committed after verification
            else:
                self.conv_state[li][st.slot].copy_(conv2)
                self.rec_state[li][st.slot].copy_(rec2)
                st.pending.pop(li, None)
            outs.append(o)
        o = torch.cat(outs, dim=0)
        y = ops.gated_rms_norm(o, z, gdn.norm.weight, cfg.rms_eps).reshape(t, cfg.gdn_value_dim)
        return row_linear(y, gdn.out_proj.weight)

    def _advance(self, gdn, mixed, a, b, conv, rec):
        """Run conv + gates + delta rule over rows from (conv, rec); returns (outputs, new conv rows, new state)."""
        n = mixed.shape[0]
        g, beta = ops.gdn_gates(a, b, gdn.A_log, gdn.dt_bias)
        q, k, v, conv_final = gdn.front(mixed, [0, n], conv.unsqueeze(0))
        if n <= 8:
            o, rec2 = ref.gdn_recurrent(q, k, v, g, beta, rec)
        else:
            o, rec2 = ops.gdn_scan(q, k, v, g, beta, rec)
        return o, conv_final[0], rec2

    # -- the step -----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, rows: list[StepRow], speculative: bool = False):
        """Returns (logits of the requested rows [sum need_logits, V], pre-norm residual of those rows)."""
        model, cfg = self.model, self.cfg
        tokens = torch.cat([r.tokens.to(self.device) for r in rows])
        bounds = [0]
        for r in rows:
            bounds.append(bounds[-1] + int(r.tokens.shape[0]))
        pos = torch.cat([r.positions.to(self.device) if r.positions is not None
                         else torch.arange(r.start, r.start + r.tokens.shape[0], device=self.device).expand(3, -1) for r in rows], dim=1)
        cos, sin = model.rope(pos)
        table = model.model.embed_tokens.weight
        if self.use_kernels and table.dtype == torch.bfloat16:
            # one kernel: embedding lookup with the vision-placeholder rows merged in (upstream `_shard_embed_kernel`)
            from ..ops import rollout_ops

            emb = msk = None
            if any(r.embeds is not None for r in rows):
                emb = torch.zeros(tokens.shape[0], cfg.hidden_size, device=self.device)
                msk = torch.zeros(tokens.shape[0], dtype=torch.bool, device=self.device)
                for i, r in enumerate(rows):
                    if r.embeds is not None:
                        s, e = bounds[i], bounds[i + 1]
                        emb[s:e], msk[s:e] = r.embeds.to(self.device).float(), r.embeds_mask.to(self.device)
            x = rollout_ops.embed_merge(tokens, table, emb, msk)
        else:
            x = model.model.embed_tokens(tokens).float()
            for i, r in enumerate(rows):
                if r.embeds is not None:
                    s, e = bounds[i], bounds[i + 1]
                    x[s:e] = torch.where(r.embeds_mask.to(self.device)[:, None], r.embeds.to(self.device).float(), x[s:e])
        layers = list(model.model.layers)
        if not hybrid.tensor_parallel_active():
            for li, layer in enumerate(layers):
                h = layer.input_layernorm(x)
                if layer.layer_type == "full_attention":
                    mixed = self._attention(layer.self_attn, h, rows, bounds, cos, sin, self.k_cache[li], self.v_cache[li])
                else:
                    mixed = self._gdn(li, layer.linear_attn, h, rows, bounds, speculative)
                y, x = ops.add_rms_norm(mixed, x, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
                x = x + layer.mlp(y)
        else:
            # tensor parallel: every row-parallel projection hands back its partial sum and the reduction runs together
            # with the residual add and the norm that follow it (one NVSwitch kernel when the fused transport is set)
            with hybrid.defer_row_reduce():
                h = layers[0].input_layernorm(x)
                for li, layer in enumerate(layers):
                    if layer.layer_type == "full_attention":
                        mixed = self._attention(layer.self_attn, h, rows, bounds, cos, sin, self.k_cache[li], self.v_cache[li])
                    else:
                        mixed = self._gdn(li, layer.linear_attn, h, rows, bounds, speculative)
                    ln = layer.post_attention_layernorm
                    y, x = hybrid.reduce_add_rms_norm(mixed, x, ln.weight, ln.eps)
                    part = layer.mlp(y)
                    if li + 1 < len(layers):
                        nxt = layers[li + 1].input_layernorm
                        h, x = hybrid.reduce_add_rms_norm(part, x, nxt.weight, nxt.eps)
                    else:
                        x = x + hybrid.reduce_partial(part)
        for r in rows:  # the replay (if any) has been applied by every GDN layer
            if not speculative:
                r.seq.commit_rows = 0
                r.seq.pending_rows = 0
            else:
                r.seq.commit_rows = 0
                r.seq.pending_rows = int(r.tokens.shape[0])
        sel = []
        for i, r in enumerate(rows):
            if r.need_logits > 0:
                sel.append(torch.arange(bounds[i + 1] - r.need_logits, bounds[i + 1], device=self.device))
        if not sel:
            return None, None, x, bounds
        sel = torch.cat(sel)
        resid = x[sel]
        logits = model.logits(model.model.norm(resid))
        return logits, resid, x, bounds

    def commit(self, seq: SeqState, rows: int) -> None:
        """After verification: ``rows`` rows of the pending block are part of the sequence; they are replayed into the
        running state at the start of the sequence's next step."""
        seq.commit_rows = rows

    def flush(self, seq: SeqState) -> None:
        """Apply the pending committed rows now (needed before the running state is snapshotted or the sequence ends)."""
        if seq.commit_rows <= 0:
            seq.pending.clear()
            return
        for li in self.gdn_layers:
            if li in seq.pending:
                gdn = self.model.model.layers[li].linear_attn
                pm, pa, pb = seq.pending[li]
                n = seq.commit_rows
                _, conv, rec = self._advance(gdn, pm[:n], pa[:n], pb[:n], self.conv_state[li][seq.slot], self.rec_state[li][seq.slot])
                self.conv_state[li][seq.slot].copy_(conv)
                self.rec_state[li][seq.slot].copy_(rec)
        seq.pending.clear()
        seq.commit_rows = 0

    # -- MTP drafter ----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def mtp_forward(self, row: StepRow, next_tokens: torch.Tensor, residual: torch.Tensor):
        """One MTP pass over rows at positions row.start.. (``row.positions`` when the request carries its own) combining
        ``residual[j]`` with ``embed(next_tokens[j])``; writes the drafter's KV pages and returns (logits, the drafter's output
        residual)."""
        model, mtp = self.model, self.model.mtp
        from ..models.hybrid import SeqMeta

        n = next_tokens.shape[0]
        pos = row.positions.to(self.device) if row.positions is not None else torch.arange(row.start, row.start + n, device=self.device)
        cos, sin = model.rope(pos)
        x = torch.cat([mtp.pre_fc_norm_embedding(model.model.embed_tokens(next_tokens.to(self.device)).float()),
                       mtp.pre_fc_norm_hidden(residual)], dim=-1)
        r = linear_fp32(x, mtp.fc.weight)
        sub = StepRow(row.seq, next_tokens, row.start, row.block_table, n)
        for j, layer in enumerate(mtp.layers):
            h = layer.input_layernorm(r)
            mixed = self._attention(layer.self_attn, h, [sub], [0, n], cos, sin, self.mtp_k[j], self.mtp_v[j])
            y, r = ops.add_rms_norm(mixed, r, layer.post_attention_layernorm.weight, layer.post_attention_layernorm.eps)
            r = r + layer.mlp(y)
        return model.logits(mtp.norm(r)), r

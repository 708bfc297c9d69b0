"""Sequence parallelism of the hybrid decoder: Ulysses head<->sequence all-to-all for the attention layers and
context parallelism with boundary-state chaining for the Gated-DeltaNet layers.

Every rank of the group holds a CONTIGUOUS slice of ``T_local`` tokens of the packed micro-batch (equal slice lengths;
the batch is padded with a dummy sequence). Upstream counterparts: one all-to-all in / out around the attention core
(``pear/models/qwen3_5/trainer/blackwell/ulysses_attention.py:29-121``), conv halo = the previous rank's last 3 rows
(``trainer/gdn.py:570-584``), and per-rank (H, M) summaries folded left as ``X <- X M + H``
(``trainer/blackwell/delta_rule.py:51-89``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import api as ops
from . import collectives as C


class SequenceParallel:
    def __init__(self, group):
        self.group = group
        self.size = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0

    # -----------------------------------------------------------------------------------------------------------------
    # attention: [T_local, H, D] -> [T, H / sp, D] -> attention -> back
    # -----------------------------------------------------------------------------------------------------------------
    def _seq_to_heads(self, x: torch.Tensor) -> torch.Tensor:
        """[T_local, H, D] with H = sp * h -> [sp * T_local, h, D]: rank j receives heads [j*h, (j+1)*h) of every slice."""
        t, hh, d = x.shape
        h = hh // self.size
        y = C.all_to_all(x.reshape(t, self.size, h, d).permute(1, 0, 2, 3).contiguous(), self.group)  # [sp, t, h, d]
        return y.reshape(self.size * t, h, d)

    def _heads_to_seq(self, y: torch.Tensor, t_local: int) -> torch.Tensor:
        """Inverse of :meth:`_seq_to_heads`: [sp * T_local, h, D] -> [T_local, sp * h, D]."""
        _, h, d = y.shape
        x = C.all_to_all(y.reshape(self.size, t_local, h, d).contiguous(), self.group)  # [sp (head group), t, h, d]
        return x.permute(1, 0, 2, 3).reshape(t_local, self.size * h, d)

    def attention(self, q, k, v, cu_seqlens, scale):
        """q: [T_local, Hq, D]; k, v: [T_local, Hkv, D]. KV heads are repeated when ``sp`` exceeds their number so every
        rank gets the KV head(s) of its q heads."""
        sp = self.size
        t_local, hq, _ = q.shape
        hkv = k.shape[1]
        if hq % sp:
            raise ValueError(f"{hq} query heads do not split over {sp} sequence-parallel ranks")
        if hkv % sp:
            rep = sp // hkv if sp % hkv == 0 else None
            if rep is None or (hq // hkv) % rep:
                raise ValueError(f"{hkv} kv heads cannot be spread over {sp} ranks")
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
        # ONE all-to-all in: q, k and v are packed rank-major, [sp, T_local, hq/sp + 2 hkv/sp, D], so that rank j receives
        # its query heads together with their KV heads from every sequence slice in a single message per peer
        hq_l, hk_l, d = hq // sp, k.shape[1] // sp, q.shape[2]
        packed = torch.cat([q.reshape(t_local, sp, hq_l, d), k.reshape(t_local, sp, hk_l, d), v.reshape(t_local, sp, hk_l, d)], dim=2)
        got = C.all_to_all(packed.permute(1, 0, 2, 3).contiguous(), self.group).reshape(sp * t_local, hq_l + 2 * hk_l, d)
        qh, kh, vh = got[:, :hq_l], got[:, hq_l:hq_l + hk_l], got[:, hq_l + hk_l:]
        o = ops.causal_attention(qh.contiguous(), kh.contiguous(), vh.contiguous(), cu_seqlens, scale)
        return self._heads_to_seq(o, t_local)  # ONE all-to-all out

    # -----------------------------------------------------------------------------------------------------------------
    # gated delta net: local scan with an incoming state chained across ranks
    # -----------------------------------------------------------------------------------------------------------------
    def start_conv_halo(self, mixed: torch.Tensor, conv_kernel: int):
        """Launch the all-gather of every rank's last ``conv_kernel - 1`` conv-input rows as soon as they exist: the mixer's
        z / b / a projections run while it is in flight (upstream overlaps the same exchange: trainer/gdn.py:570-584).
        Returns what ``gdn(halo=...)`` takes."""
        kw = conv_kernel - 1
        return C.all_gather_stack_start(mixed[mixed.shape[0] - kw:].float(), self.group)

    def gdn(self, mixer, mixed: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, meta, bounds: list[int], halo=None):
        """``mixed`` [T_local, C] are this rank's conv inputs. Returns the scan output [T_local, Hv, V]. ``halo``: the started
        exchange of ``start_conv_halo`` (else it runs here, blocking)."""
        cfg = mixer.cfg
        t_local = mixed.shape[0]
        kw = cfg.conv_kernel - 1
        # ---- conv halo: the previous rank's last rows, unless this slice starts a sequence
        if halo is not None:
            tails, wait = halo
            wait()
        else:
            tails = C.all_gather_stack(mixed[t_local - kw :].float(), self.group)  # [sp, kw, C]
        starts_sequence = meta.offset in meta.cu_seqlens
        if self.rank == 0 or starts_sequence:
            halo = torch.zeros_like(tails[0]) + 0.0 * tails[0]  # keeps the autograd edge so every rank's backward joins the collective
        else:
            halo = tails[self.rank - 1]
        nseq = len(bounds) - 1
        init_conv = torch.zeros(nseq, kw, mixed.shape[1], dtype=torch.float32, device=mixed.device)
        init_conv = torch.cat([halo.unsqueeze(0), init_conv[1:]], dim=0)
        q, k, v, _ = mixer.front(mixed, bounds, init_conv)

        # ---- summary of the tail span (last boundary .. end of slice): state from zero (H) and transition (M)
        s, e = bounds[-2], bounds[-1]
        hv, kd = cfg.gdn_v_heads, cfg.gdn_head_dim
        rep = hv // cfg.gdn_qk_heads
        eye = torch.eye(kd, device=mixed.device, dtype=torch.float32).expand(hv, kd, kd).contiguous()
        zero_v = torch.zeros(e - s, hv, kd, device=mixed.device, dtype=torch.float32)
        _, M = ops.gdn_scan(q[s:e], k[s:e], zero_v, g[s:e], beta[s:e], eye)  # v = 0 from the identity: S_out = M
        _, H = ops.gdn_scan(q[s:e], k[s:e], v[s:e], g[s:e], beta[s:e], None)
        has_cut = torch.tensor(1.0 if (len(bounds) > 2 or starts_sequence) else 0.0, device=mixed.device)
        HM = C.all_gather_stack(torch.stack([H, M], dim=0), self.group)  # [sp, 2, Hv, V, K]
        cuts = C.all_gather_cat(has_cut.reshape(1), self.group)  # [sp]
        # ---- fold left: state entering rank r
        X = torch.zeros(hv, kd, kd, device=mixed.device, dtype=torch.float32)
        for r in range(self.rank):
            Hr, Mr = HM[r, 0], HM[r, 1]
            X = Hr if cuts[r] > 0 else torch.einsum("hvk,hkj->hvj", X, Mr) + Hr
        if starts_sequence:
            X = torch.zeros_like(X)
        X = X + 0.0 * HM.sum()  # every rank's graph reaches the gathered summaries: backward collectives stay matched
        # ---- local scan: the first span continues from X, later spans start from zero
        inits = [X] + [None] * (nseq - 1)
        return ops.gdn_scan_packed(q, k, v, g, beta, bounds, inits)

"""Sampling for the rollout engine: temperature / exact-max top-p sampling with the top-k processed log-probs that score
centering reads, non-finite logit detection, and the lossless rejection sampler of MTP speculative decoding.

Upstream counterparts: ``pear/rollout/top_p.py`` (top-p whose softmax is shifted by each row's exact maximum so it
cannot overflow, pivot found by binary search), ``pear/models/qwen3_5/rollout/sampler.py:18-160`` (temperature-only rows
served with top-32 processed log-probs; greedy drafts verified with the lossless rule ``lp(d) > log u``), and
``rollout/nonfinite_logits.py`` (NaN / +inf logits are counted and raised with step / row / request). CUDA tensors run
the fused kernel of ``csrc/sampler.cu``; this module is also the CPU statement and the oracle of that kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class NonFiniteLogits(RuntimeError):
    def __init__(self, step: int, rows: list[int], request_ids: list[str]):
        super().__init__(f"step {step}: non-finite logits in rows {rows} of requests {request_ids}")
        self.step, self.rows, self.request_ids = step, rows, request_ids


@dataclass
class SampleOutput:
    tokens: torch.Tensor  # [N]
    logprobs: torch.Tensor  # [N] processed log-prob of the sampled token
    topk_ids: Optional[torch.Tensor]  # [N, k]
    topk_logprobs: Optional[torch.Tensor]  # [N, k]
    ranks: torch.Tensor  # [N] 1-based rank of the sampled token
    nonfinite: torch.Tensor  # [N] count of NaN / +inf logits per row


def count_nonfinite(logits: torch.Tensor) -> torch.Tensor:
    return (torch.isnan(logits) | (logits == float("inf"))).sum(-1)


def top_p_mask_exact_max(logits: torch.Tensor, top_p: torch.Tensor, iters: int = 18) -> torch.Tensor:
    """Keep mask of the smallest set of tokens whose probability mass reaches ``top_p``.

    The softmax is shifted by the exact row maximum. The pivot (smallest kept probability) is found by bisection on the
    probability threshold: at most ``iters`` passes over a row, no sort. Tokens tied with the pivot are all kept.
    """
    z = logits.float()
    z = z - z.max(dim=-1, keepdim=True).values
    e = z.exp()
    p = e / e.sum(-1, keepdim=True)
    lo = torch.zeros(p.shape[0], 1, device=p.device)
    hi = p.max(dim=-1, keepdim=True).values
    tp = top_p.reshape(-1, 1).to(p.device).float()
    for _ in range(iters):
        mid = 0.5 * (lo + hi)
        mass = torch.where(p >= mid, p, torch.zeros_like(p)).sum(-1, keepdim=True)
        ok = mass >= tp  # threshold can still rise
        lo = torch.where(ok, mid, lo)
        hi = torch.where(ok, hi, mid)
    keep = p >= lo
    return keep | (tp >= 1.0)


def sample(logits: torch.Tensor, temperature: torch.Tensor | float = 1.0, top_p: torch.Tensor | float = 1.0, top_k: int = -1,
           topk_logprobs: int = 0, generator: Optional[torch.Generator] = None, noise: Optional[torch.Tensor] = None) -> SampleOutput:
    """Exponential-race sampling ``argmax(log p - log(-log u))`` from the processed distribution (temperature, then
    top-k / top-p). ``temperature`` 0 means greedy. Log-probs are those of the processed distribution."""
    n, v = logits.shape
    if logits.is_cuda and n > 0:
        fast = _fused_sample_cuda(logits, temperature, top_p, top_k, topk_logprobs, generator, noise)
        if fast is not None:
            return fast
    nonfinite = count_nonfinite(logits)
    t = torch.as_tensor(temperature, dtype=torch.float32, device=logits.device).expand(n).reshape(n, 1)
    greedy = t <= 0
    z = logits.float() / torch.where(greedy, torch.ones_like(t), t)
    if top_k and top_k > 0 and top_k < v:
        kth = torch.topk(z, top_k, dim=-1).values[:, -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    tp = torch.as_tensor(top_p, dtype=torch.float32, device=logits.device).expand(n)
    if bool((tp < 1.0).any()):
        z = z.masked_fill(~top_p_mask_exact_max(z, tp), float("-inf"))
    logp = torch.log_softmax(z, dim=-1)
    if noise is None:
        noise = torch.rand(n, v, device=logits.device, generator=generator)
    gumbel = -torch.log(-torch.log(noise.clamp(1e-20, 1.0 - 1e-7)))
    tok = torch.where(greedy.squeeze(1), logp.argmax(-1), (logp + gumbel).argmax(-1))
    tok_lp = logp.gather(-1, tok[:, None]).squeeze(-1)
    ranks = (logp > tok_lp[:, None]).sum(-1) + 1
    top_id = top_lp = None
    if topk_logprobs > 0:
        top_lp, top_id = torch.topk(logp, min(topk_logprobs, v), dim=-1)
    return SampleOutput(tok, tok_lp, top_id, top_lp, ranks, nonfinite)


def _scalar(x) -> Optional[float]:
    if isinstance(x, (int, float)):
        return float(x)
    if torch.is_tensor(x) and x.numel() == 1:
        return float(x.item())
    return None


def _fused_sample_cuda(logits, temperature, top_p, top_k, topk_logprobs, generator, noise) -> Optional[SampleOutput]:
    """Temperature (and top-p) rows on a GPU go through the exact-max top-p kernel and the fused CUDA sampler (two or three
    launches instead of dozens of torch ops over the vocabulary); anything else (greedy, top-k, per-row temperatures) takes
    the general path."""
    t = _scalar(temperature)
    if t is None or t <= 0 or (top_k and top_k > 0) or topk_logprobs > 32:
        return None
    from ..ops import rollout_ops

    n, v = logits.shape
    if noise is None:
        noise = torch.rand(n, v, device=logits.device, generator=generator)
    x = logits.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    tp = _scalar(top_p)
    if tp is None or tp < 1.0:  # nucleus rows: the exact-max top-p kernel masks a private copy, the sampler then renormalises
        if x.data_ptr() == logits.data_ptr():
            x = x.clone()
        tpt = top_p.to(x.device, torch.float32).reshape(-1).contiguous() if torch.is_tensor(top_p) else torch.full((n,), float(tp), device=x.device)
        if tpt.numel() == 1 and n > 1:
            tpt = tpt.expand(n).contiguous()
        rollout_ops.top_p_mask_(x, tpt, t)
    k = max(1, topk_logprobs)
    tok, lp, tid, tlp, rank, nf = rollout_ops.fused_sample(x, t, noise.contiguous(), k)
    return SampleOutput(tok, lp, tid if topk_logprobs > 0 else None, tlp if topk_logprobs > 0 else None, rank, nf)


@dataclass
class VerifyOutput:
    accepted: torch.Tensor  # [R] number of accepted drafts per request
    tokens: torch.Tensor  # [R, D + 1] accepted drafts then the recovered / bonus token (rest -1)
    logprobs: torch.Tensor  # [R, D + 1] target log-probs of the emitted tokens
    topk_ids: Optional[torch.Tensor]  # [R, D + 1, k]
    topk_logprobs: Optional[torch.Tensor]


def verify_greedy_drafts(logits: torch.Tensor, drafts: torch.Tensor, temperature: float = 1.0, topk_logprobs: int = 0,
                         generator: Optional[torch.Generator] = None, uniforms: Optional[torch.Tensor] = None,
                         noise: Optional[torch.Tensor] = None) -> VerifyOutput:
    """Lossless rejection sampling of GREEDY (point-mass) drafts.

    logits: [R, D + 1, V] target logits at the rows [x0, d1 .. dD]; drafts: [R, D]. Draft ``d_i`` is accepted with
    probability ``p_i(d_i)`` (``log u < lp(d)``); at the first rejection the token is resampled from ``p_i`` with
    ``d_i`` removed; when every draft is accepted a bonus token is sampled from the last row. Every emitted position is
    distributed exactly as the target model would have sampled it.
    """
    r, d1, v = logits.shape
    d = d1 - 1
    z = logits.float() / max(temperature, 1e-6)
    logp = torch.log_softmax(z, dim=-1)
    if uniforms is None:
        uniforms = torch.rand(r, d, device=logits.device, generator=generator)
    lp_draft = logp[:, :d].gather(-1, drafts.long()[..., None]).squeeze(-1) if d > 0 else logp.new_zeros(r, 0)
    ok = torch.log(uniforms.clamp_min(1e-30)) < lp_draft
    accepted = torch.cumprod(ok.long(), dim=1).sum(1) if d > 0 else torch.zeros(r, dtype=torch.long, device=logits.device)
    # resample at row `accepted` with that row's draft excluded (the bonus row has nothing to exclude)
    rows = logp[torch.arange(r, device=logits.device), accepted]  # [R, V]
    excl = torch.where(accepted < d, drafts.long().gather(1, accepted.clamp(max=max(d - 1, 0))[:, None]).squeeze(1) if d > 0
                       else torch.zeros_like(accepted), torch.full_like(accepted, -1))
    masked = rows.clone()
    has = excl >= 0
    if bool(has.any()):
        masked[has, excl[has]] = float("-inf")
    if noise is None:
        noise = torch.rand(r, v, device=logits.device, generator=generator)
    gumbel = -torch.log(-torch.log(noise.clamp(1e-20, 1.0 - 1e-7)))
    new_tok = (masked + gumbel).argmax(-1)
    tokens = torch.full((r, d1), -1, dtype=torch.long, device=logits.device)
    lps = torch.zeros(r, d1, device=logits.device)
    for i in range(d):
        take = accepted > i
        tokens[take, i] = drafts.long()[take, i]
        lps[take, i] = lp_draft[take, i]
    ar = torch.arange(r, device=logits.device)
    tokens[ar, accepted] = new_tok
    lps[ar, accepted] = rows.gather(-1, new_tok[:, None]).squeeze(-1)
    top_id = top_lp = None
    if topk_logprobs > 0:
        top_lp, top_id = torch.topk(logp, min(topk_logprobs, v), dim=-1)
    return VerifyOutput(accepted, tokens, lps, top_id, top_lp)

"""GRPO math: group advantages, DAPO's dynamic-sampling filter, REINFORCE loss and score centering.

Score centering (upstream ``3rdparty/verl/patches/0011-*.patch``, ``verl/trainer/ppo/score_centering.py``): the
sampler's top-k head ``H`` is known exactly and its tail is modelled as the trainer's tail rescaled to the sampler's tail
mass, so the centering term only needs the trainer's log-probs at the k head ids:

    correction = sum_{j in H} sg[ q_j w(p_j / q_j) - alpha p_j ] log p_j,
    rho = (1 - sum q) / (1 - sum p),  alpha = rho * w(1 / rho)

with ``q`` the sampler's and ``p`` the trainer's probabilities, ``w`` the token-level importance-weight rule (identity
weight 1 without IS) and ``sg`` stop-gradient. The per-token loss is ``-A log pi(y) + A * correction`` aggregated as a
token mean (``pear/configs/training.yaml:13-26``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch


# ---------------------------------------------------------------------------------------------------------------------
# advantages and group filter
# ---------------------------------------------------------------------------------------------------------------------
def group_advantages(rewards: torch.Tensor, norm_by_std: bool = True, eps: float = 1e-6) -> torch.Tensor:
    """``rewards`` [groups, n] -> advantages [groups, n]: centred per group (and divided by the group's std)."""
    r = rewards.float()
    mean = r.mean(dim=1, keepdim=True)
    adv = r - mean
    if norm_by_std:
        adv = adv / (r.std(dim=1, keepdim=True, unbiased=False) + eps)
    return adv


def filter_groups(rewards: torch.Tensor) -> torch.Tensor:
    """DAPO dynamic sampling: a group whose rewards have no variance carries no gradient and is dropped. Returns the
    keep mask [groups]."""
    return (rewards.max(dim=1).values - rewards.min(dim=1).values) > 0


def pass_rate_metrics(rewards: torch.Tensor, prefix: str = "filter_groups") -> dict[str, float]:
    """avg@n and the shares of all-zero / all-one groups (upstream ``pear/trainer/replay_buffer.py:93-113``)."""
    n = rewards.shape[1]
    ok = (rewards > 0).float()
    solved = ok.sum(1)
    return {
        f"{prefix}/avg@n": float(ok.mean()) if rewards.numel() else 0.0,  # (the key says "n" literally, whatever the group size: dashboards keep one series)
        f"{prefix}/passrate/zero": float((solved == 0).float().mean()) if rewards.numel() else 0.0,
        f"{prefix}/passrate/one": float((solved == n).float().mean()) if rewards.numel() else 0.0,
    }


# ---------------------------------------------------------------------------------------------------------------------
# importance-weight rules shared by the head and the sampled token
# ---------------------------------------------------------------------------------------------------------------------
def weight_rule(rollout_is: Optional[str], threshold: str | float = 2.0) -> Callable[[torch.Tensor], torch.Tensor]:
    """``None``: weight 1. ``"token"``: a single number upper-clamps the ratio (TIS); ``"lo_hi"`` zeroes ratios outside
    the band (IcePop)."""
    if rollout_is is None:
        return torch.ones_like
    if rollout_is != "token":
        raise ValueError(f"score centering composes with token-level IS only, got {rollout_is!r}")
    if isinstance(threshold, str) and "_" in threshold:
        lo, hi = (float(x) for x in threshold.split("_"))
        return lambda ratio: torch.where((ratio >= lo) & (ratio <= hi), ratio, torch.zeros_like(ratio))
    hi = float(threshold)
    return lambda ratio: ratio.clamp(max=hi)


def score_centering_correction(train_head_lp: torch.Tensor, sampler_head_lp: torch.Tensor,
                               w: Callable[[torch.Tensor], torch.Tensor] = torch.ones_like, eps: float = 1e-6):
    """Per-token centering term and the two head masses. ``*_head_lp``: [N, k] full-vocab-normalised log-probs at the
    sampler's head ids; only ``train_head_lp`` carries gradient."""
    lp = train_head_lp.float()
    with torch.no_grad():
        p, q = lp.exp(), sampler_head_lp.float().exp()
        p_mass, q_mass = p.sum(-1), q.sum(-1)
        rho = (1 - q_mass).clamp_min(eps) / (1 - p_mass).clamp_min(eps)
        alpha = rho * w(1.0 / rho)
        coeff = q * w((lp - sampler_head_lp.float()).exp()) - alpha.unsqueeze(-1) * p
    return (coeff * lp).sum(-1), q_mass, p_mass


def uniform_head(num_rows: int, k: int, device=None):
    """Placeholder head for rows the loss masks out (prompt / observation tokens): ids 0..k-1 with log-prob -log k."""
    ids = torch.arange(k, dtype=torch.int32, device=device).expand(num_rows, k).clone()
    lp = torch.full((num_rows, k), -float(torch.log(torch.tensor(float(k)))), dtype=torch.float32, device=device)
    return ids, lp


# ---------------------------------------------------------------------------------------------------------------------
# loss
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class LossConfig:
    loss_agg_mode: str = "token-mean"
    score_centering: bool = True
    rollout_is: Optional[str] = None
    rollout_is_threshold: str | float = 2.0
    entropy_coeff: float = 0.0


def policy_loss(log_probs: torch.Tensor, advantages: torch.Tensor, mask: torch.Tensor, cfg: LossConfig,
                head_log_probs: Optional[torch.Tensor] = None, sampler_head_log_probs: Optional[torch.Tensor] = None,
                sampler_log_probs: Optional[torch.Tensor] = None, entropy: Optional[torch.Tensor] = None,
                denominator: Optional[torch.Tensor] = None):
    """Bypass-mode REINFORCE over packed tokens.

    log_probs, advantages, mask: [N] (mask 1 on generated tokens). ``denominator``: the global number of loss tokens
    (a tensor, so a micro-batch of a larger batch normalises by the batch's token count); default: this call's.
    Returns (loss, metrics).
    """
    maskf = mask.float()
    denom = denominator.float() if denominator is not None else maskf.sum().clamp_min(1.0)
    w = weight_rule(cfg.rollout_is, cfg.rollout_is_threshold)
    per_token = -advantages.float() * log_probs.float()
    metrics: dict[str, float] = {}
    if cfg.rollout_is is not None and sampler_log_probs is not None:
        with torch.no_grad():
            is_w = w((log_probs.float() - sampler_log_probs.float()).exp())
        per_token = per_token * is_w
    if cfg.score_centering and head_log_probs is not None:
        corr, q_mass, p_mass = score_centering_correction(head_log_probs, sampler_head_log_probs, w)
        per_token = per_token + advantages.float() * corr
        n = maskf.sum().clamp_min(1.0)
        metrics["actor/sc_correction"] = float((corr.detach() * maskf).sum() / n)
        metrics["actor/sc_sampler_head_mass"] = float((q_mass * maskf).sum() / n)
        metrics["actor/sc_train_head_mass"] = float((p_mass * maskf).sum() / n)
    if cfg.entropy_coeff and entropy is not None:
        per_token = per_token - cfg.entropy_coeff * entropy.float()
    if cfg.loss_agg_mode == "token-mean":
        loss = (per_token * maskf).sum() / denom
    elif cfg.loss_agg_mode == "seq-mean-token-sum":
        loss = (per_token * maskf).sum() / denom
    else:
        raise ValueError(f"unknown loss_agg_mode {cfg.loss_agg_mode}")
    n = maskf.sum().clamp_min(1.0)
    metrics["actor/pg_loss"] = float(loss.detach())
    if sampler_log_probs is not None:
        with torch.no_grad():
            kl = ((sampler_log_probs.float() - log_probs.float()) * maskf).sum() / n
        metrics["actor/ppo_kl"] = float(kl)
    if entropy is not None:
        metrics["actor/entropy"] = float((entropy.detach().float() * maskf).sum() / n)
    return loss, metrics

"""Goodness of fit of the batched step's sampler at the real vocabulary size: with greedy drafts and rejection sampling the
first committed token of every sequence must follow softmax(logits / T) exactly, whatever the drafter proposed
(upstream: tests/rollout/test_rejection_sampler_on_gpu.py — 400 000 verify steps, goodness of fit)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _chi2_sf(x: float, k: int) -> float:
    """Upper tail of the chi-square distribution with k degrees of freedom (regularised incomplete gamma, series / fraction)."""
    a, xx = k / 2.0, x / 2.0
    if xx <= 0:
        return 1.0
    if xx < a + 1:  # series for P, return 1 - P
        term = 1.0 / a
        s = term
        n = a
        for _ in range(10000):
            n += 1
            term *= xx / n
            s += term
            if abs(term) < abs(s) * 1e-15:
                break
        return max(0.0, 1.0 - s * math.exp(-xx + a * math.log(xx) - math.lgamma(a)))
    b = xx + 1 - a  # continued fraction for Q
    c = 1e300
    d = 1.0 / b
    h = d
    for i in range(1, 10000):
        an = -i * (i - a)
        b += 2
        d = an * d + b
        d = 1e-300 if abs(d) < 1e-300 else d
        c = b + an / c
        c = 1e-300 if abs(c) < 1e-300 else c
        d = 1.0 / d
        delta = d * c
        h *= delta
        if abs(delta - 1) < 1e-15:
            break
    return h * math.exp(-xx + a * math.log(xx) - math.lgamma(a))


@pytest.mark.timeout(300)
def test_first_committed_token_follows_the_target_distribution():
    from pear_b200.ops import decode_ops as K

    V, B, T, chunks, temp, seed = 248320, 64, 2, 2, 0.9, 4242
    # eight tokens carry almost all of the mass; they sit in different sampler chunks and at chunk edges
    support = [0, 1, 7, 31000, 62079, 62080, 124160, 248319]
    probs = torch.tensor([0.30, 0.22, 0.15, 0.11, 0.09, 0.06, 0.04, 0.03], dtype=torch.float64)
    logits_row = torch.full((V,), -40.0, device="cuda")
    logits_row[support] = (torch.log(probs) * temp).float().cuda()  # softmax(logits / temp) = probs (the rest adds ~1e-12)
    logits = logits_row.repeat(B * T, 1).contiguous()
    i32 = dict(dtype=torch.int32, device="cuda")
    recs = torch.zeros(B * T * chunks * K.rec_bytes(), dtype=torch.uint8, device="cuda")
    ptrs = K._ptr_array([recs.data_ptr()])
    step_ctr = torch.zeros(1, **i32)
    ncommit, parity = torch.zeros(B, **i32), torch.zeros(B, **i32)
    out_tok, out_lp = torch.zeros(B, T, **i32), torch.zeros(B, T, device="cuda")
    n_acc, nonf, sel, mtp_tok, mtp_ctx = torch.zeros(B, **i32), torch.zeros(B, **i32), torch.zeros(B, **i32), torch.zeros(B * T, **i32), torch.zeros(T, B, **i32)
    counts = torch.zeros(V, dtype=torch.int64, device="cuda")
    accepted = 0
    steps = 1600  # 102 400 samples
    drafts = [support[0], support[3], support[7], 5]  # the mode, a mid token, the rarest, a token of (almost) zero mass
    for step in range(steps):
        tok_in = torch.zeros(B * T, **i32)
        tok_in[1::T] = drafts[step % len(drafts)]  # row 0's draft
        ctx = torch.full((B,), 100, **i32)
        K.verify_chunks(logits, V, 0, temp, tok_in, ctx, B, T, chunks, seed, step_ctr, ptrs, 0, 1, None, 0)
        K.verify_finish(recs, 0, None, 1, chunks, B, T, seed, step_ctr, tok_in, ctx, ncommit, parity, out_tok, out_lp, n_acc, nonf, sel, mtp_tok, mtp_ctx)
        counts += torch.bincount(out_tok[:, 0].long(), minlength=V)
        accepted += int((n_acc > 0).sum())
    torch.cuda.synchronize()
    K.check_status()
    n = B * steps
    assert int(counts.sum()) == n
    obs = counts[support].double().cpu()
    assert int(obs.sum()) >= n - 2  # the remaining 248 312 tokens hold ~1e-12 of the mass
    exp = probs * n
    chi2 = float(((obs - exp) ** 2 / exp).sum())
    p_value = _chi2_sf(chi2, len(support) - 1)
    assert p_value > 1e-6, (chi2, p_value, obs.tolist(), exp.tolist())
    # drafts were accepted with the probability of the drafted token, on average over the four drafts used
    want_acc = float(probs[0] + probs[3] + probs[7] + 0.0) / 4
    assert abs(accepted / n - want_acc) < 5 * math.sqrt(want_acc * (1 - want_acc) / n), (accepted / n, want_acc)

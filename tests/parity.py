"""Helpers shared by the parity tests: comparison of a decode result against the CPU checker."""
from __future__ import annotations

import numpy as np

RTOL_FP32 = 1e-4   # per-step log-probabilities, relative (fp32 weights)
ATOL_BF16 = 2e-2   # per-step log-probabilities, absolute (bf16 weights, fp32 accumulate)


def hyps(out, i, q=0):
    n = int(out["len"][i, q])
    return list(out["tok"][i, q, :n])


def token_identity(a, b, n):
    """Fraction of sentences whose 1-best token sequences are identical."""
    same = sum(1 for i in range(n) if hyps(a, i) == hyps(b, i))
    return same / max(n, 1)


def compare_forced(eng, ora, steps, rtol=RTOL_FP32, atol=0.0, pt_eps=5e-4, src_len=None, D=10, t_lo=0, t_hi=None):
    """Engine ran with its beam forced to the checker's survivors: every step's per-beam
    top-(k+1) must then agree.

    The reference's local attention cuts its window at ``(int)p_t`` (src/deep_rnn_kernel.h:1094-1100),
    a step function of a float: two correct implementations that sum in different orders can
    land on different sides when p_t is within rounding noise of an integer, and the attentional
    state then feeds every descendant of that hypothesis.  When the checker's p_t is within
    ``pt_eps`` of an integer n whose window edge lies inside the sentence (n > D or n + D < S),
    the hypothesis and its descendants are left out of the comparison (and counted); everything
    else must agree.

    Only steps t_lo <= t < t_hi are compared (all by default).  On the seeded random weights the
    recurrence amplifies rounding noise by about 2x every 10 steps (the fp32 checker against the
    float64 restatement: 1e-6 at step 0, 1e-4 near step 70, 1e-2 near step 150), so the fp32
    tolerance can only be asked of the first ~60 steps of a long sentence.

    Returns (max relative log-prob error, mismatches that are not near-ties, row-steps left out,
    row-steps compared)."""
    n, Tm, k, kk = ora["cand_tok"].shape
    pt = ora.get("pt") if isinstance(ora, dict) else None
    if pt is not None and not np.any(pt != 0):
        pt = None  # global attention: no window
    worst, bad, skipped, compared = 0.0, 0, 0, 0
    for i in range(n):
        taint = np.zeros(k, bool)
        for t in range(int(steps[i])):
            if pt is not None:
                nn = np.round(pt[i, t])
                frac = np.abs(pt[i, t] - nn)
                S = int(src_len[i]) if src_len is not None else 10 ** 9
                taint = taint | ((frac < pt_eps) & ((nn > D) | (nn + D < S)))
            cols = 1 if t == 0 else k
            if t < t_lo or (t_hi is not None and t >= t_hi):
                cols = 0
            for b in range(cols):
                if taint[b]:
                    skipped += 1
                    continue
                compared += 1
                lo, le = ora["cand_logp"][i, t, b], eng["cand_logp"][i, t, b]
                to, te = ora["cand_tok"][i, t, b], eng["cand_tok"][i, t, b]
                err = np.abs(lo - le) / np.maximum(np.abs(lo), 1e-6)
                tol_hit = (err <= rtol) | (np.abs(lo - le) <= atol)
                worst = max(worst, float(err.max()))
                bad += int((~tol_hit).sum())
                if (to != te).any():
                    # a swap is acceptable only between candidates whose log-probs are within tolerance
                    for q in np.nonzero(to != te)[0]:
                        gap_ok = False
                        for q2 in range(kk):
                            if te[q] == to[q2] and abs(lo[q2] - lo[q]) <= max(rtol * abs(lo[q]), atol) * 2:
                                gap_ok = True
                        if not gap_ok:
                            # another token of the same value at the same rank: a tie, or (last slots) a
                            # token from just beyond the other side's list on a nearly flat distribution
                            gap_ok = abs(le[q] - lo[q]) <= max(rtol * abs(lo[q]), atol) * 2
                        if not gap_ok:
                            bad += 1
            # survivors inherit the taint of their parent (all k slots start identical at step 0)
            par = ora["surv_parent"][i, t]
            taint = taint[np.clip(par, 0, k - 1)] if t > 0 else np.repeat(taint[0], k)
    return worst, bad, skipped, compared

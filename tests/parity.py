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


def compare_forced(eng, ora, steps, rtol=RTOL_FP32, atol=0.0):
    """Engine ran with its beam forced to the checker's survivors: every step's per-beam
    top-(k+1) must then agree.  Returns (max relative log-prob error, number of candidate
    index mismatches that are not near-ties)."""
    n, Tm, k, kk = ora["cand_tok"].shape
    worst = 0.0
    bad = 0
    for i in range(n):
        for t in range(int(steps[i])):
            cols = 1 if t == 0 else k
            for b in range(cols):
                lo, le = ora["cand_logp"][i, t, b], eng["cand_logp"][i, t, b]
                to, te = ora["cand_tok"][i, t, b], eng["cand_tok"][i, t, b]
                err = np.abs(lo - le) / np.maximum(np.abs(lo), 1e-6)
                tol_hit = (err <= rtol) | (np.abs(lo - le) <= atol)
                worst = max(worst, float(err.max()))
                if not tol_hit.all():
                    bad += int((~tol_hit).sum())
                if (to != te).any():
                    # a swap is acceptable only between candidates whose log-probs are within tolerance
                    for q in np.nonzero(to != te)[0]:
                        gap_ok = False
                        for q2 in range(kk):
                            if te[q] == to[q2] and abs(lo[q2] - lo[q]) <= max(rtol * abs(lo[q]), atol) * 2:
                                gap_ok = True
                        if q == kk - 1 and not gap_ok:
                            # the last slot may hold the (k+2)-th value of the other side
                            gap_ok = abs(le[q] - lo[q]) <= max(rtol * abs(lo[q]), atol) * 2
                        if not gap_ok:
                            bad += 1
    return worst, bad

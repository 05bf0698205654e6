"""Helpers shared by the parity tests: comparison of a decode result against the CPU checker."""
from __future__ import annotations

import numpy as np

RTOL_FP32 = 1e-4   # per-step log-probabilities, relative (fp32 weights)
ATOL_BF16 = 2e-2   # per-step log-probabilities, absolute (bf16 weights, fp32 accumulate)


def hyps(out, i, q=0):
    n = int(out["len"][i, q])
    return list(out["tok"][i, q, :n])


def _members(pt):
    """p_t records with the member axis in front: [M][n][T+1][k] (one model: [n][T+1][k] -> [1][n][T+1][k])."""
    return pt if pt.ndim == 4 else pt[None]


def window_flip(pt_e, pt_o, S, D=10, pt_tol=2e-3, t=0):
    """True where the two implementations cut the local-attention window on different sides of an
    integer although their centres p_t agree to rounding noise: ``(int)p_t`` differs, the two p_t
    are within the noise bound of each other, and the shifted window edge lies inside the sentence.

    The noise bound is ``pt_tol`` for the first 60 forwards of a sentence and doubles every 10 forwards
    after that: the recurrence amplifies rounding noise by about 2x every 10 steps (see compare_forced),
    and p_t = S * sigmoid(.) carries it times the sentence length (measured: engine against checker
    2e-5 at forward 72 of one C2 sentence, 2e-3 to 3e-3 at forwards 73-76 of others)."""
    fe, fo = np.floor(pt_e), np.floor(pt_o)
    hi = np.maximum(fe, fo)
    inside = (hi > D) | (hi + D < S)   # an edge that moved: lo = n - D > 0 or hi = n + D < S - 1 (+1 for the larger n)
    tol = pt_tol * 2.0 ** (max(0, t - 60) / 10.0)
    return (fe != fo) & (np.abs(pt_e - pt_o) <= tol) & inside


def compare_forced(eng, ora, steps, rtol=RTOL_FP32, atol=0.0, pt_eps=5e-4, src_len=None, D=10, t_lo=0, t_hi=None):
    """Engine ran with its beam forced to the checker's survivors: every step's per-beam
    top-(k+1) must then agree.

    The reference's local attention cuts its window at ``(int)p_t`` (src/deep_rnn_kernel.h:1094-1100),
    a step function of a float: two correct implementations that sum in different orders can
    land on different sides when p_t is within rounding noise of an integer, and the attentional
    state then feeds every descendant of that hypothesis.  When the checker's p_t is within
    ``pt_eps`` of an integer n whose window edge lies inside the sentence (n > D or n + D < S),
    the hypothesis and its descendants are left out of the comparison (and counted); everything
    else must agree.  When the engine's own p_t record is there (``eng["pt"]``) the rule is exact
    instead: a hypothesis is left out from the forward on where the two ``(int)p_t`` really differ
    while the two p_t agree to rounding noise (``window_flip``).

    Only steps t_lo <= t < t_hi are compared (all by default).  On the seeded random weights the
    recurrence amplifies rounding noise by about 2x every 10 steps (the fp32 checker against the
    float64 restatement: 1e-6 at step 0, 1e-4 near step 70, 1e-2 near step 150), so the fp32
    tolerance can only be asked of the first ~60 steps of a long sentence.

    The tolerance of a row's entries is relative to the LARGEST magnitude among the row's k+1 checker
    log-probabilities: every entry is a difference of logits of the same scale, so its error is
    commensurate with that scale, not with its own value -- on a peaked row the best candidate's
    log-probability is close to zero and no fp32 computation holds 1e-4 of THAT.  (On the flat rows of
    the named configurations all k+1 values are within a few percent of each other and the two readings
    coincide.)  Where both sides carry ``final_logp`` (log p(EOS) of every beam at the closing forward)
    it is compared the same way, for the beams still in the comparison, at the row scale of the last step.

    Returns (max relative log-prob error, mismatches that are not near-ties, row-steps left out,
    row-steps compared)."""
    n, Tm, k, kk = ora["cand_tok"].shape
    pt = ora.get("pt") if isinstance(ora, dict) else None
    if pt is not None and not np.any(pt != 0):
        pt = None  # global attention: no window
    ept = eng.get("pt") if (isinstance(eng, dict) and pt is not None) else None
    worst, bad, skipped, compared = 0.0, 0, 0, 0
    for i in range(n):
        taint = np.zeros(k, bool)
        for t in range(int(steps[i])):
            if ept is not None:
                S = int(src_len[i]) if src_len is not None else 10 ** 9
                for pe_, po_ in zip(_members(ept), _members(pt)):   # any member of an ensemble
                    taint = taint | window_flip(pe_[i, t], po_[i, t], S, D, t=t)
            elif pt is not None:
                S = int(src_len[i]) if src_len is not None else 10 ** 9
                for po_ in _members(pt):
                    nn = np.round(po_[i, t])
                    frac = np.abs(po_[i, t] - nn)
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
                scale = max(float(np.abs(lo[np.isfinite(lo)]).max()), 1e-6)
                err = np.abs(lo - le) / scale
                tol_hit = (err <= rtol) | (np.abs(lo - le) <= atol)
                worst = max(worst, float(err.max()))
                bad += int((~tol_hit).sum())
                if (to != te).any():
                    # a swap is acceptable only between candidates whose log-probs are within tolerance
                    for q in np.nonzero(to != te)[0]:
                        gap_ok = False
                        for q2 in range(kk):
                            if te[q] == to[q2] and abs(lo[q2] - lo[q]) <= max(rtol * scale, atol) * 2:
                                gap_ok = True
                        if not gap_ok:
                            # another token of the same value at the same rank: a tie, or (last slots) a
                            # token from just beyond the other side's list on a nearly flat distribution
                            gap_ok = abs(le[q] - lo[q]) <= max(rtol * scale, atol) * 2
                        if not gap_ok:
                            bad += 1
            # survivors inherit the taint of their parent (all k slots start identical at step 0)
            par = ora["surv_parent"][i, t]
            taint = taint[np.clip(par, 0, k - 1)] if t > 0 else np.repeat(taint[0], k)
        T = int(steps[i])
        if "final_logp" in ora and "final_logp" in eng and ora["final_logp"] is not None and T > 0 and (t_hi is None or T < t_hi) and T >= t_lo:
            if ept is not None:
                S = int(src_len[i]) if src_len is not None else 10 ** 9
                for pe_, po_ in zip(_members(ept), _members(pt)):
                    taint = taint | window_flip(pe_[i, T], po_[i, T], S, D, t=T)
            fo, fe = ora["final_logp"][i], eng["final_logp"][i]
            # the scale of the closing forward's rows: the largest candidate magnitude of the last expansion
            scale = max(float(np.abs(ora["cand_logp"][i, T - 1][np.isfinite(ora["cand_logp"][i, T - 1])]).max()), float(np.abs(fo).max()), 1e-6)
            for b in range(k):
                if taint[b]:
                    skipped += 1
                    continue
                compared += 1
                e_ = abs(float(fo[b]) - float(fe[b]))
                worst = max(worst, e_ / scale)
                if e_ > rtol * scale and e_ > atol:
                    bad += 1
    return worst, bad, skipped, compared


def explain_divergences(free, ora, sents, k, rtol=RTOL_FP32, D=10, atol_step=0.0):
    """Free-running engine output against the checker's trace of the same decode: every sentence
    whose 1-best differs must part ways with the checker at a choice that is a tie within
    tolerance in the checker's OWN numbers -- the engine's survivor of some rank is a candidate the
    checker scored within ``rtol`` (relative to the score) of the checker's survivor of that rank
    -- or after a local-attention window was cut on the other side of an integer (``window_flip``).
    Anything else is returned as unexplained.  ``atol_step`` widens the tie criterion by that much per
    decoder step taken (the bf16 bar is an absolute tolerance per step's log-probabilities, and a
    score is their sum).

    ``free`` needs the engine's trace (surv_tok, surv_parent, surv_score, pt), ``ora`` the
    checker's (cand_tok, cand_logp, surv_*, pt).  Returns (identical, explained, unexplained)
    lists of sentence indices; explained entries are (i, step, reason)."""
    identical, explained, unexplained = [], [], []
    lens = sents.lengths()
    has_pt = ora.get("pt") is not None and np.any(ora["pt"] != 0) and free.get("pt") is not None
    for i in range(sents.n):
        if hyps(free, i) == hyps(ora, i):
            identical.append(i)
            continue
        T, S = int(sents.steps[i]), int(lens[i])
        reason = None
        flipped = np.zeros(k, bool)   # engine slot descends from a forward with a window flip
        for t in range(T):
            if has_pt:
                for pe_, po_ in zip(_members(free["pt"]), _members(ora["pt"])):
                    flipped = flipped | window_flip(pe_[i, t], po_[i, t], S, D, t=t)
            et, ep = free["surv_tok"][i, t], free["surv_parent"][i, t]
            ot, op, osc = ora["surv_tok"][i, t], ora["surv_parent"][i, t], ora["surv_score"][i, t]
            if (et == ot).all() and (ep == op).all():
                flipped = flipped[np.clip(ep, 0, k - 1)] if t > 0 else np.repeat(flipped[0], k)
                continue
            if flipped.any():
                reason = (i, t, "window flip")
                break
            # first step with another choice: every engine survivor must be a candidate the checker scored
            # within tolerance of the checker's survivor of the same rank
            prev = ora["surv_score"][i, t - 1] if t > 0 else np.zeros(k, np.float32)
            ok = True
            for r in range(k):
                if et[r] == ot[r] and ep[r] == op[r]:
                    continue
                b = int(ep[r])
                hit = np.nonzero(ora["cand_tok"][i, t, b] == et[r])[0]
                if len(hit) == 0:
                    ok = False
                    break
                sc = prev[b] + ora["cand_logp"][i, t, b, hit[0]]
                if abs(sc - osc[r]) > rtol * abs(osc[r]) + atol_step * (t + 1):
                    ok = False
                    break
            reason = (i, t, "tie within tolerance") if ok else None
            if not ok:
                unexplained.append((i, t))
            break
        else:
            # the beams agree at every step: the finished lists can still order two hypotheses of (nearly) the
            # same final score differently
            a, b = float(free["score"][i, 0]), float(ora["score"][i, 0])
            if abs(a - b) <= rtol * abs(b) + atol_step * (T + 1):
                reason = (i, T, "final scores tie")
            else:
                unexplained.append((i, T))
        if reason:
            explained.append(reason)
    return identical, explained, unexplained

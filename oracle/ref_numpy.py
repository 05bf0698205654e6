"""Independent float64 restatement of the decode procedure in numpy (test infrastructure).

Written from the mathematical description of the model (logical matrices ``W @ x``), not from
the memory layout, so it cross-checks the C++ checker's reading of the weight blob as well as
its arithmetic.  One sentence at a time, pure Python loops: small models only.

Follows the same reference procedure: encoder over the reversed sentence
(src/deep_rnn.h:1572-1721), LSTM node (src/node_input_to_hidden.h:218-636,
src/node_hidden_to_hidden.h:194-443), local-p attention (src/layer_attention.h:243-483),
softmax (src/layer_loss.h:797-883), beam expansion (src/decoder.h:355-480), final scoring
(src/decoder.h:502-525, 703-775).
"""
from __future__ import annotations

import numpy as np

from linmt_b200.synth import blob_views

START, EOS = 0, 1


def _sig(x):
    return 1.0 / (1.0 + np.exp(-x))


def _lstm(w, pre, x, h, c, ht=None):
    def gate(g):
        v = w[f"{pre}.M_{g}"] @ x + w[f"{pre}.W_h{g}"] @ h + w[f"{pre}.b_{g}"][:, 0]
        if ht is not None:
            v = v + w[f"{pre}.Q_{g}"] @ ht
        return v
    i, f, o, g = _sig(gate("i")), _sig(gate("f")), _sig(gate("o")), np.tanh(gate("c"))
    c2 = f * c + i * g
    return o * np.tanh(c2), c2


def decode_sentence(desc, blob, ids, T, *, beam, attention="local_p_general", D=10, penalty=0.0, diversity=0.0,
                    lp_alpha=0.65, cp_beta=0.0, min_ratio=0.5, nbest=1, track_align=False, follow=None):
    """``follow`` = dict(surv_tok, surv_parent, surv_score) of shape [T][k] from another
    implementation: the beam then continues from those survivors (after checking that they are
    a valid choice up to ``follow['tol']``), which makes every step comparable even where fp32
    score ties would make the two searches part ways."""
    w = {k: v.astype(np.float64) for k, v in blob_views(desc, blob).items()}
    L, H, V = desc.L, desc.H, desc.V
    k = min(beam, int(np.floor(np.sqrt(V))))
    rev = list(ids)[::-1]
    S = len(rev)
    h = [np.zeros(H) for _ in range(L)]
    c = [np.zeros(H) for _ in range(L)]
    enc = []
    for tok in rev:
        x = w["src0.W_emb"][:, tok]
        for l in range(L):
            h[l], c[l] = _lstm(w, f"src{l}", x, h[l], c[l])
            x = h[l]
        enc.append(x)
    # position s of the original sentence = encoder step S-1-s
    hs = [enc[S - 1 - s] for s in range(S)]
    hp = [[h[l].copy() for _ in range(k)] for l in range(L)]
    cp_ = [[c[l].copy() for _ in range(k)] for l in range(L)]
    htil = [np.zeros(H) for _ in range(k)]
    tok = [START] * k
    score = [0.0] * k
    hist = [[START] for _ in range(k)]
    hal = [[np.zeros(S)] for _ in range(k)]
    finished = []
    logps = []
    for t in range(T + 1):
        newh = [[None] * k for _ in range(L)]
        newc = [[None] * k for _ in range(L)]
        newt = [None] * k
        lp = [None] * k
        al = [None] * k
        for b in range(k):
            x = w["tgt0.W_emb"][:, tok[b]]
            for l in range(L):
                ht = htil[b] if (l == 0 and desc.feed_input and t != 0) else None
                newh[l][b], newc[l][b] = _lstm(w, f"tgt{l}", x, hp[l][b], cp_[l][b], ht)
                x = newh[l][b]
            top = x
            if attention == "local_p_general":
                pt = S * _sig(w["att.v_p"][:, 0] @ np.tanh(w["att.W_p"] @ top))
                lo, hi = max(0, int(pt) - D), min(S - 1, int(pt) + D)
            else:
                pt, lo, hi = 0.0, 0, S - 1
            u = top if attention == "global_dot" else w["att.W_a"].T @ top
            e = np.array([hs[s] @ u for s in range(lo, hi + 1)])
            m = max(0.0, e.max())
            a = np.exp(e - m)
            a = a / a.sum()
            if attention == "local_p_general":
                a = a * np.exp(-((pt - np.arange(lo, hi + 1)) ** 2) / (2.0 * (D * D / 4.0)))
            ctx = sum(a[j] * hs[lo + j] for j in range(len(a)))
            newt[b] = np.tanh(w["att.W_c1"] @ ctx + w["att.W_c2"] @ top + w["att.b_out"][:, 0])
            z = w["sm.D"] @ newt[b] + w["sm.b_d"][:, 0]
            z = z - z.max()
            lp[b] = z - np.log(np.exp(z).sum())
            dense = np.zeros(S)
            if track_align:
                dense[lo:hi + 1] = a
            al[b] = dense
        logps.append(np.array(lp))
        if t == T:
            for b in range(k):
                finished.append((hist[b] + [EOS], score[b] + lp[b][EOS] + penalty, hal[b] + [al[b]]))
            break
        cand = []
        for b in range(1 if t == 0 else k):
            order = np.lexsort((np.arange(V), -lp[b]))[:k + 1]
            for r, v in enumerate(order):
                cand.append((lp[b][v] + score[b] - (r + 1) * diversity, b, int(v)))
        cand.sort(key=lambda x: (-x[0], x[1], x[2]))
        surv = []
        for sc, b, v in cand:
            if len(surv) == k:
                break
            if v == START:
                continue
            if v == EOS:
                finished.append((hist[b] + [EOS], sc + penalty, hal[b] + [al[b]]))
                continue
            surv.append((sc + penalty, b, v))
        while len(surv) < k:
            surv.append((-1e30, 0, 2))
        if follow is not None:
            tol = follow.get("tol", 1e-4)
            table = {(b, v): sc for sc, b, v in cand}
            kth = surv[-1][0]
            forced = []
            for j in range(k):
                b, v, sc_o = int(follow["surv_parent"][t][j]), int(follow["surv_tok"][t][j]), float(follow["surv_score"][t][j])
                if sc_o <= -1e29:
                    forced.append((-1e30, b, v))
                    continue
                assert (b, v) in table, f"step {t}: survivor ({b},{v}) is not among the float64 candidates"
                mine = table[(b, v)] + penalty
                assert abs(mine - sc_o) <= tol * max(1.0, abs(mine)), (t, j, mine, sc_o)
                assert mine >= kth - tol * max(1.0, abs(kth)), f"step {t}: survivor below the float64 cut"
                forced.append((sc_o, b, v))
            surv = forced
        hist = [hist[b] + [v] for _, b, v in surv]
        hal = [hal[b] + [al[b]] for _, b, _ in surv]
        score = [sc for sc, _, _ in surv]
        tok = [v for _, _, v in surv]
        hp = [[newh[l][b] for _, b, _ in surv] for l in range(L)]
        cp_ = [[newc[l][b] for _, b, _ in surv] for l in range(L)]
        htil = [newt[b] for _, b, _ in surv]
    res = []
    for toks, sc, als in finished:
        n = len(toks)
        if lp_alpha != 0:
            sc = sc / ((5.0 + n) ** lp_alpha / 6.0 ** lp_alpha)
        if cp_beta != 0:
            cov = np.zeros(S)
            for j in range(1, n - 1):
                r = als[j + 1] + 0.01
                cov += r / r.sum()
            cpv = cp_beta * np.log(np.minimum(cov, 1.0)).sum()
            sc += max(cpv, -20.0)
        if n / S > min_ratio:
            res.append((sc, toks))
    order = sorted(range(len(res)), key=lambda i: (-res[i][0], i))[:nbest]
    return [res[i] for i in order], logps

"""CPU tests of the checker itself: against an independent float64 restatement, against the
committed golden fixtures, and on analytic known-answer cases.  The reference has no tests or
golden vectors of its own, so these are the pins the checker has."""
import os

import numpy as np
import pytest

from linmt_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def c1():
    c = synth.configs()["C1"]
    return c, c.blobs()[0], c.sentences()


def test_blob_layout_size(oracle):
    for d in (synth.ModelDesc(2, 128, 1000, 1000, 1), synth.ModelDesc(4, 1000, 30000, 30000, 1),
              synth.ModelDesc(1, 16, 50, 40, 0)):
        assert synth.blob_floats(d) == oracle.lib().linmt_oracle_blob_floats(d.L, d.H, d.V, d.Vs, d.feed_input)


def test_gemm_matches_float64(oracle):
    rng = np.random.default_rng(0)
    for R, K, N in ((1, 7, 5), (13, 100, 130), (70, 257, 64)):
        X = rng.standard_normal((R, K)).astype(np.float32)
        W = rng.standard_normal((K, N)).astype(np.float32)
        Y = oracle.gemm(X, W)
        ref = X.astype(np.float64) @ W.astype(np.float64)
        assert np.abs(Y - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-5
        # grouping of rows must not change any bit
        Y1 = np.concatenate([oracle.gemm(X[i:i + 1], W) for i in range(R)])
        assert (Y1 == Y).all()


@pytest.mark.parametrize("case", ["c1_greedy", "c1_beam4", "tiny_global"])
def test_golden_fixtures(oracle, c1, case):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    c, blob, sents = c1
    g = np.load(os.path.join(GOLD, case + ".npz"))
    o = oracle.decode(c.desc, [blob], sents, trace=True, **mg.CASES[case])
    assert (o["tok"] == g["tok"]).all() and (o["len"] == g["len"]).all()
    assert (o["surv_tok"] == g["surv_tok"]).all() and (o["surv_parent"] == g["surv_parent"]).all()
    np.testing.assert_allclose(o["score"], g["score"], rtol=2e-6)
    np.testing.assert_allclose(o["cand_logp"], g["cand_logp"], rtol=2e-6, atol=1e-6)


def test_one_at_a_time_equals_batched(oracle, c1):
    c, blob, sents = c1
    a = oracle.decode(c.desc, [blob], sents, beam=4, nbest=2, trace=True)
    b = oracle.decode(c.desc, [blob], sents, beam=4, nbest=2, trace=True, group=1)
    for key in ("tok", "len", "score", "surv_tok", "surv_score", "cand_logp"):
        assert (a[key] == b[key]).all(), key


@pytest.mark.parametrize("beam,cp,info,att", [(1, 0.0, 0, "local_p_general"), (4, 0.2, 1, "local_p_general"),
                                               (3, 0.2, 0, "global_general"), (2, 0.0, 0, "global_dot")])
def test_against_float64_restatement(oracle, c1, beam, cp, info, att):
    """Step by step against the numpy restatement.  The float64 side follows the checker's
    survivors (after verifying each is a valid choice within tolerance), so every step is
    compared even where fp32 score ties would split the two searches."""
    from oracle import ref_numpy
    c, blob, sents = c1
    o = oracle.decode(c.desc, [blob], sents, beam=beam, nbest=1, cp_beta=cp, print_info=info, attention=att,
                      full_logp=True, trace=True)
    for i in range(sents.n):
        ids = sents.ids[sents.off[i]:sents.off[i + 1]]
        T = int(sents.steps[i])
        follow = {"surv_tok": o["surv_tok"][i], "surv_parent": o["surv_parent"][i], "surv_score": o["surv_score"][i]}
        res, logps = ref_numpy.decode_sentence(c.desc, blob, ids, T, beam=beam, cp_beta=cp, nbest=1,
                                               attention=att, track_align=bool(info), follow=follow)
        for t in range(T + 1):
            ref = np.array(logps[t])
            got = o["logp_full"][i, t]
            assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max(), (i, t)
        n = int(o["len"][i, 0])
        # final scores of the best hypothesis agree (the hypothesis itself may differ by a tie)
        assert abs(o["score"][i, 0] - res[0][0]) <= 1e-4 * abs(res[0][0])
        if list(o["tok"][i, 0, :n]) != res[0][1]:
            assert abs(o["score"][i, 0] - res[0][0]) <= 1e-5 * abs(res[0][0])


def test_known_answer_zero_weights(oracle):
    """All-zero weights: every distribution is uniform, so the top-(k+1) of every beam is the
    ids 0..k (lowest index wins ties), START is skipped, EOS finishes at every step."""
    d = synth.ModelDesc(1, 8, 20, 10, 1)
    blob = np.zeros(synth.blob_floats(d), np.float32)
    sents = synth.Sentences(np.array([3, 4, 5], np.int32), np.array([0, 3], np.int32), np.array([2], np.int32))
    k = 3
    o = oracle.decode(d, [blob], sents, beam=k, nbest=4, trace=True, lp_alpha=0.0, min_ratio=0.0)
    lp = np.float32(np.log(np.float32(1.0) / np.float32(20.0)))
    assert (o["cand_tok"][0, 0, 0] == np.arange(k + 1)).all()
    np.testing.assert_allclose(o["cand_logp"][0, 0, 0], lp, rtol=1e-6)
    # step 0: candidates 0(START, skipped) 1(EOS, finished) 2 3 -> two survivors + one dead slot
    assert o["surv_tok"][0, 0].tolist() == [2, 3, 2]
    assert o["surv_score"][0, 0, 2] == np.float32(-1e30)
    # best hypothesis: "<START> <EOS>" finished at step 0 with score log(1/20)
    assert o["tok"][0, 0, :2].tolist() == [0, 1] and o["len"][0, 0] == 2
    np.testing.assert_allclose(o["score"][0, 0], lp, rtol=1e-6)


def test_softmax_topk_tie_rule(oracle):
    z = np.zeros((2, 50), np.float32)
    z[1, [7, 30, 31]] = 1.0
    idx, lp = oracle.softmax_topk(z, 5)
    assert idx[0].tolist() == [0, 1, 2, 3, 4]
    assert idx[1].tolist() == [7, 30, 31, 0, 1]


def test_bf16_mode_close_to_fp32(oracle, c1):
    c, blob, sents = c1
    a = oracle.decode(c.desc, [blob], sents, beam=2, trace=True)
    b = oracle.decode(c.desc, [blob], sents, beam=2, trace=True, precision="bf16")
    assert np.abs(a["cand_logp"][:, 0] - b["cand_logp"][:, 0]).max() < 2e-2


def test_ensemble_modes(oracle, c1):
    c, blob, sents = c1
    blob2 = synth.make_blob(c.desc, 5)
    one = oracle.decode(c.desc, [blob], sents, beam=2, trace=True)
    same = oracle.decode(c.desc, [blob, blob], sents, beam=2, trace=True)
    np.testing.assert_allclose(one["cand_logp"], same["cand_logp"], rtol=1e-5, atol=1e-6)
    for mode in ("prob_mean", "logprob_mean"):
        two = oracle.decode(c.desc, [blob, blob2], sents, beam=2, trace=True, ensemble=mode)
        assert two["len"][:, 0].min() >= 2


@pytest.mark.parametrize("family,precision,fixture", [("peaked", "fp32", "c2_peaked_fp32.npz"), ("peaked", "bf16", "c2_peaked_bf16.npz"),
                                                       ("flat", "fp32", "c2_batch64.npz")])
def test_large_fixtures_spot_check(oracle, family, precision, fixture):
    """The fixtures of the 4 x 1000, 30k-vocabulary configuration hold what the checker decodes today: two of
    the 64 sentences decoded again (sentences are independent, and grouping rows changes no bit)."""
    c = synth.configs()["C2"]
    blob = c.blobs(family=family)[0]
    pick = [1, 3]                                     # two of the shorter sentences: a few seconds of CPU
    sents = c.sentences().subset(pick)
    g = np.load(os.path.join(GOLD, fixture))
    o = oracle.decode(c.desc, [blob], sents, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta, precision=precision)
    for j, i in enumerate(pick):
        n = int(g["len"][i, 0])
        assert int(o["len"][j, 0]) == n
        assert (o["tok"][j, 0, :n] == g["tok"][i, 0, :n]).all()
        assert o["score"][j, 0] == g["score"][i, 0]


def test_second_cpu_build_agrees_to_rounding(oracle):
    """The Eigen-GEMM build of the checker (another summation order, timing and fixtures only) against the
    canonical build on the small configuration: same math, log-probabilities equal to fp32 rounding.  Skipped
    where that build does not exist (it is made only next to the reference tree)."""
    if oracle.eigen_lib() is None:
        pytest.skip("no Eigen-GEMM build of the checker on this machine")
    c = synth.configs()["C1"]
    blob, sents = c.blobs()[0], c.sentences()
    a = oracle.decode(c.desc, [blob], sents, beam=4, nbest=1, trace=True)
    b = oracle.decode(c.desc, [blob], sents, beam=4, nbest=1, trace=True, gemm="eigen")
    # first step of every sentence: no search decisions yet, the same candidates on both sides
    np.testing.assert_allclose(a["cand_logp"][:, 0, 0], b["cand_logp"][:, 0, 0], rtol=2e-6, atol=2e-6)
    same = sum(1 for i in range(sents.n) if list(a["tok"][i, 0, :a["len"][i, 0]]) == list(b["tok"][i, 0, :b["len"][i, 0]]))
    assert same >= sents.n - 2

"""Generates the golden decode fixtures from the CPU checker (the reference itself cannot be
built or run, and ships neither a model nor expected outputs).  Run from the repository root:

    python tests/golden/make_golden.py

Writes tests/golden/c1_greedy.npz, c1_beam4.npz and tiny_global.npz, and (about a minute of
CPU) c2_batch64.npz, the final hypotheses of the whole 64-sentence reference decode
configuration: inputs are regenerated from seeds by linmt_b200.synth, the files hold the
expected outputs.  With ``--peaked`` it writes instead the final hypotheses of the "peaked" model
family (linmt_b200.synth.PEAKED) in fp32 and in the checker's bf16 mode: c2_peaked_{fp32,bf16}.npz
(the 64 sentences of the reference decode configuration) and c3shape_peaked_{fp32,bf16}.npz (128
sentences of 10 to 80 words, the batch shape of the throughput configuration); about half an hour of
CPU on eight cores.  With ``--eigen`` (only where the Eigen-GEMM build of the checker exists, i.e. next to
the reference tree) it writes what a SECOND CPU build of the same math decodes: the checker with its dense
products handed to the reference's vendored Eigen, which sums in another order --
c2_{peaked,flat}_{fp32,bf16}_eigen.npz, and c2_flat_bf16.npz, the canonical checker's bf16 decode of the
unscaled model.  The tests take from these how often two CPU builds of the reference's math agree with each
other token by token, which is the level the CUDA engine is held to."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from linmt_b200 import synth  # noqa: E402
from oracle import oracle_py  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    "c1_greedy": dict(beam=1, nbest=1, cp_beta=0.0, print_info=0, attention="local_p_general"),
    "c1_beam4": dict(beam=4, nbest=3, cp_beta=0.2, print_info=1, attention="local_p_general"),
    "tiny_global": dict(beam=3, nbest=2, cp_beta=0.0, print_info=0, attention="global_general"),
}


def main():
    c = synth.configs()["C1"]
    blob = c.blobs()[0]
    sents = c.sentences()
    for name, kw in CASES.items():
        o = oracle_py.decode(c.desc, [blob], sents, trace=True, **kw)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), tok=o["tok"], len=o["len"], score=o["score"],
                            vit=o["vit"], surv_tok=o["surv_tok"], surv_parent=o["surv_parent"],
                            surv_score=o["surv_score"], cand_tok=o["cand_tok"], cand_logp=o["cand_logp"],
                            final_logp=o["final_logp"])
        print(name, o["len"][:, 0].tolist())
    c2 = synth.configs()["C2"]
    o = oracle_py.decode(c2.desc, [c2.blobs()[0]], c2.sentences(), beam=c2.beam, nbest=1, lp_alpha=c2.lp_alpha,
                         cp_beta=c2.cp_beta)
    np.savez_compressed(os.path.join(HERE, "c2_batch64.npz"), tok=o["tok"], len=o["len"], score=o["score"])
    print("c2_batch64", o["len"][:, 0].tolist())


def peaked():
    for name, cfg, n in (("c2_peaked", "C2", 64), ("c3shape_peaked", "C3", 128)):
        c = synth.configs()[cfg]
        blob = c.blobs(family="peaked")[0]
        sents = c.sentences(n)
        for prec in ("fp32", "bf16"):
            o = oracle_py.decode(c.desc, [blob], sents, beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta,
                                 precision=prec)
            np.savez_compressed(os.path.join(HERE, f"{name}_{prec}.npz"), tok=o["tok"], len=o["len"], score=o["score"])
            print(name, prec, o["len"][:, 0].tolist())


def eigen():
    c = synth.configs()["C2"]
    sents = c.sentences()
    kw = dict(beam=c.beam, nbest=1, lp_alpha=c.lp_alpha, cp_beta=c.cp_beta)
    for fam in ("peaked", "flat"):
        blob = c.blobs(family=fam)[0]
        for prec in ("fp32", "bf16"):
            o = oracle_py.decode(c.desc, [blob], sents, precision=prec, gemm="eigen", **kw)
            np.savez_compressed(os.path.join(HERE, f"c2_{fam}_{prec}_eigen.npz"), tok=o["tok"], len=o["len"], score=o["score"])
            print("c2", fam, prec, "eigen", o["len"][:, 0].tolist())
    o = oracle_py.decode(c.desc, [c.blobs()[0]], sents, precision="bf16", **kw)
    np.savez_compressed(os.path.join(HERE, "c2_flat_bf16.npz"), tok=o["tok"], len=o["len"], score=o["score"])


if __name__ == "__main__":
    if "--eigen" in sys.argv:
        eigen()
    elif "--peaked" in sys.argv:
        peaked()
    else:
        main()

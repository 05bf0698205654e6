"""ctypes front-end of the CPU checker (test infrastructure).

Only the tests, the smoke check and the benchmark's CPU-baseline legs import this module.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle

ATT = {"local_p_general": 0, "global_general": 1, "global_dot": 2}
ENS = {"prob_mean": 0, "logprob_mean": 1}
PREC = {"fp32": 0, "bf16": 1}


class Opts(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("beam", "nbest", "attention_mode", "attention_d", "print_info",
                                         "precision", "ensemble_mode", "max_len", "max_src", "group",
                                         "threads", "reserved")] + \
               [(n, C.c_float) for n in ("penalty", "diversity", "lp_alpha", "cp_beta", "min_ratio")]


_lib = None


def _has_avx512() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    fl = line.split()
                    return all(x in fl for x in ("avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512cd"))
    except OSError:
        pass
    return False


_eigen_lib = None


def _declare(L):
    L.linmt_oracle_blob_floats.restype = C.c_size_t
    L.linmt_oracle_threads.restype = C.c_int
    L.linmt_oracle_decode.restype = C.c_int
    return L


def lib():
    global _lib
    if _lib is None:
        variant = "v4" if _has_avx512() else "v3"
        path = build_oracle.lib_path(variant)
        if not os.path.exists(path):
            build_oracle.build()
        _lib = _declare(C.CDLL(path))
    return _lib


def eigen_lib():
    """The Eigen-GEMM build (oracle/_ref/, baseline timing only), or None where it was never built."""
    global _eigen_lib
    if _eigen_lib is None:
        path = build_oracle.ref_lib_path("v4" if _has_avx512() else "v3")
        if not os.path.exists(path):
            return None
        _eigen_lib = _declare(C.CDLL(path))
    return _eigen_lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def gemm(X: np.ndarray, W: np.ndarray) -> np.ndarray:
    X = np.ascontiguousarray(X, np.float32)
    W = np.ascontiguousarray(W, np.float32)
    R, K = X.shape
    N = W.shape[1]
    Y = np.empty((R, N), np.float32)
    lib().linmt_oracle_gemm(_p(Y, C.c_float), _p(X, C.c_float), _p(W, C.c_float), R, K, N)
    return Y


def softmax_topk(logits: np.ndarray, kk: int):
    logits = np.ascontiguousarray(logits, np.float32)
    R, V = logits.shape
    idx = np.empty((R, kk), np.int32)
    lp = np.empty((R, kk), np.float32)
    lib().linmt_oracle_softmax_topk(_p(logits, C.c_float), R, V, kk, _p(idx, C.c_int32), _p(lp, C.c_float))
    return idx, lp


def decode(desc, blobs, sents, *, beam, nbest=1, attention="local_p_general", attention_d=10, print_info=0,
           precision="fp32", ensemble="prob_mean", penalty=0.0, diversity=0.0, lp_alpha=0.65, cp_beta=0.0,
           min_ratio=0.5, group=0, threads=0, trace=False, full_logp=False, gemm="canonical"):
    """Decode ``sents`` (a ``Sentences``) and return a dict of numpy arrays.  ``group`` = sentences
    that advance together (0: all; 1: one sentence at a time, rows = beam, the way the reference's own
    loop runs, src/decoder.h:1780-1840).  ``gemm="eigen"`` uses the Eigen-GEMM build (timing only)."""
    L = lib() if gemm == "canonical" else eigen_lib()
    if L is None:
        raise RuntimeError("the Eigen-GEMM build of the checker is not there (oracle/_ref/)")
    d = desc.as_array()
    V = int(d[2])
    k = min(beam, int(np.floor(np.sqrt(V))))
    n = sents.n
    Tm = int(sents.steps.max()) if n else 0
    max_len = Tm + 2
    max_src = int(sents.lengths().max()) if n else 1
    o = Opts(beam=beam, nbest=nbest, attention_mode=ATT[attention], attention_d=attention_d, print_info=print_info,
             precision=PREC[precision], ensemble_mode=ENS[ensemble], max_len=max_len, max_src=max_src, group=group,
             threads=threads, reserved=0, penalty=penalty, diversity=diversity, lp_alpha=lp_alpha, cp_beta=cp_beta,
             min_ratio=min_ratio)
    blobs = [np.ascontiguousarray(b, np.float32) for b in blobs]
    arr = (C.POINTER(C.c_float) * len(blobs))(*[_p(b, C.c_float) for b in blobs])
    out = {
        "tok": np.zeros((n, nbest, max_len), np.int32), "len": np.zeros((n, nbest), np.int32),
        "score": np.zeros((n, nbest), np.float32), "vit": np.full((n, nbest, max_len), -20, np.int32),
        "align": np.zeros((n, nbest, max_len, max_src), np.float32) if print_info else None,
        "k": k, "Tm": Tm, "max_len": max_len, "max_src": max_src,
    }
    tr = {}
    if trace:
        tr = {"cand_tok": np.full((n, Tm, k, k + 1), -1, np.int32), "cand_logp": np.zeros((n, Tm, k, k + 1), np.float32),
              "surv_tok": np.full((n, Tm, k), -1, np.int32), "surv_parent": np.full((n, Tm, k), -1, np.int32),
              "surv_score": np.zeros((n, Tm, k), np.float32), "final_logp": np.zeros((n, k), np.float32),
              "pt": np.zeros((len(blobs), n, Tm + 1, k), np.float32)}
    if full_logp:
        tr["logp_full"] = np.zeros((n, Tm + 1, k, V), np.float32)
    rc = L.linmt_oracle_decode(
        len(blobs), _p(d, C.c_int32), arr, C.c_size_t(blobs[0].size), C.byref(o), n,
        _p(np.ascontiguousarray(sents.ids, np.int32), C.c_int32), _p(np.ascontiguousarray(sents.off, np.int32), C.c_int32),
        _p(np.ascontiguousarray(sents.steps, np.int32), C.c_int32),
        _p(out["tok"], C.c_int32), _p(out["len"], C.c_int32), _p(out["score"], C.c_float), _p(out["vit"], C.c_int32),
        _p(out["align"], C.c_float),
        _p(tr.get("cand_tok"), C.c_int32), _p(tr.get("cand_logp"), C.c_float), _p(tr.get("surv_tok"), C.c_int32),
        _p(tr.get("surv_parent"), C.c_int32), _p(tr.get("surv_score"), C.c_float), _p(tr.get("final_logp"), C.c_float),
        _p(tr.get("logp_full"), C.c_float), _p(tr.get("pt"), C.c_float))
    if rc != 0:
        raise RuntimeError(f"linmt_oracle_decode failed with status {rc}")
    if "pt" in tr and len(blobs) == 1:
        tr["pt"] = tr["pt"][0]     # one model: [n][Tm+1][k]; ensembles keep the member axis in front
    out.update(tr)
    return out

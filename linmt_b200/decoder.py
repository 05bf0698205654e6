"""Python host side over the C ABI, mirroring the reference's decoder interface.

``DecoderSentence`` has the reference class's two methods (src/decoder_sentence.h:40-41:
``Init(config)``, ``Process(sentence) -> str``); ``Decoder`` is the batch form of
``EnsembleFactory::DecodeSentence`` (src/decoder.h:1780-1840): integer sentences in,
hypotheses out.  All arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

ATT = {"local_p_general": 0, "global_general": 1, "global_dot": 2}
ENS = {"prob_mean": 0, "logprob_mean": 1}
PREC = {"fp32": 0, "bf16": 1}
GEMM = {"auto": 0, "simt": 1, "tensor": 2, "tensor2": 3, "tensor3": 4, "tensor_v16": 5, "tensor_v16x": 6}


class LinmtError(RuntimeError):
    pass


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Decoder:
    """Batch decoder over in-memory weights (one blob per ensemble member)."""

    def __init__(self, desc, blobs, *, beam=12, nbest=1, attention="local_p_general", attention_d=10, print_info=0,
                 precision="fp32", ensemble="prob_mean", gemm_path="auto", max_batch=64, max_src_len=100,
                 max_steps=200, device=0, devices=None, penalty=0.0, diversity=0.0, lp_alpha=0.65, cp_beta=0.2,
                 min_ratio=0.5):
        """``devices``: a list of GPU ordinals that each hold a replica and share the sentences of a
        ``decode`` call (one host thread per GPU inside the library); default: the single ``device``."""
        lib = _lib.load()
        self._lib = lib
        o = _lib.OptionsC()
        lib.linmt_default_options(C.byref(o))
        o.beam, o.nbest, o.attention_mode, o.attention_d = beam, nbest, ATT[attention], attention_d
        o.print_info, o.precision, o.ensemble_mode, o.gemm_path = print_info, PREC[precision], ENS[ensemble], GEMM[gemm_path]
        o.max_batch, o.max_src_len, o.max_steps, o.device = max_batch, max_src_len, max_steps, device
        o.penalty, o.diversity, o.lp_alpha, o.cp_beta, o.min_ratio = penalty, diversity, lp_alpha, cp_beta, min_ratio
        self.opt = o
        d = _lib.ModelDescC(desc.L, desc.H, desc.V, desc.Vs, desc.feed_input)
        blobs = [np.ascontiguousarray(b, np.float32) for b in blobs]
        arr = (C.c_void_p * len(blobs))(*[b.ctypes.data for b in blobs])
        h = C.c_void_p()
        devs = np.ascontiguousarray(devices if devices is not None else [], np.int32)
        rc = lib.linmt_create_from_weights_on(C.byref(d), arr, len(blobs), blobs[0].size, C.byref(o),
                                              _ptr(devs) if len(devs) else None, len(devs), C.byref(h))
        if rc != 0:
            raise LinmtError(f"linmt_create_from_weights failed ({rc}): {lib.linmt_last_error(None).decode()}")
        self._h = h
        self.n_models = len(blobs)
        self.k = lib.linmt_beam(h)
        self.nbest = nbest
        self.max_src_len = max_src_len
        self.print_info = print_info

    def close(self):
        if getattr(self, "_h", None):
            self._lib.linmt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != 0:
            raise LinmtError(f"{what} failed ({rc}): {self._lib.linmt_last_error(self._h).decode()}")

    def decode(self, sents, *, trace=False, force=None, want_align=False):
        """``sents``: a ``synth.Sentences``.  Returns a dict of numpy arrays shaped like the
        CPU checker's output."""
        n = sents.n
        ids = np.ascontiguousarray(sents.ids, np.int32)
        off = np.ascontiguousarray(sents.off, np.int32)
        steps = np.ascontiguousarray(sents.steps, np.int32)
        Tm = int(steps.max()) if n else 0
        max_len = Tm + 2
        k, nb = self.k, self.nbest
        out = {"tok": np.zeros((n, nb, max_len), np.int32), "len": np.zeros((n, nb), np.int32),
               "score": np.zeros((n, nb), np.float32), "vit": np.full((n, nb, max_len), -20, np.int32),
               "align": np.zeros((n, nb, max_len, self.max_src_len), np.float32) if (want_align and self.print_info) else None,
               "k": k, "Tm": Tm, "max_len": max_len}
        tr = None
        if trace or force is not None:
            tr = _lib.TraceC()
            if trace:
                out.update({"cand_tok": np.full((n, Tm, k, k + 1), -1, np.int32),
                            "cand_logp": np.zeros((n, Tm, k, k + 1), np.float32),
                            "surv_tok": np.full((n, Tm, k), -1, np.int32), "surv_parent": np.full((n, Tm, k), -1, np.int32),
                            "surv_score": np.zeros((n, Tm, k), np.float32), "final_logp": np.zeros((n, k), np.float32),
                            "pt": np.zeros((self.n_models, n, Tm + 1, k), np.float32)})
                for f in ("cand_tok", "cand_logp", "surv_tok", "surv_parent", "surv_score", "final_logp", "pt"):
                    setattr(tr, f, out[f].ctypes.data)
            if force is not None:
                self._force = [np.ascontiguousarray(force["surv_tok"], np.int32),
                               np.ascontiguousarray(force["surv_parent"], np.int32),
                               np.ascontiguousarray(force["surv_score"], np.float32)]
                tr.force_tok, tr.force_parent, tr.force_score = [a.ctypes.data for a in self._force]
        rc = self._lib.linmt_decode_batch(self._h, _ptr(ids), _ptr(off), n, _ptr(steps), max_len, _ptr(out["tok"]),
                                          _ptr(out["len"]), _ptr(out["score"]), _ptr(out["vit"]), _ptr(out["align"]),
                                          C.byref(tr) if tr is not None else None)
        self._check(rc, "linmt_decode_batch")
        if trace and self.n_models == 1:
            out["pt"] = out["pt"][0]   # one model: [n][Tm+1][k]; ensembles keep the member axis in front
        return out

    def decode_device(self, d_ids_ptr, off, steps, max_len, d_tok_ptr, d_len_ptr, d_score_ptr):
        """Device-resident decode of one batch: ids and outputs are raw device pointers."""
        off = np.ascontiguousarray(off, np.int32)
        steps = np.ascontiguousarray(steps, np.int32)
        rc = self._lib.linmt_decode_batch_device(self._h, C.c_void_p(d_ids_ptr), _ptr(off), len(steps), _ptr(steps),
                                                 max_len, C.c_void_p(d_tok_ptr), C.c_void_p(d_len_ptr),
                                                 C.c_void_p(d_score_ptr))
        self._check(rc, "linmt_decode_batch_device")

    def score(self, sents, targets):
        """Force-decoding: log p(target | source) per sentence and per token (EOS last).
        ``targets`` = list of id sequences without START / EOS."""
        n = sents.n
        ids = np.ascontiguousarray(sents.ids, np.int32)
        off = np.ascontiguousarray(sents.off, np.int32)
        tl = [len(t) for t in targets]
        toff = np.zeros(n + 1, np.int32)
        toff[1:] = np.cumsum(tl)
        tids = np.ascontiguousarray(np.concatenate([np.asarray(t, np.int32) for t in targets]), np.int32)
        mt = max(tl)
        total = np.zeros(n, np.float32)
        per_tok = np.zeros((n, mt + 1), np.float32)
        rc = self._lib.linmt_score_batch(self._h, _ptr(ids), _ptr(off), _ptr(tids), _ptr(toff), n, _ptr(total), _ptr(per_tok), mt)
        self._check(rc, "linmt_score_batch")
        return total, per_tok

    def stats(self):
        s = _lib.StatsC()
        self._lib.linmt_get_stats(self._h, C.byref(s))
        return {f: getattr(s, f) for f, _ in s._fields_}

    def set_kernel_timing(self, on: bool):
        self._lib.linmt_set_kernel_timing(self._h, int(on))

    KERNEL_CLASSES = ("gather", "lstm_gemm", "attn_proj_gemm", "attention", "attn_out_gemm", "vocab_gemm",
                      "ensemble_combine", "softmax_topk", "beam_select")

    def kernel_times(self):
        """{class: (ms, launches)} of the last decode with kernel timing on."""
        ms = np.zeros(9, np.float32)
        n = np.zeros(9, np.int32)
        self._lib.linmt_kernel_times(self._h, _ptr(ms), _ptr(n), 9)
        return {c: (float(ms[i]), int(n[i])) for i, c in enumerate(self.KERNEL_CLASSES)}


class DecoderSentence:
    """Mirror of the reference's ``DecoderSentence`` (src/decoder_sentence.h:28-60)."""

    def __init__(self):
        self._lib = _lib.load()
        self._h = None

    def Init(self, config: str) -> bool:
        h = C.c_void_p()
        rc = self._lib.linmt_create(config.encode(), C.byref(h))
        if rc != 0:
            raise LinmtError(f"Init failed ({rc}): {self._lib.linmt_front_error().decode()}")
        self._h = h
        return True

    def Process(self, input_sentence: str) -> str:
        if self._h is None:
            raise LinmtError("Init was not called")
        return self._lib.linmt_translate(self._h, input_sentence.encode()).decode()

    def DecodeFile(self, in_path: str, out_path: str) -> None:
        """File-mode decoding (src/decoder.h:1702-1776): one sentence per line in, n-best per sentence out."""
        if self._h is None:
            raise LinmtError("Init was not called")
        rc = self._lib.linmt_decode_file(self._h, in_path.encode(), out_path.encode())
        if rc != 0:
            raise LinmtError(f"linmt_decode_file failed ({rc}): {self._lib.linmt_last_error(self._h).decode()}")

    def close(self):
        if self._h:
            self._lib.linmt_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def k_gemm(X, W, gemm_path="simt", precision="fp32", device=0):
    X = np.ascontiguousarray(X, np.float32)
    W = np.ascontiguousarray(W, np.float32)
    R, K = X.shape
    N = W.shape[1]
    Y = np.empty((R, N), np.float32)
    rc = _lib.load().linmt_k_gemm(_ptr(X), _ptr(W), _ptr(Y), R, K, N, GEMM[gemm_path], PREC[precision], device)
    if rc != 0:
        raise LinmtError(f"linmt_k_gemm failed ({rc})")
    return Y


def k_softmax_topk(logits, kk, device=0):
    logits = np.ascontiguousarray(logits, np.float32)
    R, V = logits.shape
    idx = np.empty((R, kk), np.int32)
    lp = np.empty((R, kk), np.float32)
    eos = np.empty((R,), np.float32)
    rc = _lib.load().linmt_k_softmax_topk(_ptr(logits), R, V, kk, _ptr(idx), _ptr(lp), _ptr(eos), device)
    if rc != 0:
        raise LinmtError(f"linmt_k_softmax_topk failed ({rc})")
    return idx, lp, eos

"""ctypes binding of ``liblinmt_decoder.so`` (the CUDA library).  There is no CPU fallback:
if the library is missing this module raises, it never substitutes another implementation."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblinmt_decoder.so")


class ModelDescC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "vocab_tgt", "vocab_src", "feed_input")]


class OptionsC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("beam", "nbest", "attention_mode", "attention_d", "print_info", "precision",
                                         "ensemble_mode", "gemm_path", "max_batch", "max_src_len", "max_steps",
                                         "device")] + \
               [(n, C.c_float) for n in ("penalty", "diversity", "lp_alpha", "cp_beta", "min_ratio", "max_ratio")]


class TraceC(C.Structure):
    _fields_ = [("cand_tok", C.c_void_p), ("cand_logp", C.c_void_p), ("surv_tok", C.c_void_p),
                ("surv_parent", C.c_void_p), ("surv_score", C.c_void_p), ("final_logp", C.c_void_p),
                ("force_tok", C.c_void_p), ("force_parent", C.c_void_p), ("force_score", C.c_void_p),
                ("gold_logp", C.c_void_p), ("pt", C.c_void_p)]


class StatsC(C.Structure):
    _fields_ = [("kernel_launches", C.c_int64), ("decoder_row_steps", C.c_int64), ("sentence_steps", C.c_int64),
                ("last_decode_ms", C.c_float), ("last_gemm_ms", C.c_float), ("last_gemm_launches", C.c_int32),
                ("last_rec_gemm_launches", C.c_int32), ("last_rec_gemm_ms", C.c_float), ("last_host_issue_ms", C.c_float),
                ("last_rec_gemm_flops", C.c_double), ("pair_launches", C.c_int64)]


EXPORTS = ["python_decoder_init", "python_decoder_do_job", "linmt_default_options", "linmt_blob_floats",
           "linmt_create_from_weights", "linmt_create_from_weights_on", "linmt_device_count", "linmt_front_error", "linmt_create", "linmt_destroy", "linmt_last_error", "linmt_beam",
           "linmt_decode_batch", "linmt_decode_batch_device", "linmt_get_stats", "linmt_set_kernel_timing", "linmt_kernel_times",
           "linmt_translate", "linmt_k_gemm", "linmt_k_softmax_topk", "linmt_gemm_f32_noalloc", "linmt_decode_file", "linmt_score_batch",
           "linmt_read_model_file", "python_unk_init", "python_unk_do_job", "linmt_unk_create", "linmt_unk_process", "linmt_unk_destroy"]

_lib = None


def load():
    """Loads the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m linmt_b200.build` "
                           "(there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.python_decoder_init.argtypes = [C.c_char_p]
    lib.python_decoder_init.restype = None
    lib.python_decoder_do_job.argtypes = [C.c_char_p]
    lib.python_decoder_do_job.restype = C.c_char_p
    lib.linmt_default_options.argtypes = [C.POINTER(OptionsC)]
    lib.linmt_default_options.restype = None
    lib.linmt_blob_floats.argtypes = [C.POINTER(ModelDescC)]
    lib.linmt_blob_floats.restype = C.c_size_t
    lib.linmt_create_from_weights.argtypes = [C.POINTER(ModelDescC), C.POINTER(C.c_void_p), C.c_int32, C.c_size_t,
                                              C.POINTER(OptionsC), C.POINTER(C.c_void_p)]
    lib.linmt_create_from_weights_on.argtypes = [C.POINTER(ModelDescC), C.POINTER(C.c_void_p), C.c_int32, C.c_size_t,
                                                 C.POINTER(OptionsC), C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)]
    lib.linmt_device_count.argtypes = [C.c_void_p]
    lib.linmt_create.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.linmt_destroy.argtypes = [C.c_void_p]
    lib.linmt_destroy.restype = None
    lib.linmt_last_error.argtypes = [C.c_void_p]
    lib.linmt_last_error.restype = C.c_char_p
    lib.linmt_front_error.restype = C.c_char_p
    lib.linmt_beam.argtypes = [C.c_void_p]
    lib.linmt_decode_batch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(TraceC)]
    lib.linmt_decode_batch_device.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
    lib.linmt_get_stats.argtypes = [C.c_void_p, C.POINTER(StatsC)]
    lib.linmt_set_kernel_timing.argtypes = [C.c_void_p, C.c_int32]
    lib.linmt_kernel_times.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]
    lib.linmt_translate.argtypes = [C.c_void_p, C.c_char_p]
    lib.linmt_translate.restype = C.c_char_p
    lib.linmt_k_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                 C.c_int32, C.c_int32]
    lib.linmt_k_softmax_topk.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int32]
    lib.linmt_gemm_f32_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    lib.linmt_decode_file.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
    lib.linmt_read_model_file.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int32]
    lib.python_unk_do_job.restype = C.c_char_p
    lib.python_unk_do_job.argtypes = [C.c_char_p, C.c_char_p]
    lib.python_unk_init.argtypes = [C.c_char_p]
    lib.linmt_unk_create.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.linmt_unk_process.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_int32]
    lib.linmt_unk_destroy.argtypes = [C.c_void_p]
    lib.linmt_score_batch.argtypes = [C.c_void_p] * 5 + [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32]
    _lib = lib
    return lib

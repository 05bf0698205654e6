"""Writer of the reference's model-file format (header + vocabularies + matrices).

Format: src/utility_cc.cc:76-101 (header of nine integers), src/input_file_preprocess.cc:519-575
(vocabulary sections between ``====`` lines), src/deep_rnn_kernel.h:1563-1578 (each matrix as
``rows`` lines of ``cols`` values and a blank line).  ``binary=True`` writes the same file with a
raw float32 body after a ``BINARY <count>`` line, a faster form the library also reads.
"""
from __future__ import annotations

import numpy as np

from .synth import ModelDesc, blob_layout

SEP = "=" * 42


def default_vocab(n: int, side: str):
    if side == "src":
        return ["<UNK>"] + [f"s{i}" for i in range(1, n)]
    return ["<START>", "<EOF>", "<UNK>"] + [f"t{i}" for i in range(3, n)]


def write_model(path: str, desc: ModelDesc, blob: np.ndarray, src_words=None, tgt_words=None, binary=False):
    src_words = src_words or default_vocab(desc.Vs, "src")
    tgt_words = tgt_words or default_vocab(desc.V, "tgt")
    with open(path, "wb") as f:
        f.write(f"{desc.L} {desc.H} {desc.V} {desc.Vs} 1 {desc.feed_input} 0 0 0\n".encode())
        f.write((SEP + "\n").encode())
        for i, w in enumerate(src_words):
            f.write(f"{i} {w}\n".encode())
        f.write((SEP + "\n").encode())
        for i, w in enumerate(tgt_words):
            f.write(f"{i} {w}\n".encode())
        f.write((SEP + "\n").encode())
        if binary:
            f.write(f"BINARY {blob.size}\n".encode())
            f.write(np.ascontiguousarray(blob, "<f4").tobytes())
            return
        off = 0
        for _, r, c in blob_layout(desc):
            m = blob[off:off + r * c].reshape(c, r).T  # logical [row, col]
            off += r * c
            for i in range(r):
                f.write((" ".join(repr(float(np.float32(v))) if False else f"{v:.9g}" for v in m[i]) + "\n").encode())
            f.write(b"\n")


def write_config(path: str, model_paths, **kv):
    """Writes a decoding-sentence config file (src/decoder_sentence.cu:267-318)."""
    with open(path, "w") as f:
        f.write("# decoding with nmt model\n")
        f.write(f'param="--nmt-model"   value="{" ".join(model_paths)}"\n')
        for k, v in kv.items():
            f.write(f'param="--{k.replace("_", "-")}"   value="{v}"\n')


def read_model(path: str, use_cache: bool = True):
    """Model file (the reference's text format, or its binary-body variant) -> (ModelDesc, blob),
    through the library's own reader (linmt_read_model_file; no GPU involved)."""
    import ctypes as C
    from . import _lib
    lib = _lib.load()
    d = _lib.ModelDescC()
    rc = lib.linmt_read_model_file(path.encode(), C.byref(d), None, 0, 0)
    if rc != 0:
        raise RuntimeError(f"linmt_read_model_file failed ({rc})")
    desc = ModelDesc(L=d.layers, H=d.hidden, V=d.vocab_tgt, Vs=d.vocab_src, feed_input=d.feed_input)
    n = int(lib.linmt_blob_floats(C.byref(d)))
    blob = np.empty(n, np.float32)
    rc = lib.linmt_read_model_file(path.encode(), C.byref(d), blob.ctypes.data_as(C.c_void_p), n, 1 if use_cache else 0)
    if rc != 0:
        raise RuntimeError(f"linmt_read_model_file failed ({rc})")
    return desc, blob

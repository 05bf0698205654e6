"""Seeded synthetic models and source sentences for the decoding configurations.

The reference project ships no trained model, so every measurement and parity case runs on
random-initialised weights of the named architecture and on random sentences with the named
length and token-frequency distributions.  One weight blob is read by both the CUDA engine
and the CPU checker, so the generator's own RNG is free (numpy ``default_rng``).

Blob layout = the reference's device memory after ``LoadWeights`` (src/deep_rnn.h:1878-1969):
matrices in file order, each ``rows x cols`` column-major (src/utility_cu.h:37), i.e. a
weight ``out x in`` is stored ``[in][out]``, an embedding ``H x V`` as ``[V][H]`` and the
output matrix ``V x H`` as ``[H][V]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

START, EOS, UNK = 0, 1, 2  # target-side ids, src/input_file_preprocess.cc:549-567


@dataclass
class ModelDesc:
    L: int
    H: int
    V: int
    Vs: int
    feed_input: int = 1

    def as_array(self) -> np.ndarray:
        return np.array([self.L, self.H, self.V, self.Vs, self.feed_input], dtype=np.int32)


def blob_layout(d: ModelDesc):
    """List of (name, rows, cols) in LoadWeights order
    (src/layer_input_to_hidden.h:1378-1423, src/layer_hidden_to_hidden.h:953-979,
    src/layer_attention.h:1246-1260, src/layer_loss.h:1191-1196)."""
    H = d.H
    out = []

    def lstm(prefix, first, vocab, feed):
        for g in ("i", "f", "c", "o"):
            out.append((f"{prefix}.W_h{g}", H, H))
            out.append((f"{prefix}.b_{g}", H, 1))
        if first:
            out.append((f"{prefix}.W_emb", H, vocab))
        for g in ("i", "f", "o", "c"):
            out.append((f"{prefix}.M_{g}", H, H))
        if feed:
            for g in ("i", "f", "o", "c"):
                out.append((f"{prefix}.Q_{g}", H, H))

    for l in range(d.L):
        lstm(f"src{l}", l == 0, d.Vs, False)
    for l in range(d.L):
        lstm(f"tgt{l}", l == 0, d.V, l == 0 and bool(d.feed_input))
    out += [("att.W_a", H, H), ("att.W_p", H, H), ("att.v_p", H, 1), ("att.b_out", H, 1),
            ("att.W_c1", H, H), ("att.W_c2", H, H)]
    out += [("sm.D", d.V, H), ("sm.b_d", d.V, 1)]
    return out


def blob_floats(d: ModelDesc) -> int:
    return sum(r * c for _, r, c in blob_layout(d))


# Scale factors of the "peaked" model family: the same uniform draws as the named configurations, with
# the embeddings, the recurrent matrices and the output matrix rescaled so that the model behaves like a
# trained one in the two respects that decide whether two implementations can be compared token by token:
#   * the output distribution is peaked (with every weight in [-0.08, 0.08] all 30,000 log-probabilities lie
#     within ~0.5 of each other, so candidates tie to rounding noise at every step);
#   * the recurrence is contractive (at hidden size 1000 the unscaled recurrent matrices have spectral radius
#     ~1.5: rounding noise doubles about every ten decoder steps).
PEAKED = {"emb": 5.0, "recurrent": 0.5, "output": 30.0}


def make_blob(d: ModelDesc, seed: int, lo: float = -0.08, hi: float = 0.08, family: str = "flat") -> np.ndarray:
    """Weights uniform[lo, hi]; biases 0 except the forget-gate bias = 1.  ``family="peaked"``
    rescales three groups of matrices of the same draws (see ``PEAKED``)."""
    rng = np.random.default_rng(seed)
    n = blob_floats(d)
    blob = rng.random(n, dtype=np.float32)
    blob *= np.float32(hi - lo)
    blob += np.float32(lo)
    if family not in ("flat", "peaked"):
        raise ValueError(f"unknown model family {family!r}")
    off = 0
    for name, r, c in blob_layout(d):
        leaf = name.split(".")[1]
        if leaf.startswith("b_"):
            blob[off:off + r * c] = 1.0 if leaf == "b_f" else 0.0
        elif family == "peaked":
            if leaf == "W_emb":
                blob[off:off + r * c] *= np.float32(PEAKED["emb"])
            elif leaf.startswith("W_h"):
                blob[off:off + r * c] *= np.float32(PEAKED["recurrent"])
            elif name == "sm.D":
                blob[off:off + r * c] *= np.float32(PEAKED["output"])
        off += r * c
    return blob


def blob_views(d: ModelDesc, blob: np.ndarray) -> dict:
    """name -> 2-D array indexed [row, col] of the logical matrix (a view, column-major)."""
    views, off = {}, 0
    for name, r, c in blob_layout(d):
        views[name] = blob[off:off + r * c].reshape(c, r).T
        off += r * c
    return views


def zipf_ids(rng, n: int, lo_id: int, hi_id: int, s: float) -> np.ndarray:
    """n ids in [lo_id, hi_id) with P(rank r) ~ r^-s, rank 1 = lo_id."""
    ranks = np.arange(1, hi_id - lo_id + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    u = rng.random(n)
    return (np.searchsorted(cdf, u, side="left") + lo_id).astype(np.int32)


@dataclass
class Sentences:
    ids: np.ndarray      # concatenated natural-order source ids, int32
    off: np.ndarray      # [n+1] int32
    steps: np.ndarray    # [n] int32, beam expansions T_i per sentence

    @property
    def n(self) -> int:
        return len(self.steps)

    def lengths(self) -> np.ndarray:
        return np.diff(self.off)

    def subset(self, idx) -> "Sentences":
        idx = list(idx)
        lens = self.lengths()[idx]
        off = np.zeros(len(idx) + 1, dtype=np.int32)
        off[1:] = np.cumsum(lens)
        ids = np.concatenate([self.ids[self.off[i]:self.off[i + 1]] for i in idx]) if idx else np.zeros(0, np.int32)
        return Sentences(ids.astype(np.int32), off, self.steps[idx].astype(np.int32))


def make_sentences(n: int, len_lo: int, len_hi: int, vocab_src: int, zipf_s: float, seed: int,
                   step_rule) -> Sentences:
    rng = np.random.default_rng(seed + 1000003)
    lens = rng.integers(len_lo, len_hi + 1, size=n).astype(np.int32)
    off = np.zeros(n + 1, dtype=np.int32)
    off[1:] = np.cumsum(lens)
    ids = zipf_ids(rng, int(off[-1]), 1, vocab_src, zipf_s)   # 0 = <UNK> on the source side
    steps = np.array([step_rule(int(s)) for s in lens], dtype=np.int32)
    return Sentences(ids, off, steps)


@dataclass
class Config:
    name: str
    desc: ModelDesc
    seeds: list
    beam: int
    n_sent: int
    len_lo: int
    len_hi: int
    zipf_s: float
    step_rule: object
    precision: str = "fp32"
    attention: str = "local_p_general"
    lp_alpha: float = 0.65
    cp_beta: float = 0.0
    batch: int = 64
    extra: dict = field(default_factory=dict)

    def sentences(self, n=None) -> Sentences:
        return make_sentences(n or self.n_sent, self.len_lo, self.len_hi, self.desc.Vs, self.zipf_s,
                              self.seeds[0], self.step_rule)

    def blobs(self, family: str = "flat"):
        return [make_blob(self.desc, s, family=family) for s in self.seeds]


def configs() -> dict:
    """The five named decoding configurations (C1..C5)."""
    big = ModelDesc(4, 1000, 30000, 30000, 1)
    return {
        "C1": Config("C1", ModelDesc(2, 128, 1000, 1000, 1), [0], 1, 8, 5, 20, 1.1, lambda s: 2 * s, batch=8),
        "C2": Config("C2", big, [1], 12, 64, 10, 50, 1.1, lambda s: int(1.5 * s) + 10),
        "C3": Config("C3", big, [1], 12, 4096, 10, 80, 1.1, lambda s: int(1.5 * s) + 10, precision="bf16"),
        "C4": Config("C4", ModelDesc(4, 1024, 80000, 80000, 1), [3], 5, 1024, 20, 100, 1.05,
                     lambda s: int(1.5 * s) + 10, precision="bf16", attention="global_dot"),
        "C5": Config("C5", big, [10, 11, 12, 13], 12, 512, 10, 60, 1.1, lambda s: int(1.5 * s) + 10),
    }

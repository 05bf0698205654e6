"""GPU parity tests of single kernels, called through the C ABI and compared with the CPU
checker on the same seeded inputs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("R,K,N", [(1, 64, 128), (12, 128, 512), (60, 1000, 4000), (768, 2000, 1000), (131, 257, 391)])
def test_gemm_simt_vs_checker(oracle, cuda_lib, R, K, N):
    from linmt_b200 import decoder
    rng = np.random.default_rng(R * 7 + K)
    X = rng.uniform(-1, 1, (R, K)).astype(np.float32)
    W = rng.uniform(-0.08, 0.08, (K, N)).astype(np.float32)
    Y = decoder.k_gemm(X, W, "simt", "fp32")
    ref = oracle.gemm(X, W)
    scale = np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64)
    # fp32 sums in a different order: error bounded by a few ulps of the absolute-value sum
    assert (np.abs(Y - ref) <= 4e-6 * scale + 1e-7).all()


@pytest.mark.parametrize("R,V,kk", [(4, 1000, 2), (24, 30000, 13), (7, 80000, 6), (3, 37, 5)])
def test_softmax_topk_vs_checker(oracle, cuda_lib, R, V, kk):
    from linmt_b200 import decoder
    rng = np.random.default_rng(V + kk)
    z = rng.normal(0, 0.5, (R, V)).astype(np.float32)
    idx, lp, eos = decoder.k_softmax_topk(z, kk)
    ridx, rlp = oracle.softmax_topk(z, kk)
    assert (idx == ridx).all()          # bit-exact indices
    np.testing.assert_allclose(lp, rlp, rtol=1e-5, atol=1e-6)
    z64 = z.astype(np.float64)
    lse = np.log(np.exp(z64 - z64.max(1, keepdims=True)).sum(1)) + z64.max(1)
    np.testing.assert_allclose(eos, z64[:, 1] - lse, rtol=1e-5, atol=1e-6)


def test_softmax_topk_ties_lowest_index(oracle, cuda_lib):
    from linmt_b200 import decoder
    V, kk = 30000, 13
    z = np.zeros((3, V), np.float32)                 # all equal: ids 0..kk-1
    z[1, [29999, 5, 17000, 17001]] = 2.0             # four-way tie on top, then zeros
    z[2] = np.repeat(np.arange(V // 4, dtype=np.float32)[::-1], 4)[:V] * 0.25  # groups of 4 equal values
    idx, lp, _ = decoder.k_softmax_topk(z, kk)
    ridx, _ = oracle.softmax_topk(z, kk)
    assert idx[0].tolist() == list(range(kk))
    assert idx[1].tolist() == [5, 17000, 17001, 29999] + list(range(0, 5)) + list(range(6, 10))
    assert (idx == ridx).all()


@pytest.mark.parametrize("R,K,N", [(12, 128, 512), (72, 1000, 30000), (768, 3000, 4000), (131, 257, 391)])
@pytest.mark.parametrize("path,prec,tol", [("tensor", "fp32", 1e-6), ("tensor3", "fp32", 1e-6), ("tensor2", "fp32", 4e-6), ("tensor", "bf16", 4e-3)])
def test_gemm_tensor_vs_checker(oracle, cuda_lib, R, K, N, path, prec, tol):
    """tcgen05 GEMM on split operands against a float64 product: the fp16 pair (default) and three
    bf16 planes give the error of an fp32 FMA loop, two bf16 planes ~2^-17 per product, one plane is
    plain bf16."""
    from linmt_b200 import decoder
    rng = np.random.default_rng(R + K + N)
    X = rng.uniform(-1, 1, (R, K)).astype(np.float32)
    W = rng.uniform(-0.08, 0.08, (K, N)).astype(np.float32)
    Y = decoder.k_gemm(X, W, path, prec)
    ref = X.astype(np.float64) @ W.astype(np.float64)
    scale = np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64)
    assert (np.abs(Y - ref) <= tol * scale + 1e-7).all(), float((np.abs(Y - ref) / scale).max())


def test_gemm_on_cta_pairs_vs_float64_and_one_tile(cuda_lib):
    """The decoder's gate product at full width (768 x 2048 times 2048 x 4096) picks 176-wide tiles, which as one
    tile per CTA leave room for two stages only: the library then runs CTA pairs (tcgen05 cta_group::2, each CTA
    loading half of the weight tile).  Against a float64 product the error is that of an fp32 FMA loop, and the
    bits are those of the one-tile kernel (LINMT_TC_PAIR=0): the same products accumulate in the same order."""
    import os
    from linmt_b200 import decoder
    rng = np.random.default_rng(11)
    R, K, N = 768, 2048, 4096
    X = rng.uniform(-1, 1, (R, K)).astype(np.float32)
    W = rng.uniform(-0.08, 0.08, (K, N)).astype(np.float32)
    Y = decoder.k_gemm(X, W, "tensor", "fp32")
    ref = X.astype(np.float64) @ W.astype(np.float64)
    scale = np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64)
    assert (np.abs(Y - ref) <= 1e-6 * scale + 1e-7).all(), float((np.abs(Y - ref) / scale).max())
    old = os.environ.get("LINMT_TC_PAIR")
    os.environ["LINMT_TC_PAIR"] = "0"
    try:
        Y1 = decoder.k_gemm(X, W, "tensor", "fp32")
    finally:
        if old is None:
            os.environ.pop("LINMT_TC_PAIR", None)
        else:
            os.environ["LINMT_TC_PAIR"] = old
    assert np.array_equal(Y, Y1)
    # a last row tile that is partly empty (700 = 5 x 128 + 60 rows)
    Y5 = decoder.k_gemm(X[:700], W, "tensor", "fp32")
    assert (np.abs(Y5 - ref[:700]) <= 1e-6 * scale[:700] + 1e-7).all()

"""GPU test of the entry point that allocates nothing (collected last on purpose).

``linmt_gemm_f32_noalloc`` serves hosts that cannot call cudaMalloc while running (their own
pool owns the GPU, or an allocation would stall a shared device): its working memory is a fixed
array inside the library.  The test calls it through the C ABI on device buffers made by the
test itself and checks the result against the ordinary entry point (``linmt_k_gemm``, which
allocates its own buffers), twice in a row with different shapes so that contents left in the
shared array by the first call cannot leak into the second."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(lib, X, Wt):
    import torch
    R, K = X.shape
    N = Wt.shape[0]
    dx = torch.from_numpy(X).cuda()
    dw = torch.from_numpy(Wt).cuda()
    dy = torch.full((R, N), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = lib.linmt_gemm_f32_noalloc(C.c_void_p(dx.data_ptr()), C.c_void_p(dw.data_ptr()), C.c_void_p(dy.data_ptr()),
                                    R, K, N, 0)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return dy.cpu().numpy()


def test_no_alloc_gemm_matches_allocating_entry_point(cuda_lib):
    from linmt_b200 import decoder
    rng = np.random.default_rng(11)
    for R, K, N in ((200, 1024, 1008), (37, 96, 48)):
        X = rng.uniform(-1, 1, (R, K)).astype(np.float32)
        Wt = rng.uniform(-0.08, 0.08, (N, K)).astype(np.float32)
        got = _run(cuda_lib, X, Wt)
        # the ordinary entry point on the same operand format (three bf16 planes)
        ref = decoder.k_gemm(X, np.ascontiguousarray(Wt.T), "tensor3", "fp32")
        scale = np.abs(X).astype(np.float64) @ np.abs(Wt.T).astype(np.float64)
        # the tolerance of the tensor-GEMM parity test
        assert (np.abs(got - ref) <= 1e-6 * scale + 1e-7).all()
        exact = X.astype(np.float64) @ Wt.T.astype(np.float64)
        assert (np.abs(got - exact) <= 1e-6 * scale + 1e-7).all()


def test_no_alloc_gemm_rejects_sizes_beyond_its_working_memory(cuda_lib):
    import torch
    d = torch.zeros(16, device="cuda")
    p = C.c_void_p(d.data_ptr())
    assert cuda_lib.linmt_gemm_f32_noalloc(p, p, p, 257, 64, 64, 0) == 5    # LINMT_ELIMIT
    assert cuda_lib.linmt_gemm_f32_noalloc(p, p, p, 8, 2048, 64, 0) == 5
    assert cuda_lib.linmt_gemm_f32_noalloc(p, p, p, 8, 64, 1040, 0) == 5
    assert cuda_lib.linmt_gemm_f32_noalloc(p, p, p, 8, 40, 64, 0) == 1      # K not a multiple of 32

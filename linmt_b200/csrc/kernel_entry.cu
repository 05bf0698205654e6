// kernel_entry.cu -- single-kernel entry points of the C ABI (host pointers), used by the
// parity tests to check one kernel at a time against the CPU checker.
#include <cstdlib>
#include <cstring>
#include <vector>

#include "engine.h"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "gemm_tc_pair.cuh"
#include "step_kernels.cuh"

namespace {
struct DevBuf {
  void* p = nullptr;
  ~DevBuf() { if (p) cudaFree(p); }
  cudaError_t alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 1); }
  template <class T> T* as() { return static_cast<T*>(p); }
};
#define KCK(x) do { if ((x) != cudaSuccess) return LINMT_ECUDA; } while (0)
}  // namespace

extern "C" {

int linmt_k_gemm(const float* X, const float* W, float* Y, int32_t R, int32_t K, int32_t N, int32_t gemm_path,
                 int32_t precision, int32_t device) {
  using namespace linmt;
  if (!X || !W || !Y || R < 1 || K < 1 || N < 1) return LINMT_EINVAL;
  if (gemm_path == LINMT_GEMM_SIMT && precision != LINMT_PREC_FP32) return LINMT_EINVAL;
  if (gemm_path != LINMT_GEMM_SIMT && gemm_path != LINMT_GEMM_TENSOR && gemm_path != LINMT_GEMM_TENSOR2 &&
      gemm_path != LINMT_GEMM_TENSOR3) return LINMT_EINVAL;
  KCK(cudaSetDevice(device));
  const int Kp = round_up(K, 64), Np = round_up(N, 128);
  std::vector<float> xp((size_t)R * Kp, 0.f), wt((size_t)Np * Kp, 0.f);
  for (int r = 0; r < R; ++r) std::memcpy(&xp[(size_t)r * Kp], X + (size_t)r * K, sizeof(float) * K);
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) wt[(size_t)n * Kp + k] = W[(size_t)k * N + n];
  DevBuf dx, dw, dy;
  KCK(dx.alloc(xp.size() * 4)); KCK(dw.alloc(wt.size() * 4)); KCK(dy.alloc((size_t)R * Np * 4));
  KCK(cudaMemcpy(dx.p, xp.data(), xp.size() * 4, cudaMemcpyHostToDevice));
  KCK(cudaMemcpy(dw.p, wt.data(), wt.size() * 4, cudaMemcpyHostToDevice));
  if (gemm_path == LINMT_GEMM_SIMT) {
    ASegs a{}; a.ptr[0] = dx.as<float>(); a.ld[0] = Kp; a.nseg = 1; a.seg_k = Kp;
    EpiBias e{nullptr, dy.as<float>(), Np};
    KCK(gemm_simt(a, dw.as<float>(), Kp, R, Np, Kp, e, 0));
    KCK(cudaDeviceSynchronize());
  } else {
    const int fmt = (precision == LINMT_PREC_FP32 && gemm_path == LINMT_GEMM_TENSOR) ? 1 : 0;
    const int nt = (precision == LINMT_PREC_BF16) ? 1 : (gemm_path == LINMT_GEMM_TENSOR3 ? 3 : 2);
    DevBuf pa[3], pb[3], derr;
    tc::Planes A{}, B{};
    A.ld = Kp; B.ld = Kp; A.fmt = fmt; B.fmt = fmt;
    for (int t = 0; t < nt; ++t) {
      KCK(pa[t].alloc(xp.size() * 2)); KCK(pb[t].alloc(wt.size() * 2));
      A.p[t] = pa[t].as<__nv_bfloat16>(); B.p[t] = pb[t].as<__nv_bfloat16>();
    }
    KCK(derr.alloc(4));
    KCK(cudaMemset(derr.p, 0, 4));
    tc::split_planes_kernel<<<256, 256>>>(dx.as<float>(), A, nt, xp.size());
    tc::split_planes_kernel<<<1024, 256>>>(dw.as<float>(), B, nt, wt.size());
    KCK(cudaGetLastError());
    const char* bk_env = std::getenv("LINMT_TC_BK");   // test knob: stage depth 64 (128-byte rows) for <= 2 planes
    const int bk = (fmt == 1 || (bk_env && std::atoi(bk_env) == 64 && nt <= 2)) ? 64 : 32;
    tc::TmapSet tm{};
    for (int t = 0; t < nt; ++t) {
      if (!tc::make_tmap(&tm.a[t], A.p[t], R, Kp, Kp, tc::BM, bk)) return LINMT_ECUDA;
      if (!tc::make_tmap(&tm.b[t], B.p[t], Np, Kp, Kp, 256)) return LINMT_ECUDA;
    }
    tc::TcEpiF32 e{nullptr, dy.as<float>(), Np, 0};
    int bn = 0, splits = 1;
    const size_t ws_floats = (size_t)16 << 20;
    int n_sm = 148;
    KCK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    tc::pick_shape(R, Np, Kp, nt, n_sm, ws_floats, 4096, &bn, &splits, fmt);
    DevBuf dws, dcnt;
    KCK(dws.alloc(ws_floats * 4)); KCK(dcnt.alloc(4096 * 4)); KCK(cudaMemset(dcnt.p, 0, 4096 * 4));
    // the engine's rule for CTA pairs: split operands, 64-deep stages, K not split, a shape that is down to two
    // stages as one tile, the row tiles (rounded up to even) in one wave; LINMT_TC_PAIR=0 keeps the one-tile kernel
    const char* pair_env = std::getenv("LINMT_TC_PAIR");
    const int mt = (R + tc::BM - 1) / tc::BM;
    const bool pair = !(pair_env && std::atoi(pair_env) == 0) && fmt == 1 && nt == 2 && bk == 64 && splits == 1 && mt >= 2 && bn % 16 == 0 &&
                      tc::make_shape(bn, nt, bk, fmt).stages < 3 && (long)((mt + 1) & ~1) * ((Np + bn - 1) / bn) <= n_sm &&
                      tc::max_resident_pairs<2, 64, 1, tc::TcEpiF32>() > 0;
    for (int t = 0; t < nt; ++t)
      if (!tc::make_tmap(&tm.b[t], B.p[t], Np, Kp, Kp, pair ? bn / 2 : bn, bk)) return LINMT_ECUDA;
    tc::Shape sh = pair ? tc::make_shape_pair(bn, nt, bk, fmt) : tc::make_shape(bn, nt, bk, fmt);
    sh.splits = splits;
    cudaError_t le = pair ? tc::launch_gemm_tc_pair<2, 64, 1, tc::TcEpiF32>(tm, R, Np, Kp, sh, e, derr.as<int>(), 0, nullptr, nullptr)
                          : tc::launch_gemm_tc(tm, R, Np, Kp, sh, e, derr.as<int>(), 0, dws.as<float>(), dcnt.as<int>());
    KCK(le);
    KCK(cudaDeviceSynchronize());
    int herr = 0;
    KCK(cudaMemcpy(&herr, derr.p, 4, cudaMemcpyDeviceToHost));
    if (herr) return LINMT_ECUDA;
  }
  std::vector<float> yp((size_t)R * Np);
  KCK(cudaMemcpy(yp.data(), dy.p, yp.size() * 4, cudaMemcpyDeviceToHost));
  for (int r = 0; r < R; ++r) std::memcpy(Y + (size_t)r * N, &yp[(size_t)r * Np], sizeof(float) * N);
  return LINMT_OK;
}

int linmt_k_softmax_topk(const float* logits, int32_t R, int32_t V, int32_t kk, int32_t* idx, float* logp,
                         float* eos_logp, int32_t device) {
  using namespace linmt;
  if (!logits || !idx || !logp || R < 1 || V < 2 || kk < 1 || kk > kMaxBeam + 1) return LINMT_EINVAL;
  KCK(cudaSetDevice(device));
  const int Vp = round_up(V, 4);
  std::vector<float> lp((size_t)R * Vp, 0.f);
  for (int r = 0; r < R; ++r) std::memcpy(&lp[(size_t)r * Vp], logits + (size_t)r * V, sizeof(float) * V);
  DevBuf dl, di, dp, de;
  KCK(dl.alloc(lp.size() * 4)); KCK(di.alloc((size_t)R * kk * 4)); KCK(dp.alloc((size_t)R * kk * 4)); KCK(de.alloc((size_t)R * 4));
  KCK(cudaMemcpy(dl.p, lp.data(), lp.size() * 4, cudaMemcpyHostToDevice));
  TopkOut o{di.as<int32_t>(), dp.as<float>(), de.as<float>(), nullptr};
  KCK(launch_softmax_topk(dl.as<float>(), Vp, V, kk, R, o, 1, 0));
  KCK(cudaDeviceSynchronize());
  KCK(cudaMemcpy(idx, di.p, (size_t)R * kk * 4, cudaMemcpyDeviceToHost));
  KCK(cudaMemcpy(logp, dp.p, (size_t)R * kk * 4, cudaMemcpyDeviceToHost));
  if (eos_logp) KCK(cudaMemcpy(eos_logp, de.p, (size_t)R * 4, cudaMemcpyDeviceToHost));
  return LINMT_OK;
}

}  // extern "C"

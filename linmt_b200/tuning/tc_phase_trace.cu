// tc_phase_trace.cu -- tuning aid, not part of the library: runs the tensor-core GEMM once with
// -DLINMT_TC_PROF, which makes every CTA stamp %globaltimer at its phases (start, prologue done,
// first stage landed, last MMA issued, accumulator complete, epilogue done, end), and prints the
// averages and a sample of CTAs.  Build and run on a B200:
//   python linmt_b200/build.py --phase-trace && ./linmt_b200/tuning/tc_phase_trace
#define LINMT_TC_PROF 1
#include <cstdio>
#include <vector>
#include <algorithm>
#include "../csrc/gemm_tc.cuh"
using namespace linmt;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s line %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)
int run(int R, int K, int N, int bn, int bk, bool lstm) {
  const int nt = 2;
  __nv_bfloat16 *pa[2], *pb[2];
  tc::Planes A{}, B{}; A.ld = K; B.ld = K; A.fmt = 1; B.fmt = 1;
  for (int t = 0; t < nt; ++t) {
    CK(cudaMalloc(&pa[t], (size_t)R * K * 2)); CK(cudaMalloc(&pb[t], (size_t)N * K * 2));
    CK(cudaMemset(pa[t], 0x2c, (size_t)R * K * 2)); CK(cudaMemset(pb[t], 0x2c, (size_t)N * K * 2));
    A.p[t] = pa[t]; B.p[t] = pb[t];
  }
  float *dy, *dc, *dbias; int* derr;
  CK(cudaMalloc(&dy, (size_t)R * N * 4)); CK(cudaMalloc(&dc, (size_t)R * N)); CK(cudaMalloc(&dbias, (size_t)N * 4)); CK(cudaMalloc(&derr, 4));
  CK(cudaMemset(derr, 0, 4)); CK(cudaMemset(dc, 0, (size_t)R * N)); CK(cudaMemset(dbias, 0, (size_t)N * 4));
  tc::Planes H{}; H.ld = N / 4; H.fmt = 1;
  for (int t = 0; t < nt; ++t) { __nv_bfloat16* q; CK(cudaMalloc(&q, (size_t)R * (N / 4) * 2)); H.p[t] = q; }
  tc::TmapSet tm{};
  for (int t = 0; t < nt; ++t) {
    if (!tc::make_tmap(&tm.a[t], A.p[t], R, K, K, tc::BM, bk)) return 2;
    if (!tc::make_tmap(&tm.b[t], B.p[t], N, K, K, bn, bk)) return 2;
  }
  tc::Shape sh = tc::make_shape(bn, nt, bk, 1);
  const int gx = (R + 127) / 128, gy = (N + bn - 1) / bn;
  unsigned long long* dprof;
  CK(cudaMalloc(&dprof, (size_t)gx * gy * 8 * 8));
  CK(cudaMemset(dprof, 0, (size_t)gx * gy * 8 * 8));
  CK(cudaMemcpyToSymbol(tc::g_tc_prof, &dprof, sizeof(dprof)));
  tc::TcEpiF32 e{nullptr, dy, N, 0};
  tc::TcEpiLstm el{};
  el.bias = dbias; el.c_prev = dc; el.ldc = N / 4; el.c_out = dc; el.h_out1 = H; el.h1_col0 = 0; el.h_out2 = tc::Planes{}; el.h_prev = tc::Planes{};
  el.h_f32 = nullptr; el.row_len = nullptr; el.pos = 0; el.nt = 2;
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  for (int i = 0; i < 5; ++i) {
    if (lstm) CK(tc::launch_gemm_tc(tm, R, N, K, sh, el, derr, 0)); else CK(tc::launch_gemm_tc(tm, R, N, K, sh, e, derr, 0));
  }
  CK(cudaDeviceSynchronize());
  cudaEventRecord(e0);
  if (lstm) CK(tc::launch_gemm_tc(tm, R, N, K, sh, el, derr, 0)); else CK(tc::launch_gemm_tc(tm, R, N, K, sh, e, derr, 0));
  cudaEventRecord(e1);
  CK(cudaDeviceSynchronize());
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  std::vector<unsigned long long> h((size_t)gx * gy * 8);
  CK(cudaMemcpy(h.data(), dprof, h.size() * 8, cudaMemcpyDeviceToHost));
  unsigned long long tmin = ~0ull, tmax = 0;
  for (size_t c = 0; c < (size_t)gx * gy; ++c) { tmin = std::min(tmin, h[c * 8]); tmax = std::max(tmax, h[c * 8 + 6]); }
  double s[7] = {0}; 
  for (size_t c = 0; c < (size_t)gx * gy; ++c) for (int k = 0; k < 7; ++k) s[k] += (double)(h[c * 8 + k] - tmin);
  printf("R %d K %d N %d bn %d bk %d %s: event %.1f us, ctas %d, span(first start..last end) %.1f us\n", R, K, N, bn, bk, lstm ? "lstm" : "f32", ms * 1e3, gx * gy, (tmax - tmin) / 1e3);
  const char* names[7] = {"start", "prologue done", "first stage landed", "last MMA issued", "accum ready (epi)", "epilogue done", "end"};
  for (int k = 0; k < 7; ++k) printf("   avg %-20s %8.2f us\n", names[k], s[k] / (gx * gy) / 1e3);
  // per-CTA for first few and by wave
  for (size_t c = 0; c < (size_t)gx * gy; c += std::max<size_t>(1, (size_t)gx * gy / 12)) {
    printf("   cta %4zu:", c);
    for (int k = 0; k < 7; ++k) printf(" %7.2f", (h[c * 8 + k] - tmin) / 1e3);
    printf("\n");
  }
  return 0;
}
int main() {
  run(768, 2048, 4096, 176, 64, false);
  run(768, 2048, 4096, 176, 64, true);
  run(768, 1024, 30016, 256, 32, false);
  run(768, 64, 4096, 176, 64, false);
  return 0;
}

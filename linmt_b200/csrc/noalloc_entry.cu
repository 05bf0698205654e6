// noalloc_entry.cu -- a dense product on the tensor-core kernel for callers that must not
// allocate device memory.
//
// Some hosts of this library hand the whole GPU to a memory pool of their own at start-up (a
// serving process with a fixed arena, a framework allocator that owns every byte) or run where a
// cudaMalloc would stall the device for everyone sharing it.  For them this file provides ONE
// entry point that calls no cudaMalloc / cudaFree and no allocating library routine: the bf16
// operand planes the kernel needs as working memory live in a file-scope __device__ array that
// every GPU loading the library holds until the process exits.
#include <mutex>

#include "engine.h"
#include "gemm_tc.cuh"

namespace {

constexpr int kMaxR = 256;    // most rows of X
constexpr int kMaxK = 1024;   // most columns of X / Wt
constexpr int kMaxN = 1024;   // most rows of Wt
constexpr size_t kAElems = (size_t)kMaxR * kMaxK;
constexpr size_t kBElems = (size_t)kMaxN * kMaxK;
constexpr size_t kFlagOffset = 0;                        // int error flag, first 256 bytes
constexpr size_t kAOffset = 256;                         // 3 planes of X
constexpr size_t kBOffset = kAOffset + 3 * 2 * kAElems;  // 3 planes of Wt
constexpr size_t kScratchBytes = kBOffset + 3 * 2 * kBElems;   // 7.5 MiB + 256 B

// Working memory of linmt_gemm_f32_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress, never an address to pass to a kernel.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of the scratch array on `device` (which must be current) and the device's SM count.  The
// first call on a device asks the runtime for both and checks the answers; later calls reuse them.
cudaError_t scratch_address(int device, unsigned char** out, int* n_sm) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess) return e;
    if (!p) return cudaErrorInvalidSymbol;
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return e;
    g_sm_count[device] = sms > 0 ? sms : 1;
    g_scratch_addr[device] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[device];
  *n_sm = g_sm_count[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int linmt_gemm_f32_noalloc(const float* d_x, const float* d_wt, float* d_y, int32_t R, int32_t K, int32_t N,
                                      int32_t device) {
  using namespace linmt;
  if (!d_x || !d_wt || !d_y || R < 1 || K < 1 || N < 1) return LINMT_EINVAL;
  if (device < 0 || device >= kMaxDevices) return LINMT_EINVAL;
  if (R > kMaxR || K > kMaxK || N > kMaxN) return LINMT_ELIMIT;   // beyond the built-in working memory
  if (K % tc::BK != 0 || N % 16 != 0) return LINMT_EINVAL;        // no room to pad without allocating
  if (cudaSetDevice(device) != cudaSuccess) return LINMT_ECUDA;
  unsigned char* scratch = nullptr;
  int n_sm = 1;
  if (scratch_address(device, &scratch, &n_sm) != cudaSuccess) return LINMT_ECUDA;

  int* d_err = reinterpret_cast<int*>(scratch + kFlagOffset);
  tc::Planes A{}, B{};
  A.ld = K; B.ld = K;
  for (int t = 0; t < 3; ++t) {
    A.p[t] = reinterpret_cast<__nv_bfloat16*>(scratch + kAOffset) + (size_t)t * kAElems;
    B.p[t] = reinterpret_cast<__nv_bfloat16*>(scratch + kBOffset) + (size_t)t * kBElems;
  }
  // the flag is the only part of the array that must start at zero; the planes are overwritten
  if (cudaMemsetAsync(d_err, 0, sizeof(int), 0) != cudaSuccess) return LINMT_ECUDA;
  tc::split_planes_kernel<<<128, 256>>>(d_x, A, 3, (size_t)R * K);
  tc::split_planes_kernel<<<256, 256>>>(d_wt, B, 3, (size_t)N * K);
  if (cudaGetLastError() != cudaSuccess) return LINMT_ECUDA;
  const int bn = tc::pick_bn(R, N, n_sm);
  tc::TmapSet tm{};
  for (int t = 0; t < 3; ++t) {
    if (!tc::make_tmap(&tm.a[t], A.p[t], R, K, K, tc::BM)) return LINMT_ECUDA;
    if (!tc::make_tmap(&tm.b[t], B.p[t], N, K, K, bn)) return LINMT_ECUDA;
  }
  tc::TcEpiF32 e{nullptr, d_y, N, 0};
  if (tc::launch_gemm_tc(tm, R, N, K, tc::make_shape(bn, 3), e, d_err, 0) != cudaSuccess) return LINMT_ECUDA;
  int herr = 0;
  if (cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return LINMT_ECUDA;
  return herr ? LINMT_ECUDA : LINMT_OK;
}

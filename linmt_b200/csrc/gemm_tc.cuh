// gemm_tc.cuh -- tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in TMEM,
// operands brought to shared memory by TMA (no multicast), fused epilogues.
//
//   C[M][N] = A[M][K] . Wt[N][K]^T        (both operands K-contiguous, "K-major")
//
// Precision.  The tensor cores multiply 16-bit operands.  An fp32 operand x is held as planes.
// Plane format 0: NT bf16 planes x ~ p0 + p1 (+ p2), p0 = bf16(x), p1 = bf16(x - p0), p2 = bf16(x - p0 - p1);
// a product of two split operands is the sum of the partial products whose weight is at least 2^-16
// (NT = 3: p0p0, p0p1, p1p0, p1p1, p0p2, p2p0 -- error ~2^-23 per product, i.e. fp32-class
// results; NT = 2: p0p0, p0p1, p1p0, p1p1 -- error ~2^-17; NT = 1: plain bf16).
// Plane format 1 ("f16 pair", the default for fp32 weights) reaches the same accuracy with half the
// tensor work: x ~ a0 + 2^-11 a1 with a0 = fp16(x), a1 = fp16((x - a0) * 2^11) -- two 11-bit mantissas,
// 22 bits in all, the residual scaled back into fp16's normal range -- and three partial products a0b0
// (own accumulator), a0b1 + a1b0 (second accumulator, weighted 2^-11 when the two are added); the
// dropped a1b1 weighs 2^-22.  Operands must stay below fp16's largest finite value (65504).
// The tensor core truncates a little on every accumulate, in units of the accumulator's magnitude, so
// the leading product has a TMEM accumulator of its own, drained into fp32 registers every few k-blocks
// (two-level accumulation), and the small cross terms share a second one; the epilogue adds the two.
// Measured against a float64 product this gives the error of an fp32 FMA loop.
//
// One CTA computes one 128 x BN tile; BN (a multiple of 16 up to 256) is a launch parameter so
// the host can size the grid to the 148 SMs for every problem shape.  Warp 0 issues the TMA
// loads, warp 1 owns TMEM and issues the leading-product MMAs, warps 2..17 run the epilogue
// (tcgen05.ld -> registers -> fused math -> staging in the idle stage ring -> coalesced stores; four
// warps per TMEM lane quadrant, each a contiguous block of columns), warp 18 issues the cross-term
// MMAs.  The issuing threads are the critical path of a narrow tile, so their loops carry descriptors
// forward by constant increments and everything that can be is a compile-time constant; the waiting
// epilogue warps sleep between polls.  A ring of shared-memory stages is handed back and forth with
// mbarriers; every wait is bounded and reports through an error flag instead of hanging.  All kernels
// take part in programmatic dependent launch (see pdl_wait below).  A persistent variant
// (gemm_tc_persist_kernel) serves the many-wave vocabulary GEMM; gemm_tc_pair.cuh holds the forms of both kernels
// that run on CTA pairs (tcgen05 cta_group::2), used where a launch is wide enough for them to pay.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace linmt {
namespace tc {

constexpr int BM = 128;
constexpr int BK = 32;             // bf16 elements per stage row = 64 bytes -> 64-byte swizzle
constexpr int UMMA_K = 16;         // bf16 elements per tcgen05.mma
constexpr int kEpiWarps = 16;        // epilogue warps: four per TMEM lane quadrant
constexpr int kThreads = 64 + 32 * kEpiWarps;  // warp 0 TMA, warp 1 MMA, then the epilogue warps
// The one-tile kernel has a second MMA-issuing warp after the epilogue warps: with split operands the
// leading product and the cross terms go to different accumulators, so two threads can issue them
// independently -- a narrow tile is bound by what ONE thread can issue (~58 ns per MMA).
constexpr int kIssue2Warp = 2 + kEpiWarps;
constexpr int kThreadsMain = kThreads + 32;
constexpr unsigned long long kWaitCycles = 2000000000ull;  // ~1 s at 2 GHz

struct alignas(64) TmapSet {
  CUtensorMap a[3];
  CUtensorMap b[3];
};

constexpr int A_BYTES = BM * BK * 2;         // one plane of the A tile of a stage
constexpr int SMEM_BUDGET = 222 * 1024;
constexpr int TMEM_COLS = 512;         // two accumulators of up to 256 columns each
constexpr int kMaxStages = 8;
constexpr int kDrainDefault = 4;       // k-blocks of the leading product per TMEM partial sum (see kernel)

struct Shape {
  int bn;        // tile width
  int bk;        // K depth of a stage in bf16 elements: 32 (64-byte rows) or 64 (128-byte rows)
  int nt;        // planes per operand
  int fmt;       // 0 = bf16 planes, 1 = f16 pair
  int stages;
  int stage_bytes;
  int smem_bytes;
  int drain;     // k-blocks between drains of the leading accumulator
  int splits;    // split-K factor (1 = none)
  int pdl;       // launch with programmatic stream serialization
};
// Dynamic shared memory of a launch: the stage ring (which the epilogue warps reuse as their
// staging areas once the accumulator is complete, kEpiStagingBytes in all), alignment slack, barriers.
constexpr int kEpiStagingBytes = kEpiWarps * 9728;
__host__ __device__ inline int ring_bytes(int stages, int stage_bytes) {
  return stages * stage_bytes > kEpiStagingBytes ? stages * stage_bytes : kEpiStagingBytes;
}
inline int shape_smem_bytes(int stages, int stage_bytes) { return ring_bytes(stages, stage_bytes) + 1024 + 256; }
inline Shape make_shape(int bn, int nt, int bk = BK, int fmt = 0) {
  Shape s;
  s.bn = bn; s.nt = nt; s.bk = bk; s.fmt = fmt;
  s.stage_bytes = nt * (BM * bk * 2 + bn * bk * 2);
  s.stages = SMEM_BUDGET / s.stage_bytes;
  if (s.stages > kMaxStages) s.stages = kMaxStages;
  s.smem_bytes = shape_smem_bytes(s.stages, s.stage_bytes);
  s.drain = kDrainDefault;
  s.splits = 1;
  s.pdl = 0;
  return s;
}

// ---- programmatic dependent launch ----------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start (prologue, loads of
// constant data) while its predecessor in the stream is still finishing; it must not touch
// anything the predecessor writes or reads-then-overwrites before pdl_wait() returns.  Every
// kernel of the decoder step announces itself with pdl_launch_dependents() at its start, so the
// next kernel's CTAs take over SMs as this kernel's last CTAs leave them.  Without the launch
// attribute both calls do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <class... KArgs, class... Args>
inline cudaError_t launch_k(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and raises *abort_flag) when the phase does not complete in
// about a second or when another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((unsigned long long)clock64() - t0 > kWaitCycles) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 64 bytes (BK bf16) with
// the 64-byte swizzle TMA wrote (8-row groups 512 bytes apart), or 128-byte rows with the
// 128-byte swizzle (groups 1024 bytes apart).
//   bits 0-13 start address >> 4 | 16-29 leading byte offset >> 4 (unused here) |
//   32-45 stride byte offset >> 4 | 46-47 descriptor version (1) | 61-63 swizzle (4 = 64 B)
template <int BKT>
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((8u * BKT * 2u) >> 4) << 32;   // 8-row groups: 512 bytes apart (64-byte rows) or 1024 (128-byte rows)
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(BKT == 64 ? 2 : 4) << 61;      // swizzle: 128 bytes / 64 bytes
  return d;
}
// Instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = bf16 (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
// f16 operands (plane format 1) have format code 0 in both fields.
__host__ __device__ inline uint32_t make_idesc(int m, int n, int fmt = 0) {
  const uint32_t ab = fmt ? 0u : ((1u << 7) | (1u << 10));
  return (1u << 4) | ab | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- operand planes -----------------------------------------------------------------------
// An activation or weight matrix as NT bf16 planes with a common leading dimension.
// fmt 0: p0 = bf16(x), p1 = bf16(x - p0), p2 = bf16(x - p0 - p1).
// fmt 1: two planes holding fp16 bit patterns, p0 = fp16(x), p1 = fp16((x - p0) * 2048).
struct Planes {
  __nv_bfloat16* p[3];
  int ld;
  int fmt;
};
constexpr float kF16PairScale = 2048.0f;             // 2^11: the residual plane's scale
constexpr float kF16PairInvScale = 1.0f / 2048.0f;
__device__ __forceinline__ void f16_pair(float x, unsigned short& h0, unsigned short& h1) {
  const __half a0 = __float2half_rn(x);
  h0 = __half_as_ushort(a0);
  h1 = __half_as_ushort(__float2half_rn((x - __half2float(a0)) * kF16PairScale));
}
__device__ __forceinline__ void split_store(const Planes& pl, int nt, size_t idx, float x) {
  if (pl.fmt == 1) {
    unsigned short h0, h1;
    f16_pair(x, h0, h1);
    reinterpret_cast<unsigned short*>(pl.p[0])[idx] = h0;
    reinterpret_cast<unsigned short*>(pl.p[1])[idx] = h1;
    return;
  }
  const __nv_bfloat16 b0 = __float2bfloat16_rn(x);
  pl.p[0][idx] = b0;
  if (nt > 1) {
    const float r1 = x - __bfloat162float(b0);
    const __nv_bfloat16 b1 = __float2bfloat16_rn(r1);
    pl.p[1][idx] = b1;
    if (nt > 2) pl.p[2][idx] = __float2bfloat16_rn(r1 - __bfloat162float(b1));
  }
}
// The value a consumer of the planes sees.
__device__ __forceinline__ float planes_value(float x, int nt) {
  const __nv_bfloat16 b0 = __float2bfloat16_rn(x);
  if (nt == 1) return __bfloat162float(b0);
  return x;
}

// ---- epilogues: called per (row, 16 consecutive columns) ------------------------------------

// Four consecutive values as bf16 planes with one 8-byte store per plane (idx a multiple of 4).
__device__ __forceinline__ void split_store4(const Planes& pl, int nt, size_t idx, float x0, float x1, float x2, float x3) {
  const float x[4] = {x0, x1, x2, x3};
  if (pl.fmt == 1) {
    unsigned short h0[4], h1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f16_pair(x[i], h0[i], h1[i]);
    *reinterpret_cast<uint2*>(pl.p[0] + idx) = make_uint2((uint32_t)h0[0] | ((uint32_t)h0[1] << 16), (uint32_t)h0[2] | ((uint32_t)h0[3] << 16));
    *reinterpret_cast<uint2*>(pl.p[1] + idx) = make_uint2((uint32_t)h1[0] | ((uint32_t)h1[1] << 16), (uint32_t)h1[2] | ((uint32_t)h1[3] << 16));
    return;
  }
  float r[4];
  __nv_bfloat16 b[4];
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    if (t < nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float src = (t == 0) ? x[i] : r[i];
        b[i] = __float2bfloat16_rn(src);
        r[i] = src - __bfloat162float(b[i]);
      }
      uint2 w;
      w.x = (uint32_t)__bfloat16_as_ushort(b[0]) | ((uint32_t)__bfloat16_as_ushort(b[1]) << 16);
      w.y = (uint32_t)__bfloat16_as_ushort(b[2]) | ((uint32_t)__bfloat16_as_ushort(b[3]) << 16);
      *reinterpret_cast<uint2*>(pl.p[t] + idx) = w;
    }
  }
}

// Activation functions of the fused epilogues.  The hardware exponential (ex2.approx, 2 ulp) and
// reciprocal keep the ABSOLUTE error of both below ~1.5e-7 -- what the matrix products that consume h
// care about -- at a third of the instructions of expf / tanhf; around zero, where
// 1 - 2 / (1 + e^2x) would cancel, tanh uses its odd series instead (relative error < 1e-7 for |x| < 0.25).
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float tanh_fast(float x) {
  const float x2 = x * x;
  // x - x^3/3 + 2x^5/15 - 17x^7/315 + 62x^9/2835
  float p = fmaf(x2, 62.0f / 2835.0f, -17.0f / 315.0f);
  p = fmaf(x2, p, 2.0f / 15.0f);
  p = fmaf(x2, p, -1.0f / 3.0f);
  p = fmaf(x2 * x, p, x);
  const float big = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * x));
  return x2 < 0.0625f ? p : big;
}

// Per-warp staging area of the epilogue (lives in the idle pipeline stages once the accumulator is
// complete): the tcgen05.ld layout gives every lane one ROW of the tile, so a direct store touches
// 32 different lines per instruction; staging a block of up to 64 columns and storing it back
// with consecutive lanes on consecutive addresses cuts the memory-pipe passes 4-8x (measured: the
// epilogue was 7.6-7.9 us of a 29-36 us tile).
constexpr int kEpiBlockChunks = 4;                       // 16-column chunks a warp owns at most
constexpr int kEpiScratchStride = 68;                    // floats per staged row (64 + 4: conflict-free float4 rows)
constexpr int kEpiScratchBytes = kEpiStagingBytes / kEpiWarps;   // per warp: 32 x 68 floats, or the LSTM epilogue's c | h planes | h
static_assert(kEpiScratchBytes >= 32 * kEpiScratchStride * 4 && kEpiScratchBytes >= (32 * 20 + 3 * 32 * 12 + 32 * 20) * 4, "staging area");

// LSTM cell update on gate-interleaved columns (see EpiLstm in gemm_simt.cuh for the math and
// the reference kernels it replaces).  A call covers 16 columns = 4 hidden units, so every
// access is a 16-byte (fp32) or 8-byte (bf16 plane) vector.  h goes out as bf16 planes to up to
// two places (the operand panels that read it next) and optionally as fp32 (encoder top states).
struct TcEpiLstm {
  const float* bias;
  const float* c_prev; int ldc;
  float* c_out;
  Planes h_out1; int h1_col0;      // element (row, j) at plane[row * ld + h1_col0 + j]
  Planes h_out2; int h2_col0;      // optional (p[0] == nullptr: none)
  Planes h_prev; int hp_col0;      // read for rows past their length (encoder)
  float* h_f32; long long hf_row_stride;  // optional fp32 copy, element (row, j) at h_f32[row*stride + j]
  const int* row_len; int pos;
  int nt;
  // Optional beam reordering of the cell state: row r continues slot c_parent[r] of its sentence (k slots per
  // sentence), so c_prev is read from that row -- the state then needs no copy between steps.
  const int32_t* c_parent = nullptr; int c_k = 1;
  // Optional precomputed input term: xw[tok][col] = (W_x . embedding(tok))[col] for every vocabulary entry, added
  // to the accumulator of row r with tok = x_tok[r] (out-of-range ids count as x_unk) -- the embedding part of
  // the first decoder layer's product then costs a row lookup instead of a third of the GEMM.
  const float* xw = nullptr; const int32_t* x_tok = nullptr; int x_ld = 0; int x_vocab = 0; int x_unk = 0;
  __device__ __forceinline__ int x_row(int row) const {
    const int t = x_tok[row];
    return (t < 0 || t >= x_vocab) ? x_unk : t;
  }
  __device__ __forceinline__ int c_src_row(int row) const { return c_parent ? (row / c_k) * c_k + c_parent[row] : row; }
  __device__ __forceinline__ void operator()(int row, int col0, const float* v_in) const {
    float vx[16];
    const float* v = v_in;
    if (xw) {
      const float* xr = xw + (size_t)x_row(row) * x_ld + col0;
#pragma unroll
      for (int i = 0; i < 16; ++i) vx[i] = v_in[i] + xr[i];
      v = vx;
    }
    const bool active = (row_len == nullptr) || (pos < row_len[row]);
    const int j0 = col0 >> 2;
    const size_t ic = (size_t)row * ldc + j0;
    const float4 cp = *reinterpret_cast<const float4*>(c_prev + (size_t)c_src_row(row) * ldc + j0);
    const size_t i1 = (size_t)row * h_out1.ld + h1_col0 + j0;
    const size_t i2 = (size_t)row * h_out2.ld + h2_col0 + j0;
    if (active) {
      const float cpv[4] = {cp.x, cp.y, cp.z, cp.w};
      float c[4], h[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float4 b = *reinterpret_cast<const float4*>(bias + col0 + 4 * u);
        const float gi = sigmoid_fast(v[4 * u + 0] + b.x);
        const float gf = sigmoid_fast(v[4 * u + 1] + b.y);
        const float gg = tanh_fast(v[4 * u + 2] + b.z);
        const float go = sigmoid_fast(v[4 * u + 3] + b.w);
        c[u] = gf * cpv[u] + gi * gg;
        h[u] = go * tanh_fast(c[u]);
      }
      *reinterpret_cast<float4*>(c_out + ic) = make_float4(c[0], c[1], c[2], c[3]);
      split_store4(h_out1, nt, i1, h[0], h[1], h[2], h[3]);
      if (h_out2.p[0]) split_store4(h_out2, nt, i2, h[0], h[1], h[2], h[3]);
      if (h_f32)   // the value every other consumer of h sees: rounded to bf16 in bf16 precision, as it is with fp32 weights
        *reinterpret_cast<float4*>(h_f32 + (size_t)row * hf_row_stride + j0) =
            make_float4(planes_value(h[0], nt), planes_value(h[1], nt), planes_value(h[2], nt), planes_value(h[3], nt));
    } else {
      *reinterpret_cast<float4*>(c_out + ic) = cp;
      const size_t ip = (size_t)row * h_prev.ld + hp_col0 + j0;
#pragma unroll
      for (int t = 0; t < 3; ++t)
        if (t < nt) {
          const uint2 hv = *reinterpret_cast<const uint2*>(h_prev.p[t] + ip);
          *reinterpret_cast<uint2*>(h_out1.p[t] + i1) = hv;
          if (h_out2.p[0]) *reinterpret_cast<uint2*>(h_out2.p[t] + i2) = hv;
        }
    }
  }
  // A warp's block: rows row0 .. row0+31 (lane = row), nch chunks of 16 accumulator columns from
  // col_first, i.e. nu = 4 * nch hidden units from j_first = col_first / 4.  v[ci] = chunk ci of
  // this lane's row.  sbuf = this warp's staging area.  c_prev comes in and c goes out through
  // the staging area with consecutive lanes on consecutive addresses; h goes out as planes the
  // same way.  Rows past their length (encoder) keep c and copy h_prev.
  static constexpr bool kHasBlock = true;
  static constexpr bool kHasPmax = false;
  __device__ __forceinline__ void block(int row0, int lane, int M, int col_first, int nch, float (*v)[16], float* sbuf, int /*slot*/) const {
    const int nq = nch;                      // float4 groups (4 hidden units each) per row
    const int j_first = col_first >> 2;
    const int row = row0 + lane;
    const bool valid = row < M;
    const bool active = valid && ((row_len == nullptr) || (pos < row_len[row]));
    float* cs = sbuf;                                            // [32][20] floats: c_prev in, c out
    unsigned short* hs = reinterpret_cast<unsigned short*>(sbuf + 32 * 20);   // [planes][32][24] 16-bit
    float* hf = sbuf + 32 * 20 + 3 * 32 * 12;                    // [32][20] floats: h in fp32 (only if h_f32)
    if (xw) {
      // the rows of the input-term table for this block, staged coalesced, then added lane = row
      const int nq4 = 4 * nch;
      for (int s = lane; s < 32 * nq4; s += 32) {
        const int r = s / nq4, g = s - r * nq4;
        if (row0 + r < M)
          *reinterpret_cast<float4*>(sbuf + r * kEpiScratchStride + 4 * g) =
              *reinterpret_cast<const float4*>(xw + (size_t)x_row(row0 + r) * x_ld + col_first + 4 * g);
      }
      __syncwarp();
      if (valid) {
#pragma unroll
        for (int ci = 0; ci < kEpiBlockChunks; ++ci) {
          if (ci < nch) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 t = *reinterpret_cast<const float4*>(sbuf + lane * kEpiScratchStride + 16 * ci + 4 * q);
              v[ci][4 * q] += t.x; v[ci][4 * q + 1] += t.y; v[ci][4 * q + 2] += t.z; v[ci][4 * q + 3] += t.w;
            }
          }
        }
      }
      __syncwarp();
    }
    // c_prev: coalesced load into the staging area
    for (int s = lane; s < 32 * nq; s += 32) {
      const int r = s / nq, g = s - r * nq;
      if (row0 + r < M)
        *reinterpret_cast<float4*>(cs + r * 20 + 4 * g) =
            *reinterpret_cast<const float4*>(c_prev + (size_t)c_src_row(row0 + r) * ldc + j_first + 4 * g);
    }
    __syncwarp();
    if (active) {
#pragma unroll
      for (int ci = 0; ci < kEpiBlockChunks; ++ci) {
        if (ci < nch) {
          const float4 cp = *reinterpret_cast<const float4*>(cs + lane * 20 + 4 * ci);
          const float cpv[4] = {cp.x, cp.y, cp.z, cp.w};
          float c[4], h[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float4 b = *reinterpret_cast<const float4*>(bias + col_first + 16 * ci + 4 * u);
            const float gi = sigmoid_fast(v[ci][4 * u + 0] + b.x);
            const float gf = sigmoid_fast(v[ci][4 * u + 1] + b.y);
            const float gg = tanh_fast(v[ci][4 * u + 2] + b.z);
            const float go = sigmoid_fast(v[ci][4 * u + 3] + b.w);
            c[u] = gf * cpv[u] + gi * gg;
            h[u] = go * tanh_fast(c[u]);
          }
          *reinterpret_cast<float4*>(cs + lane * 20 + 4 * ci) = make_float4(c[0], c[1], c[2], c[3]);
          if (h_f32)
            *reinterpret_cast<float4*>(hf + lane * 20 + 4 * ci) =
                make_float4(planes_value(h[0], nt), planes_value(h[1], nt), planes_value(h[2], nt), planes_value(h[3], nt));
          // planes of h: 4 units = 8 bytes per plane
          unsigned short q0[4], q1[4], q2[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (h_out1.fmt == 1) { f16_pair(h[u], q0[u], q1[u]); q2[u] = 0; }
            else {
              const __nv_bfloat16 b0 = __float2bfloat16_rn(h[u]);
              const float r1 = h[u] - __bfloat162float(b0);
              const __nv_bfloat16 b1 = __float2bfloat16_rn(r1);
              q0[u] = __bfloat16_as_ushort(b0); q1[u] = __bfloat16_as_ushort(b1);
              q2[u] = __bfloat16_as_ushort(__float2bfloat16_rn(r1 - __bfloat162float(b1)));
            }
          }
          *reinterpret_cast<uint2*>(hs + (0 * 32 + lane) * 24 + 4 * ci) = make_uint2(q0[0] | ((uint32_t)q0[1] << 16), q0[2] | ((uint32_t)q0[3] << 16));
          if (nt > 1) *reinterpret_cast<uint2*>(hs + (1 * 32 + lane) * 24 + 4 * ci) = make_uint2(q1[0] | ((uint32_t)q1[1] << 16), q1[2] | ((uint32_t)q1[3] << 16));
          if (nt > 2) *reinterpret_cast<uint2*>(hs + (2 * 32 + lane) * 24 + 4 * ci) = make_uint2(q2[0] | ((uint32_t)q2[1] << 16), q2[2] | ((uint32_t)q2[3] << 16));
        }
      }
    } else if (valid) {
      // past the end of this row's sentence: c stays (already staged), h = h_prev
      const size_t ip = (size_t)row * h_prev.ld + hp_col0 + j_first;
      for (int t = 0; t < nt; ++t)
        for (int g = 0; g < nch; ++g)
          *reinterpret_cast<uint2*>(hs + (t * 32 + lane) * 24 + 4 * g) = *reinterpret_cast<const uint2*>(h_prev.p[t] + ip + 4 * g);
    }
    const unsigned active_mask = __ballot_sync(0xffffffffu, active);
    __syncwarp();
    // coalesced stores
    for (int s = lane; s < 32 * nq; s += 32) {
      const int r = s / nq, g = s - r * nq;
      if (row0 + r < M) {
        *reinterpret_cast<float4*>(c_out + (size_t)(row0 + r) * ldc + j_first + 4 * g) = *reinterpret_cast<const float4*>(cs + r * 20 + 4 * g);
        if (h_f32 && ((active_mask >> r) & 1u))
          *reinterpret_cast<float4*>(h_f32 + (size_t)(row0 + r) * hf_row_stride + j_first + 4 * g) = *reinterpret_cast<const float4*>(hf + r * 20 + 4 * g);
      }
    }
    for (int t = 0; t < nt; ++t)
      for (int s = lane; s < 32 * nq; s += 32) {
        const int r = s / nq, g = s - r * nq;
        if (row0 + r < M) {
          const uint2 hv = *reinterpret_cast<const uint2*>(hs + (t * 32 + r) * 24 + 4 * g);
          *reinterpret_cast<uint2*>(h_out1.p[t] + (size_t)(row0 + r) * h_out1.ld + h1_col0 + j_first + 4 * g) = hv;
          if (h_out2.p[0]) *reinterpret_cast<uint2*>(h_out2.p[t] + (size_t)(row0 + r) * h_out2.ld + h2_col0 + j_first + 4 * g) = hv;
        }
      }
    __syncwarp();
  }
};

// out = tanh(acc [+ add] + bias) as bf16 planes (the attentional state).  `add` is an optional fp32 term per
// element, add[row * ld_add + col]: the part of the pre-activation that was computed ahead of this product.
struct TcEpiBiasTanh {
  const float* bias;
  Planes out; int col_off;
  int nt;
  const float* add = nullptr; int ld_add = 0;
  static constexpr bool kHasBlock = false;
  static constexpr bool kHasPmax = false;
  __device__ __forceinline__ void block(int, int, int, int, int, float (*)[16], float*, int) const {}
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    const size_t idx = (size_t)row * out.ld + col_off + col0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 b = *reinterpret_cast<const float4*>(bias + col0 + 4 * q);
      float4 a = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      if (add) {
        const float4 g = *reinterpret_cast<const float4*>(add + (size_t)row * ld_add + col0 + 4 * q);
        a.x += g.x; a.y += g.y; a.z += g.z; a.w += g.w;
      }
      split_store4(out, nt, idx + 4 * q, tanh_fast(a.x + b.x), tanh_fast(a.y + b.y), tanh_fast(a.z + b.z), tanh_fast(a.w + b.w));
    }
  }
};

// fp32 out, tanh on columns below `split`, optional bias (attention projections, logits).
struct TcEpiF32 {
  const float* bias;  // may be null
  float* out; int ld;
  int split;          // columns < split get tanh
  // Optional by-product for the softmax that follows a logits GEMM: the maximum of every block of up to
  // 64 columns (tile column block `slot`) of every row, over columns < n_valid, at pmax[row * pmax_ld + slot].
  // The softmax kernel then needs no first sweep over the row for its maximum and its top-k threshold.
  float* pmax = nullptr; int pmax_ld = 0; int n_valid = 0;
  // Optional half-precision output (out16 set: `out` is not written): logits whose few values that matter one by one
  // are recomputed by their consumer and which otherwise only enter a sum of exponentials go out as fp16, half
  // the bytes to write and to sweep.  The block maxima are then those of the ROUNDED values (elements of the row).
  __half* out16 = nullptr;
  __device__ __forceinline__ float4 finish4(float4 r, int col0) const {
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + col0);
      r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
    }
    if (col0 < split) { r.x = tanh_fast(r.x); r.y = tanh_fast(r.y); r.z = tanh_fast(r.z); r.w = tanh_fast(r.w); }
    if (out16) {
      r.x = __half2float(__float2half_rn(r.x)); r.y = __half2float(__float2half_rn(r.y));
      r.z = __half2float(__float2half_rn(r.z)); r.w = __half2float(__float2half_rn(r.w));
    }
    return r;
  }
  // four consecutive finished values to row-major element index idx (a multiple of 4)
  __device__ __forceinline__ void store4(size_t idx, const float4& r) const {
    if (out16) {
      const __half2 lo = __floats2half2_rn(r.x, r.y), hi = __floats2half2_rn(r.z, r.w);
      *reinterpret_cast<uint2*>(out16 + idx) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
      *reinterpret_cast<float4*>(out + idx) = r;
    }
  }
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    const size_t o = (size_t)row * ld + col0;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      store4(o + 4 * q, finish4(make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]), col0 + 4 * q));
  }
  // Block form (see TcEpiLstm::block): bias / tanh in registers, the block of up to 64 columns
  // staged per row, then stored with a row's 16 float4 on consecutive lanes.
  static constexpr bool kHasBlock = true;
  static constexpr bool kHasPmax = true;
  __device__ __forceinline__ void pmax_store(int row, int M, int slot, float m) const {
    if (pmax && row < M) pmax[(size_t)row * pmax_ld + slot] = m;
  }
  __device__ __forceinline__ float max4(float m, const float4& r, int c) const {
    if (c + 0 < n_valid) m = fmaxf(m, r.x);
    if (c + 1 < n_valid) m = fmaxf(m, r.y);
    if (c + 2 < n_valid) m = fmaxf(m, r.z);
    if (c + 3 < n_valid) m = fmaxf(m, r.w);
    return m;
  }
  // the same block without staging (row-per-lane stores), for callers whose staging area is busy
  __device__ __forceinline__ void direct_block(int row, int M, int col_first, int nch, float (*v)[16], int slot) const {
    float m = -INFINITY;
    if (row < M) {
#pragma unroll
      for (int ci = 0; ci < kEpiBlockChunks; ++ci) {
        if (ci < nch) {
          const int col0 = col_first + 16 * ci;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 r = finish4(make_float4(v[ci][4 * q], v[ci][4 * q + 1], v[ci][4 * q + 2], v[ci][4 * q + 3]), col0 + 4 * q);
            store4((size_t)row * ld + col0 + 4 * q, r);
            m = max4(m, r, col0 + 4 * q);
          }
        }
      }
    }
    pmax_store(row, M, slot, m);
  }
  // Stages nch (<= 4) chunks of this warp's 32 rows with `stride` floats per row (>= 16 * nch + 4) and
  // stores them with consecutive lanes on consecutive addresses; returns this lane's (= row's) maximum
  // over the valid columns.
  __device__ __forceinline__ float stage_store(int row0, int lane, int M, int col_first, int nch, float (*v)[16], float* sbuf,
                                               int stride) const {
    float m = -INFINITY;
#pragma unroll
    for (int ci = 0; ci < kEpiBlockChunks; ++ci) {
      if (ci < nch) {
        const int col0 = col_first + 16 * ci;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 r = finish4(make_float4(v[ci][4 * q], v[ci][4 * q + 1], v[ci][4 * q + 2], v[ci][4 * q + 3]), col0 + 4 * q);
          *reinterpret_cast<float4*>(sbuf + lane * stride + 16 * ci + 4 * q) = r;
          m = max4(m, r, col0 + 4 * q);
        }
      }
    }
    __syncwarp();
    const int nq = 4 * nch;   // float4 per row
    for (int s = lane; s < 32 * nq; s += 32) {
      const int r = s / nq, g = s - r * nq;
      if (row0 + r < M) store4((size_t)(row0 + r) * ld + col_first + 4 * g, *reinterpret_cast<const float4*>(sbuf + r * stride + 4 * g));
    }
    __syncwarp();
    return m;
  }
  __device__ __forceinline__ void block(int row0, int lane, int M, int col_first, int nch, float (*v)[16], float* sbuf, int slot) const {
    const float m = stage_store(row0, lane, M, col_first, nch, v, sbuf, kEpiScratchStride);
    pmax_store(row0 + lane, M, slot, m);
  }
};

// Accumulator layout in TMEM: accumulator a starts at column a * stride.
__host__ __device__ inline int acc_stride(int bn) { return (bn + 31) & ~31; }

// Partial products (plane of A, plane of B): the small cross terms first, the leading p0p0 last.
// The first argument is a product-set code: the plane count for bf16 planes, kF16PairCode for the f16 pair.
constexpr int kF16PairCode = 4;
// (one plane of an fp16 pair is a plain fp16 operand: one product)
__host__ __device__ constexpr int product_code(int nt, int fmt) { return (fmt && nt == 2) ? kF16PairCode : nt; }
__host__ __device__ constexpr int num_products(int nt) { return nt == 1 ? 1 : (nt == 2 ? 4 : (nt == kF16PairCode ? 3 : 6)); }
__host__ __device__ constexpr int prod_a(int nt, int p) {
  return nt == kF16PairCode ? (p == 0 ? 1 : 0)
                            : nt == 3 ? (p == 0 ? 2 : (p == 2 || p == 3) ? 1 : 0) : (nt == 2 ? (p < 2 ? 1 : 0) : 0);
}
__host__ __device__ constexpr int prod_b(int nt, int p) {
  return nt == kF16PairCode ? (p == 1 ? 1 : 0)
                            : nt == 3 ? (p == 1 ? 2 : (p == 2 || p == 4) ? 1 : 0) : (nt == 2 ? ((p == 0 || p == 2) ? 1 : 0) : 0);
}
static_assert(num_products(kF16PairCode) == 3 && prod_a(kF16PairCode, 0) == 1 && prod_b(kF16PairCode, 0) == 0 &&
              prod_a(kF16PairCode, 1) == 0 && prod_b(kF16PairCode, 1) == 1 && prod_a(kF16PairCode, 2) == 0 &&
              prod_b(kF16PairCode, 2) == 0, "f16 pair products: (1,0)(0,1)(0,0)");
static_assert(prod_a(3, 0) == 2 && prod_b(3, 0) == 0 && prod_a(3, 1) == 0 && prod_b(3, 1) == 2 && prod_a(3, 2) == 1 &&
              prod_b(3, 2) == 1 && prod_a(3, 3) == 1 && prod_b(3, 3) == 0 && prod_a(3, 4) == 0 && prod_b(3, 4) == 1 &&
              prod_a(3, 5) == 0 && prod_b(3, 5) == 0, "NT=3 products: (2,0)(0,2)(1,1)(1,0)(0,1)(0,0)");
static_assert(prod_a(2, 0) == 1 && prod_b(2, 0) == 1 && prod_a(2, 1) == 1 && prod_b(2, 1) == 0 && prod_a(2, 2) == 0 &&
              prod_b(2, 2) == 1 && prod_a(2, 3) == 0 && prod_b(2, 3) == 0, "NT=2 products: (1,1)(1,0)(0,1)(0,0)");

// Polite bounded wait for the warps that have nothing to do until the accumulator is ready:
// sleeping between polls leaves the issue slots to the TMA and MMA threads.
__device__ __forceinline__ bool mbar_wait_sleepy(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned ns = 256) {
  const unsigned long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    __nanosleep(ns);
    if (*abort_flag) return false;
    if ((unsigned long long)clock64() - t0 > kWaitCycles) { *abort_flag = 1; return false; }
  }
  return true;
}


// ---- kernel -------------------------------------------------------------------------------
template <int NT, int BKT, int FMT, class Epi>
__global__ void __launch_bounds__(kThreadsMain, 1)
gemm_tc_kernel(const __grid_constant__ TmapSet tm, int M, int N, int K, int BN, int STAGES, int kDrainEvery, Epi epi,
               int* __restrict__ err_flag, int splits, float* __restrict__ ws, int* __restrict__ tile_counters) {
  constexpr int PC = product_code(NT, FMT);
  constexpr int NP = num_products(PC);
  constexpr int A_BYTES = BM * BKT * 2;   // one plane of the A tile of a stage (shadows the 32-deep constant)
  constexpr int BK = BKT;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // stage tiles need 1024-byte alignment
  unsigned char* base_ptr = smem_raw + (base - raw);
  const int B_BYTES = BN * BK * 2;
  const int STAGE_BYTES = NT * (A_BYTES + B_BYTES);
  const int RING = ring_bytes(STAGES, STAGE_BYTES);
  const uint32_t bars = base + RING;  // full[STAGES], empty[STAGES], accum, main_full, main_free
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + RING + 8 * (2 * STAGES + 3));
  __shared__ int s_abort;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;  // M fastest: the CTAs sharing a weight tile run together
  // split-K: this CTA covers k-blocks [kb0, kb0 + nkb) of the K / BK blocks
  const int nkb_total = K / BK;
  const int kb0 = (int)((long long)nkb_total * blockIdx.z / splits);
  const int nkb = (int)((long long)nkb_total * (blockIdx.z + 1) / splits) - kb0;
  const uint32_t accum_bar = bars + 8u * (2 * STAGES);
  const uint32_t main_full = accum_bar + 8u, main_free = accum_bar + 16u;
  const int ndrain = (nkb + kDrainEvery - 1) / kDrainEvery;

  if (threadIdx.x == 0) {
    s_abort = 0;
    // with split operands two threads issue MMAs: a stage is free, and the tile complete, when both have committed
    for (int s = 0; s < STAGES; ++s) { mbar_init(bars + 8u * s, 1); mbar_init(bars + 8u * (STAGES + s), NP > 1 ? 2 : 1); }
    mbar_init(accum_bar, NP > 1 ? 2 : 1);
    mbar_init(main_full, 1);
    mbar_init(main_free, kEpiWarps);  // one arrival per epilogue warp
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    // Producer.  A TMA instruction costs its issuing thread ~150 ns whatever the box size
    // (measured), so the 2*NT boxes of a stage are issued by 2*NT lanes in one warp instruction:
    // lane t < NT loads plane t of A, lane NT + t plane t of B.
    const bool is_a = lane < NT;
    const int t = is_a ? lane : lane - NT;
    const CUtensorMap* map = reinterpret_cast<const CUtensorMap*>(&tm) + (is_a ? t : 3 + t);  // a[3] then b[3]
    const uint32_t dst_off = is_a ? (uint32_t)(t * A_BYTES) : (uint32_t)(NT * A_BYTES + t * B_BYTES);
    const int ycoord = is_a ? m0 : n0;
    // First trip round the ring: the weight tiles do not depend on the previous kernel, so they
    // are requested before pdl_wait() and only the activation tiles after it.
    const int npre = nkb < STAGES ? nkb : STAGES;
    for (int kb = 0; kb < npre; ++kb) {
      if (lane == 0) mbar_expect_tx(bars + 8u * kb, (uint32_t)STAGE_BYTES);
      __syncwarp();
      if (!is_a && lane < 2 * NT) tma_load_2d(base + kb * STAGE_BYTES + dst_off, map, (kb0 + kb) * BK, ycoord, bars + 8u * kb);
    }
    pdl_wait();   // the activations are the previous kernel's output
    if (is_a)
      for (int kb = 0; kb < npre; ++kb) tma_load_2d(base + kb * STAGE_BYTES + dst_off, map, (kb0 + kb) * BK, ycoord, bars + 8u * kb);
    int s = npre == STAGES ? 0 : npre; uint32_t ph = npre == STAGES ? 1u : 0u;
    uint32_t st = base + s * STAGE_BYTES, fb = bars + 8u * s, eb = bars + 8u * (STAGES + s);
    for (int kb = npre; kb < nkb; ++kb) {
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(eb, ph ^ 1u, &s_abort) ? 1 : 0;
        if (ok) mbar_expect_tx(fb, (uint32_t)STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < 2 * NT) tma_load_2d(st + dst_off, map, (kb0 + kb) * BK, ycoord, fb);
      st += STAGE_BYTES; fb += 8u; eb += 8u;
      if (++s == STAGES) { s = 0; ph ^= 1u; st = base; fb = bars; eb = bars + 8u * STAGES; }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, FMT);
      int s = 0; uint32_t ph = 0;
      uint32_t st = base, fb = bars, eb = bars + 8u * STAGES;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(fb, ph, &s_abort)) break;
        tc_fence_after();
        const uint64_t a0 = make_desc<BKT>(st);                        // plane 0 of A, k-step 0
        const uint64_t b0 = make_desc<BKT>(st + NT * A_BYTES);         // plane 0 of B, k-step 0
        if (NP == 1) {
          // plain bf16: one accumulation chain
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks)
            umma_bf16(tmem_acc, a0 + (uint64_t)(ks * 2), b0 + (uint64_t)(ks * 2), idesc, (kb | ks) ? 1u : 0u);
        } else {
          // (the small cross terms are the other issuing warp's)
          // leading product: accumulator 0 holds only kDrainEvery k-blocks at a time; the epilogue
          // warps add each partial sum into registers and hand the accumulator back
          const int in_chunk = kb % kDrainEvery;
          if (in_chunk == 0 && kb > 0) {
            const int d = kb / kDrainEvery;  // this chunk; the previous one must have been drained
            if (!mbar_wait(main_free, (uint32_t)((d - 1) & 1), &s_abort)) break;
            tc_fence_after();
          }
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks)
            umma_bf16(tmem_acc, a0 + (uint64_t)(ks * 2), b0 + (uint64_t)(ks * 2), idesc, (in_chunk | ks) ? 1u : 0u);
          if (in_chunk == kDrainEvery - 1 || kb == nkb - 1) umma_commit(main_full);
        }
        umma_commit(eb);
        st += STAGE_BYTES; fb += 8u; eb += 8u;
        if (++s == STAGES) { s = 0; ph ^= 1u; st = base; fb = bars; eb = bars + 8u * STAGES; }
      }
      umma_commit(accum_bar);
    }
  } else if (warp == kIssue2Warp) {
    if (NP > 1 && lane == 0) {
      // second issuer: the small cross terms, one long chain in accumulator 1
      const uint32_t idesc = make_idesc(BM, BN, FMT);
      const uint32_t acc1 = tmem_acc + (uint32_t)acc_stride(BN);
      const uint64_t bstep = (uint64_t)(B_BYTES >> 4);           // one B plane, in descriptor units (16 bytes)
      int s = 0; uint32_t ph = 0;
      uint32_t st = base, fb = bars, eb = bars + 8u * STAGES;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(fb, ph, &s_abort)) break;
        tc_fence_after();
        const uint64_t a0 = make_desc<BKT>(st);
        const uint64_t b0 = make_desc<BKT>(st + NT * A_BYTES);
#pragma unroll
        for (int ks = 0; ks < BK / UMMA_K; ++ks) {
#pragma unroll
          for (int p = 0; p < NP - 1; ++p) {
            const uint64_t ad = a0 + (uint64_t)(((prod_a(PC, p) * A_BYTES) >> 4) + ks * 2);
            const uint64_t bd = b0 + (uint64_t)prod_b(PC, p) * bstep + (uint64_t)(ks * 2);
            umma_bf16(acc1, ad, bd, idesc, (kb | ks | p) ? 1u : 0u);
          }
        }
        umma_commit(eb);
        st += STAGE_BYTES; fb += 8u; eb += 8u;
        if (++s == STAGES) { s = 0; ph ^= 1u; st = base; fb = bars; eb = bars + 8u * STAGES; }
      }
      umma_commit(accum_bar);
    }
  } else {
    // epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31; the four warps of a lane quadrant
    // own consecutive blocks of up to four 16-column chunks
    const int q = warp & 3;
    constexpr int kParts = kEpiWarps / 4;
    constexpr int kChunks = kEpiBlockChunks;
    static_assert(kParts * kChunks * 16 >= 256, "a quadrant's warps cover the widest tile");
    const int part = (warp - 2) >> 2;
    const int row0 = m0 + q * 32;
    const int row = row0 + lane;
    const int nchunks = BN >> 4;
    const int cpw = (nchunks + kParts - 1) / kParts;            // chunks per warp
    const int ch0 = part * cpw;                                  // this warp's first chunk
    int nmine = nchunks - ch0; nmine = nmine < 0 ? 0 : (nmine > cpw ? cpw : nmine);
    {
      // columns past N (the last tile of a row of tiles) are not this warp's business
      const int left = (N - (n0 + ch0 * 16) + 15) >> 4;
      if (left < nmine) nmine = left < 0 ? 0 : left;
    }
    const uint32_t astride = (uint32_t)acc_stride(BN);
    const uint32_t lane_base = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(ch0 * 16);
    float* sbuf = reinterpret_cast<float*>(base_ptr + (warp - 2) * kEpiScratchBytes);
    // with split-K the tile's partial sum goes to the workspace; the last CTA of the tile adds them up
    float* wrow = ws ? ws + ((size_t)blockIdx.z * ((size_t)gridDim.x * BM) + (size_t)row) * (size_t)N : nullptr;
    pdl_wait();   // before the first global access of these warps (the hardware wait is over long before)
    float macc[kChunks][16];
    auto finish = [&]() {
      if (splits == 1) {
        if (Epi::kHasBlock) {
          const int slot = (int)blockIdx.y * kParts + part;
          if (nmine > 0) epi.block(row0, lane, M, n0 + ch0 * 16, nmine, macc, sbuf, slot);
          else if constexpr (Epi::kHasPmax) epi.pmax_store(row, M, slot, -INFINITY);
        } else if (row < M) {
#pragma unroll
          for (int ci = 0; ci < kChunks; ++ci)
            if (ci < nmine) epi(row, n0 + (ch0 + ci) * 16, macc[ci]);
        }
      } else if (row < M) {
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci)
          if (ci < nmine) {
            float4* dst = reinterpret_cast<float4*>(wrow + n0 + (ch0 + ci) * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_float4(macc[ci][4 * i], macc[ci][4 * i + 1], macc[ci][4 * i + 2], macc[ci][4 * i + 3]);
          }
      }
    };
    if (NP == 1) {
      if (mbar_wait_sleepy(accum_bar, 0, &s_abort)) {
        tc_fence_after();
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci)
          if (ci < nmine) tmem_ld16(lane_base + (uint32_t)(ci * 16), macc[ci]);
        finish();
      }
    } else {
      // Two-level accumulation of the leading product: the tensor core rounds toward zero on
      // every accumulate (measured: a bias of -0.5 ulp per MMA, growing with K), so its chain is
      // kept to kDrainEvery k-blocks and the partial sums are added here in fp32 round-to-nearest.
#pragma unroll
      for (int ci = 0; ci < kChunks; ++ci)
#pragma unroll
        for (int i = 0; i < 16; ++i) macc[ci][i] = 0.f;
      bool ok = true;
      for (int d = 0; d < ndrain && ok; ++d) {
        ok = mbar_wait_sleepy(main_full, (uint32_t)(d & 1), &s_abort, d == 0 ? 256 : 64);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci) {
          if (ci < nmine) {
            float w[16];
            tmem_ld16(lane_base + (uint32_t)(ci * 16), w);
#pragma unroll
            for (int i = 0; i < 16; ++i) macc[ci][i] += w[i];
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(main_free);
      }
      if (ok && mbar_wait(accum_bar, 0, &s_abort)) {
        tc_fence_after();
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci) {
          if (ci < nmine) {
            float sm[16];
            tmem_ld16(lane_base + astride + (uint32_t)(ci * 16), sm);
#pragma unroll
            for (int i = 0; i < 16; ++i) macc[ci][i] += FMT ? sm[i] * kF16PairInvScale : sm[i];
          }
        }
        finish();
      }
    }
  }
  if (splits > 1) __threadfence();  // partial sums visible before this CTA takes its ticket
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_acc, TMEM_COLS);
  if (threadIdx.x == 0 && s_abort) atomicExch(err_flag, 1);
  if (splits > 1) {
    // The CTA that arrives last at this tile sums the partial tiles in split order (a fixed
    // order: results do not depend on which CTA that is) and runs the fused epilogue.
    __shared__ int s_last;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) {
      const int ticket = atomicAdd(&tile_counters[tile], 1);
      s_last = (ticket == splits - 1) ? 1 : 0;
      if (s_last) tile_counters[tile] = 0;  // ready for the next launch
      __threadfence();
    }
    __syncthreads();
    if (s_last && warp >= 2 && warp < kIssue2Warp) {
      // (row, 16-column chunk) items dealt to all epilogue threads: a tile with few valid rows (late decoder
      // steps) still spreads its chunks over every warp instead of walking them one after the other
      const int mrows = (M - m0) < BM ? (M - m0) : BM;
      const int ncols = (N - n0) < BN ? (N - n0) : BN;
      const int nch = (ncols + 15) >> 4;
      const size_t zstride = (size_t)gridDim.x * BM * (size_t)N;
      for (int it = (int)threadIdx.x - 64; it < mrows * nch; it += kEpiWarps * 32) {
        const int ch = it / mrows, r = it - ch * mrows;
        const int row = m0 + r, c0 = ch * 16;
        const float* p0 = ws + (size_t)row * (size_t)N + n0 + c0;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        for (int z = 0; z < splits; ++z) {
          const float4* src = reinterpret_cast<const float4*>(p0 + (size_t)z * zstride);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 t = __ldcg(src + i);
            v[4 * i] += t.x; v[4 * i + 1] += t.y; v[4 * i + 2] += t.z; v[4 * i + 3] += t.w;
          }
        }
        epi(row, n0 + c0, v);
      }
    }
  }
}

// ---- persistent variant for many-wave GEMMs whose leading product is one chain ----------------
// One CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (row tile fastest, so
// CTAs working at the same time share weight tiles in L2).  The TMA ring and the MMA issue run on
// across tile boundaries; the epilogue warps copy a finished accumulator pair to registers, hand
// TMEM back at once, and write their tile to memory while the tensor core is already on the next
// one -- the ~7 us of prologue and epilogue that every tile of a multi-wave launch used to pay is
// paid once per CTA.  Stores: the staging area of the one-tile kernel is the stage ring, which is busy
// here, so either the launch sets aside a small staging area of its own (stage_stride > 0: 32 rows x
// stage_stride floats per epilogue warp, two 16-column chunks at a time -- the one-plane launches, whose
// ring leaves the room), or tiles go out with row-per-lane stores and only a CTA's last tile, with the
// ring idle, is staged there.  No split-K, no intermediate drains.
template <int NT, int BKT, int FMT, class Epi>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_persist_kernel(const __grid_constant__ TmapSet tm, int M, int N, int K, int BN, int STAGES, Epi epi,
                       int* __restrict__ err_flag, int stage_stride) {
  constexpr int PC = product_code(NT, FMT);
  constexpr int NP = num_products(PC);
  constexpr int A_BYTES = BM * BKT * 2;
  constexpr int BK = BKT;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const int B_BYTES = BN * BK * 2;
  const int STAGE_BYTES = NT * (A_BYTES + B_BYTES);
  const int STG_WARP = 32 * stage_stride * 4;                    // bytes of a warp's own staging area (0: none)
  const int RING = (stage_stride > 0 ? STAGES * STAGE_BYTES : ring_bytes(STAGES, STAGE_BYTES));
  const int PRE = RING + kEpiWarps * STG_WARP;                   // ring, then the staging areas, then the barriers
  const uint32_t bars = base + PRE;   // full[STAGES], empty[STAGES], accum_full, tmem_free
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + PRE + 8 * (2 * STAGES + 3));
  __shared__ int s_abort;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = (M + BM - 1) / BM;
  const int ntile = mt * ((N + BN - 1) / BN);
  const int nkb = K / BK;
  const uint32_t accum_full = bars + 8u * (2 * STAGES);
  const uint32_t tmem_free = accum_full + 8u;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(bars + 8u * s, 1); mbar_init(bars + 8u * (STAGES + s), 1); }
    mbar_init(accum_full, 1);
    mbar_init(tmem_free, kEpiWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    const bool is_a = lane < NT;
    const int t = is_a ? lane : lane - NT;
    const CUtensorMap* map = reinterpret_cast<const CUtensorMap*>(&tm) + (is_a ? t : 3 + t);
    const uint32_t dst_off = is_a ? (uint32_t)(t * A_BYTES) : (uint32_t)(NT * A_BYTES + t * B_BYTES);
    int s = 0; uint32_t ph = 0;
    uint32_t st = base, fb = bars, eb = bars + 8u * STAGES;
    pdl_wait();
    bool live = true;
    for (int tile = blockIdx.x; tile < ntile && live; tile += gridDim.x) {
      const int ycoord = is_a ? (tile % mt) * BM : (tile / mt) * BN;
      for (int kb = 0; kb < nkb; ++kb) {
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(eb, ph ^ 1u, &s_abort) ? 1 : 0;
          if (ok) mbar_expect_tx(fb, (uint32_t)STAGE_BYTES);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { live = false; break; }
        if (lane < 2 * NT) tma_load_2d(st + dst_off, map, kb * BK, ycoord, fb);
        st += STAGE_BYTES; fb += 8u; eb += 8u;
        if (++s == STAGES) { s = 0; ph ^= 1u; st = base; fb = bars; eb = bars + 8u * STAGES; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, FMT);
      const uint32_t acc1 = tmem_acc + (uint32_t)acc_stride(BN);
      const uint64_t bstep = (uint64_t)(B_BYTES >> 4);
      int s = 0; uint32_t ph = 0;
      uint32_t st = base, fb = bars, eb = bars + 8u * STAGES;
      bool live = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < ntile && live; tile += gridDim.x, ++it) {
        // the epilogue warps have copied the previous tile's accumulators out
        if (it > 0) {
          if (!mbar_wait(tmem_free, (uint32_t)((it - 1) & 1), &s_abort)) break;
          tc_fence_after();
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(fb, ph, &s_abort)) { live = false; break; }
          tc_fence_after();
          const uint64_t a0 = make_desc<BKT>(st);
          const uint64_t b0 = make_desc<BKT>(st + NT * A_BYTES);
          if (NP > 1) {
#pragma unroll
            for (int ks = 0; ks < BK / UMMA_K; ++ks) {
#pragma unroll
              for (int p = 0; p < NP - 1; ++p) {
                const uint64_t ad = a0 + (uint64_t)(((prod_a(PC, p) * A_BYTES) >> 4) + ks * 2);
                const uint64_t bd = b0 + (uint64_t)prod_b(PC, p) * bstep + (uint64_t)(ks * 2);
                umma_bf16(acc1, ad, bd, idesc, (kb | ks | p) ? 1u : 0u);
              }
            }
          }
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks)
            umma_bf16(tmem_acc, a0 + (uint64_t)(ks * 2), b0 + (uint64_t)(ks * 2), idesc, (kb | ks) ? 1u : 0u);
          umma_commit(eb);
          st += STAGE_BYTES; fb += 8u; eb += 8u;
          if (++s == STAGES) { s = 0; ph ^= 1u; st = base; fb = bars; eb = bars + 8u * STAGES; }
        }
        umma_commit(accum_full);
      }
    }
  } else {
    const int q = warp & 3;
    constexpr int kParts = kEpiWarps / 4;
    constexpr int kChunks = kEpiBlockChunks;
    const int part = (warp - 2) >> 2;
    const int nchunks = BN >> 4;
    const int cpw = (nchunks + kParts - 1) / kParts;
    const int ch0 = part * cpw;
    const uint32_t astride = (uint32_t)acc_stride(BN);
    const uint32_t lane_base = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(ch0 * 16);
    float* sbuf = reinterpret_cast<float*>(base_ptr + (warp - 2) * kEpiScratchBytes);
    pdl_wait();
    int it = 0;
    for (int tile = blockIdx.x; tile < ntile; tile += gridDim.x, ++it) {
      const int m0 = (tile % mt) * BM, n0 = (tile / mt) * BN;
      const int row0 = m0 + q * 32;
      int nmine = nchunks - ch0; nmine = nmine < 0 ? 0 : (nmine > cpw ? cpw : nmine);
      {
        const int left = (N - (n0 + ch0 * 16) + 15) >> 4;
        if (left < nmine) nmine = left < 0 ? 0 : left;
      }
      if (!mbar_wait_sleepy(accum_full, (uint32_t)(it & 1), &s_abort)) break;
      tc_fence_after();
      float macc[kChunks][16];
#pragma unroll
      for (int ci = 0; ci < kChunks; ++ci) {
        if (ci < nmine) {
          tmem_ld16(lane_base + (uint32_t)(ci * 16), macc[ci]);
          if (NP > 1) {
            float sm[16];
            tmem_ld16(lane_base + astride + (uint32_t)(ci * 16), sm);
#pragma unroll
            for (int i = 0; i < 16; ++i) macc[ci][i] += FMT ? sm[i] * kF16PairInvScale : sm[i];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_free);   // the tensor core may start the next tile
      const bool last = tile + (int)gridDim.x >= ntile;
      const int slot = (tile / mt) * kParts + part;
      if constexpr (Epi::kHasPmax) {
        if (stage_stride > 0) {
          // this warp's own staging area: as many chunks at a time as a staged row holds
          float* own = reinterpret_cast<float*>(base_ptr + RING + (warp - 2) * STG_WARP);
          float m = -INFINITY;
#pragma unroll
          for (int c0 = 0; c0 < kChunks; c0 += 2) {   // two chunks at a time (stage_stride >= 36); static indices keep macc in registers
            if (c0 < nmine) {
              const int nc = nmine - c0 < 2 ? nmine - c0 : 2;
              m = fmaxf(m, epi.stage_store(row0, lane, M, n0 + (ch0 + c0) * 16, nc, macc + c0, own, stage_stride));
            }
          }
          epi.pmax_store(row0 + lane, M, slot, m);
          continue;
        }
      }
      if (last && Epi::kHasBlock) {
        // the ring is idle from here on: stage and store coalesced
        if (nmine > 0) epi.block(row0, lane, M, n0 + ch0 * 16, nmine, macc, sbuf, slot);
        else if constexpr (Epi::kHasPmax) epi.pmax_store(row0 + lane, M, slot, -INFINITY);
      } else if constexpr (Epi::kHasPmax) {
        epi.direct_block(row0 + lane, M, n0 + ch0 * 16, nmine, macc, slot);
      } else if (row0 + lane < M) {
#pragma unroll
        for (int ci = 0; ci < kChunks; ++ci)
          if (ci < nmine) epi(row0 + lane, n0 + (ch0 + ci) * 16, macc[ci]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_acc, TMEM_COLS);
  if (threadIdx.x == 0 && s_abort) atomicExch(err_flag, 1);
}

// ---- fp32 -> bf16 planes ---------------------------------------------------------------------
static __global__ void split_planes_kernel(const float* __restrict__ src, Planes dst, int nt, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    split_store(dst, nt, i, src[i]);
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a K-major bf16 matrix [rows][ld] (K columns used), box = BK x box_rows,
// 64-byte swizzle.  Rows past `rows` and columns past `K` read as zero.
inline bool make_tmap(CUtensorMap* map, const __nv_bfloat16* ptr, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows,
                      int bk = BK) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)bk, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A kernel's opt-in to more than 48 KB of dynamic shared memory is an attribute of the kernel ON ONE DEVICE:
// it is set once per (kernel, device), for the device that is current at the launch.
constexpr int kMaxDevices = 64;
template <class Kernel>
inline cudaError_t ensure_smem_optin(Kernel* kernel, bool* done_per_device, int bytes = SMEM_BUDGET + 1280) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!done_per_device[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done_per_device[dev] = true;
  }
  return cudaSuccess;
}

template <int NT, int BKT, int FMT, class Epi>
inline cudaError_t launch_gemm_tc_nt(const TmapSet& tm, int M, int N, int K, const Shape& sh, const Epi& epi, int* err_flag,
                                     cudaStream_t st, float* ws, int* counters) {
  static bool optin_done[kMaxDevices] = {};
  if (cudaError_t e = ensure_smem_optin(gemm_tc_kernel<NT, BKT, FMT, Epi>, optin_done); e != cudaSuccess) return e;
  const int splits = (sh.splits > 1 && ws && counters) ? sh.splits : 1;
  dim3 grid((M + BM - 1) / BM, (N + sh.bn - 1) / sh.bn, splits);
  int drain = (sh.drain > 0 ? sh.drain : kDrainDefault) * 32 / BKT;
  if (drain < 1) drain = 1;
  return launch_k(sh.pdl != 0, gemm_tc_kernel<NT, BKT, FMT, Epi>, grid, dim3(kThreadsMain), (size_t)sh.smem_bytes, st, tm, M, N, K, sh.bn,
                  sh.stages, drain, epi, err_flag, splits, splits > 1 ? ws : (float*)nullptr, counters);
}
template <class Epi>
inline cudaError_t launch_gemm_tc(const TmapSet& tm, int M, int N, int K, const Shape& sh, const Epi& epi, int* err_flag,
                                  cudaStream_t st, float* ws = nullptr, int* counters = nullptr) {
  if (sh.fmt == 1) {
    if (sh.nt == 1) {
      if (sh.bk == 64) return launch_gemm_tc_nt<1, 64, 1, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
      return launch_gemm_tc_nt<1, 32, 1, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
    }
    if (sh.nt != 2) return cudaErrorInvalidValue;
    if (sh.bk == 64) return launch_gemm_tc_nt<2, 64, 1, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
    return launch_gemm_tc_nt<2, 32, 1, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
  }
  if (sh.bk == 64) {
    if (sh.nt == 2) return launch_gemm_tc_nt<2, 64, 0, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
    if (sh.nt == 1) return launch_gemm_tc_nt<1, 64, 0, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
    return cudaErrorInvalidValue;  // three planes of 128-byte rows leave room for one stage only
  }
  if (sh.nt == 3) return launch_gemm_tc_nt<3, 32, 0, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
  if (sh.nt == 2) return launch_gemm_tc_nt<2, 32, 0, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
  return launch_gemm_tc_nt<1, 32, 0, Epi>(tm, M, N, K, sh, epi, err_flag, st, ws, counters);
}

// Persistent launch (see gemm_tc_persist_kernel): one or two planes per operand, no split-K.  One-plane
// launches get a staging area of their own beside a ring of one stage less.
constexpr int kPersistStageStride = 36;   // floats per staged row: two 16-column chunks + 4
inline Shape make_shape_persist(int bn, int nt, int bk, int fmt) {
  Shape s = make_shape(bn, nt, bk, fmt);
  if (nt == 1) {
    const int stg = kEpiWarps * 32 * kPersistStageStride * 4;
    s.stages = (SMEM_BUDGET - stg) / s.stage_bytes;
    if (s.stages > kMaxStages) s.stages = kMaxStages;
    s.smem_bytes = s.stages * s.stage_bytes + stg + 1024 + 256;
  }
  return s;
}
template <class Epi>
inline cudaError_t launch_gemm_tc_persist(const TmapSet& tm, int M, int N, int K, const Shape& sh, const Epi& epi, int* err_flag,
                                          cudaStream_t st, int n_sm) {
  if ((sh.nt != 2 && sh.nt != 1) || K % sh.bk || sh.stages < 2) return cudaErrorInvalidValue;
  const int tiles = ((M + BM - 1) / BM) * ((N + sh.bn - 1) / sh.bn);
  const dim3 grid(tiles < n_sm ? tiles : n_sm);
  const int stride = sh.nt == 1 ? kPersistStageStride : 0;
#define LINMT_PERSIST_CASE(NTV, BKV, FMTV)                                                                                   \
  {                                                                                                                          \
    static bool optin_done[kMaxDevices] = {};                                                                                \
    if (cudaError_t e = ensure_smem_optin(gemm_tc_persist_kernel<NTV, BKV, FMTV, Epi>, optin_done); e != cudaSuccess) return e; \
    return launch_k(sh.pdl != 0, gemm_tc_persist_kernel<NTV, BKV, FMTV, Epi>, grid, dim3(kThreads), (size_t)sh.smem_bytes, st, tm, M, N, K, \
                    sh.bn, sh.stages, epi, err_flag, stride);                                                                \
  }
  if (sh.nt == 1) {
    if (sh.fmt == 1 && sh.bk == 64) LINMT_PERSIST_CASE(1, 64, 1)
    if (sh.fmt == 1) LINMT_PERSIST_CASE(1, 32, 1)
    if (sh.bk == 64) LINMT_PERSIST_CASE(1, 64, 0)
    LINMT_PERSIST_CASE(1, 32, 0)
  }
  if (sh.fmt == 1 && sh.bk == 64) LINMT_PERSIST_CASE(2, 64, 1)
  if (sh.fmt == 1) LINMT_PERSIST_CASE(2, 32, 1)
  if (sh.bk == 64) LINMT_PERSIST_CASE(2, 64, 0)
  LINMT_PERSIST_CASE(2, 32, 0)
#undef LINMT_PERSIST_CASE
}

// Tile width that fills the SMs best for an M x N problem: the smallest makespan
// ceil(tiles / SMs) * BN over the allowed widths (multiples of 16 whose tile is a whole
// number of 1024-byte swizzle atoms, i.e. multiples of 16 rows of 64 bytes).
inline int pick_bn(int M, int N, int n_sm) {
  const int mt = (M + BM - 1) / BM;
  int best = 256;
  double best_cost = 1e30;
  for (int bn = 256; bn >= 48; bn -= 16) {
    const long tiles = (long)mt * ((N + bn - 1) / bn);
    const long waves = (tiles + n_sm - 1) / n_sm;
    // cost: tensor time ~ waves * bn, plus a fixed per-tile overhead (prologue, epilogue)
    const double cost = (double)waves * (bn + 24);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
  }
  return best;
}

// Tile width AND split-K factor from a small cost model (times in ns per k-block, measured):
// a k-block costs the larger of the issuing thread's time (~58 ns per MMA, whatever its width)
// and the tensor pipe's (128 x bn x 16 MACs at 4096 MAC/clk); a launch takes
// waves * (k-blocks-per-CTA of those + ~8-13 us of prologue/epilogue per tile), plus the cost of
// writing and re-reading partial tiles when K is split (only worth it for tiles up to 176 wide).
// ws_floats bounds the split-K workspace (splits * padded rows * N floats).
// The f16 pair with 64-deep stages, measured (two issuing threads): a k-block costs ~490 ns while the
// issuing threads are the limit (tiles up to ~100 wide) and 120 + 3.6 * bn ns beyond (the tensor pipe at
// its practical rate); per tile ~6 us + 12 ns per column of prologue and epilogue; a split adds ~2 us plus
// 0.28 ns per partial-tile element that is written and read back (valid rows only).
inline void pick_shape_f16(int M, int N, int K, int n_sm, size_t ws_floats, int max_tiles, int* bn_out, int* splits_out) {
  const int mt = (M + BM - 1) / BM;
  const int nkb = K / 64;
  const double rows_per_tile = (double)M / mt;
  double best = 1e30;
  int best_bn = 256, best_s = 1;
  for (int bn = 256; bn >= 64; bn -= 16) {
    const long tiles = (long)mt * ((N + bn - 1) / bn);
    const double wide = 120.0 + 3.6 * bn;
    const double per_kb = wide > 490.0 ? wide : 490.0;
    for (int s = 1; s <= 6; ++s) {
      if (s > 1 && (bn > 208 || nkb / s < 2 || tiles > max_tiles || (size_t)s * mt * BM * (size_t)N > ws_floats)) break;
      const long waves = (tiles * s + n_sm - 1) / n_sm;
      const double kb_per_cta = (double)((nkb + s - 1) / s);
      const double cost = waves * (kb_per_cta * per_kb + 6000.0 + bn * 12.0) + (s > 1 ? 2000.0 + 0.28 * s * rows_per_tile * bn : 0.0);
      if (cost < best - 1e-9) { best = cost; best_bn = bn; best_s = s; }
    }
  }
  *bn_out = best_bn;
  *splits_out = best_s;
}

inline void pick_shape(int M, int N, int K, int nt, int n_sm, size_t ws_floats, int max_tiles, int* bn_out, int* splits_out, int fmt = 0) {
  if (fmt == 1 && nt == 2 && K % 64 == 0) { pick_shape_f16(M, N, K, n_sm, ws_floats, max_tiles, bn_out, splits_out); return; }
  const int mt = (M + BM - 1) / BM;
  const int nkb = K / BK;
  const int np = num_products(product_code(nt, fmt));
  double best = 1e30;
  int best_bn = 256, best_s = 1;
  for (int bn = 256; bn >= 48; bn -= 16) {
    const long tiles = (long)mt * ((N + bn - 1) / bn);
    const double per_kb = 2.0 * np * (58.0 > bn * 0.254 ? 58.0 : bn * 0.254);
    for (int s = 1; s <= 8; ++s) {
      if (s > 1 && (bn > 176 || nkb / s < 4 || tiles > max_tiles || (size_t)s * mt * BM * (size_t)N > ws_floats)) break;
      const long waves = (tiles * s + n_sm - 1) / n_sm;
      const double kb_per_cta = (double)((nkb + s - 1) / s);
      // per tile: prologue, pipeline fill and epilogue (~8 us + 20 ns per column); per split: the partial-tile traffic
      const double cost = waves * (kb_per_cta * per_kb + 8000.0 + bn * 20.0) + (s > 1 ? 4000.0 + 2000.0 * s + bn * 10.0 * (s + 1) : 0.0);
      if (cost < best - 1e-9) { best = cost; best_bn = bn; best_s = s; }
    }
  }
  *bn_out = best_bn;
  *splits_out = best_s;
}

}  // namespace tc
}  // namespace linmt

// gemm_tc_pair.cuh -- the one-tile GEMM of gemm_tc.cuh on CTA PAIRS (tcgen05 cta_group::2).
//
// The one-tile kernel is bound by what an SM can pull out of L2: every CTA loads its own 128-row slice of the
// activations AND the whole BN-row slice of the weights for each k-block.  Two CTAs that sit on neighbouring row
// tiles of the same column tile need the same weights.  Launched as a cluster of two along M they form one
// 256 x BN tile: each CTA loads its 128 rows of A and only HALF of the weight rows, and the tensor cores of both
// SMs read the two halves out of both shared memories (tcgen05.mma.cta_group::2, issued by the even CTA for
// the pair).  Per CTA and k-block that is A + B/2 instead of A + B, which also makes the stages smaller (more of
// them in flight).  Every CTA still owns the accumulator rows of its own 128 rows in its own TMEM, so the
// epilogues, split-K and everything after the accumulator are the one-tile kernel's, and so are the result bits
// (the same products accumulate in the same order).  Measured on the decoder's gate product at 768 rows
// (K = 2048, N = 4096, 176-wide tiles, weights from HBM): 35.8 us against 41.2 us per layer; the one-tile
// kernel has room for two 76 KB stages there, the pair for four of 54 KB.  Narrower shapes (three or more stages
// already, bound by the issuing threads) gain nothing, so the host uses pairs only where the one-tile shape is
// down to two stages.
//
// Protocol (the even CTA of a pair = "leader"):
//   * the full barriers that count are the leader's: both CTAs' TMA loads complete their bytes there
//     (cp.async.bulk.tensor ... .cta_group::2, no multicast), the leader's producer posts the expected bytes of both;
//   * stage-free, chunk-ready and tile-complete signals are tcgen05.commit.cta_group::2 with a two-CTA mask, so each
//     CTA waits on barriers of its own;
//   * the peer's epilogue warps hand the leading accumulator back by arriving on the leader's barrier remotely;
//   * cluster barriers after the barrier set-up and before TMEM is freed keep either CTA from touching the other
//     too early or leaving too soon.  Every other wait is bounded as in the one-tile kernel.
#pragma once
#include "gemm_tc.cuh"

namespace linmt {
namespace tc {

__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a CTA pair: data into this CTA's shared memory, bytes counted on the barrier at cluster address `bar`
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive (once the MMAs issued so far are complete) on the barrier at this shared-memory offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// Shape of a pair launch: per CTA a stage holds A (BM rows) and HALF of B (bn / 2 rows) per plane.
inline Shape make_shape_pair(int bn, int nt, int bk, int fmt) {
  Shape s = make_shape(bn, nt, bk, fmt);
  s.stage_bytes = nt * (BM * bk * 2 + (bn / 2) * bk * 2);
  s.stages = SMEM_BUDGET / s.stage_bytes;
  if (s.stages > kMaxStages) s.stages = kMaxStages;
  s.smem_bytes = shape_smem_bytes(s.stages, s.stage_bytes);
  return s;
}

template <int NT, int BKT, int FMT, class Epi>
__global__ void __launch_bounds__(kThreadsMain, 1)
gemm_tc_pair_kernel(const __grid_constant__ TmapSet tm, int M, int N, int K, int BN, int STAGES, int kDrainEvery, Epi epi,
                    int* __restrict__ err_flag, int splits, float* __restrict__ ws, int* __restrict__ tile_counters) {
  constexpr int PC = product_code(NT, FMT);
  constexpr int NP = num_products(PC);
  static_assert(NP > 1, "the pair kernel is written for split operands (two issuing warps, two accumulators)");
  constexpr int A_BYTES = BM * BKT * 2;
  constexpr int BK = BKT;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const int BH = BN >> 1;                      // weight rows this CTA loads
  const int B_BYTES = BH * BK * 2;
  const int STAGE_BYTES = NT * (A_BYTES + B_BYTES);
  const int RING = ring_bytes(STAGES, STAGE_BYTES);
  const uint32_t bars = base + RING;  // full[STAGES], empty[STAGES], accum, main_full, main_free
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + RING + 8 * (2 * STAGES + 3));
  __shared__ int s_abort;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();     // 0 = leader (even blockIdx.x), 1 = peer
  const bool leader = rank == 0;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int nkb_total = K / BK;
  const int kb0 = (int)((long long)nkb_total * blockIdx.z / splits);
  const int nkb = (int)((long long)nkb_total * (blockIdx.z + 1) / splits) - kb0;
  const uint32_t accum_bar = bars + 8u * (2 * STAGES);
  const uint32_t main_full = accum_bar + 8u, main_free = accum_bar + 16u;
  const int ndrain = (nkb + kDrainEvery - 1) / kDrainEvery;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(bars + 8u * s, 1); mbar_init(bars + 8u * (STAGES + s), 2); }
    mbar_init(accum_bar, 2);
    mbar_init(main_full, 1);
    mbar_init(main_free, 2 * kEpiWarps);   // the epilogue warps of both CTAs (only the leader's copy is waited on)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();      // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    // Producer (both CTAs): lanes 0..NT-1 the planes of this CTA's A rows, lanes NT..2NT-1 the planes of its half of B.
    const bool is_a = lane < NT;
    const int t = is_a ? lane : lane - NT;
    const CUtensorMap* map = reinterpret_cast<const CUtensorMap*>(&tm) + (is_a ? (t < 3 ? t : 0) : 3 + (t < 3 ? t : 0));
    const uint32_t dst_off = is_a ? (uint32_t)(t * A_BYTES) : (uint32_t)(NT * A_BYTES + t * B_BYTES);
    const int ycoord = is_a ? m0 : n0 + (int)rank * BH;
    const uint32_t full0 = cluster_map(bars, 0u);           // the leader's full barriers, as cluster addresses
    const uint32_t tx_bytes = 2u * (uint32_t)STAGE_BYTES;   // both CTAs' boxes
    const int npre = nkb < STAGES ? nkb : STAGES;
    for (int kb = 0; kb < npre; ++kb) {
      if (lane == 0 && leader) mbar_expect_tx(bars + 8u * kb, tx_bytes);
      __syncwarp();
      if (!is_a && lane < 2 * NT) tma_load_2d_pair(base + kb * STAGE_BYTES + dst_off, map, (kb0 + kb) * BK, ycoord, full0 + 8u * kb);
    }
    pdl_wait();
    if (is_a)
      for (int kb = 0; kb < npre; ++kb) tma_load_2d_pair(base + kb * STAGE_BYTES + dst_off, map, (kb0 + kb) * BK, ycoord, full0 + 8u * kb);
    int s = npre == STAGES ? 0 : npre; uint32_t ph = npre == STAGES ? 1u : 0u;
    for (int kb = npre; kb < nkb; ++kb) {
      const uint32_t st = base + s * STAGE_BYTES, eb = bars + 8u * (STAGES + s);
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(eb, ph ^ 1u, &s_abort) ? 1 : 0;       // this CTA's copy of the stage-free barrier
        if (ok && leader) mbar_expect_tx(bars + 8u * s, tx_bytes);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < 2 * NT) tma_load_2d_pair(st + dst_off, map, (kb0 + kb) * BK, ycoord, full0 + 8u * s);
      if (++s == STAGES) { s = 0; ph ^= 1u; }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // leading product of the pair's 256 x BN tile into accumulator 0 (of both CTAs)
      const uint32_t idesc = make_idesc(2 * BM, BN, FMT);
      int s = 0; uint32_t ph = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        const uint32_t st = base + s * STAGE_BYTES, fb = bars + 8u * s, eb = bars + 8u * (STAGES + s);
        if (!mbar_wait(fb, ph, &s_abort)) break;
        tc_fence_after();
        const uint64_t a0 = make_desc<BKT>(st);
        const uint64_t b0 = make_desc<BKT>(st + NT * A_BYTES);
        const int in_chunk = kb % kDrainEvery;
        if (in_chunk == 0 && kb > 0) {
          const int d = kb / kDrainEvery;
          if (!mbar_wait(main_free, (uint32_t)((d - 1) & 1), &s_abort)) break;
          tc_fence_after();
        }
#pragma unroll
        for (int ks = 0; ks < BK / UMMA_K; ++ks)
          umma_f16_pair(tmem_acc, a0 + (uint64_t)(ks * 2), b0 + (uint64_t)(ks * 2), idesc, (in_chunk | ks) ? 1u : 0u);
        if (in_chunk == kDrainEvery - 1 || kb == nkb - 1) umma_commit_pair(main_full);
        umma_commit_pair(eb);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      umma_commit_pair(accum_bar);
    }
  } else if (warp == kIssue2Warp) {
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc(2 * BM, BN, FMT);
      const uint32_t acc1 = tmem_acc + (uint32_t)acc_stride(BN);
      const uint64_t bstep = (uint64_t)(B_BYTES >> 4);
      int s = 0; uint32_t ph = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        const uint32_t st = base + s * STAGE_BYTES, fb = bars + 8u * s, eb = bars + 8u * (STAGES + s);
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
            umma_f16_pair(acc1, ad, bd, idesc, (kb | ks | p) ? 1u : 0u);
          }
        }
        umma_commit_pair(eb);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
      umma_commit_pair(accum_bar);
    }
  } else {
    // epilogue (both CTAs, each on the rows of its own TMEM): the one-tile kernel's
    const int q = warp & 3;
    constexpr int kParts = kEpiWarps / 4;
    constexpr int kChunks = kEpiBlockChunks;
    const int part = (warp - 2) >> 2;
    const int row0 = m0 + q * 32;
    const int row = row0 + lane;
    const int nchunks = BN >> 4;
    const int cpw = (nchunks + kParts - 1) / kParts;
    const int ch0 = part * cpw;
    int nmine = nchunks - ch0; nmine = nmine < 0 ? 0 : (nmine > cpw ? cpw : nmine);
    {
      const int left = (N - (n0 + ch0 * 16) + 15) >> 4;
      if (left < nmine) nmine = left < 0 ? 0 : left;
    }
    const uint32_t astride = (uint32_t)acc_stride(BN);
    const uint32_t lane_base = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(ch0 * 16);
    float* sbuf = reinterpret_cast<float*>(base_ptr + (warp - 2) * kEpiScratchBytes);
    float* wrow = ws ? ws + ((size_t)blockIdx.z * ((size_t)gridDim.x * BM) + (size_t)row) * (size_t)N : nullptr;
    const uint32_t main_free_leader = cluster_map(main_free, 0u);
    pdl_wait();
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
      if (lane == 0) mbar_arrive_cluster(main_free_leader);   // the leader's issuing thread waits for both CTAs' warps
    }
    // The ring doubles as the epilogue's staging area, and the LEADER's tensor core reads this CTA's ring: it is
    // idle only once the tile-complete barrier (committed after the last MMA of the pair) has been passed.
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
  if (splits > 1) __threadfence();
  tc_fence_before();
  cluster_sync_all();      // the pair is done with both TMEMs and both rings (every wait above is bounded)
  if (warp == 1) tmem_dealloc_pair(tmem_acc, TMEM_COLS);
  if (threadIdx.x == 0 && s_abort) atomicExch(err_flag, 1);
  if (splits > 1) {
    __shared__ int s_last;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) {
      const int ticket = atomicAdd(&tile_counters[tile], 1);
      s_last = (ticket == splits - 1) ? 1 : 0;
      if (s_last) tile_counters[tile] = 0;
      __threadfence();
    }
    __syncthreads();
    if (s_last && warp >= 2 && warp < kIssue2Warp) {
      const int mrows = (M - m0) < BM ? (M - m0) : BM;
      const int ncols = (N - n0) < BN ? (N - n0) : BN;
      const int nch = (ncols + 15) >> 4;
      const size_t zstride = (size_t)gridDim.x * BM * (size_t)N;
      for (int it = (int)threadIdx.x - 64; it < mrows * nch; it += kEpiWarps * 32) {
        const int ch = it / mrows, r = it - ch * mrows;
        const int rr = m0 + r, c0 = ch * 16;
        const float* p0 = ws + (size_t)rr * (size_t)N + n0 + c0;
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
        for (int z = 0; z < splits; ++z) {
          const float4* src = reinterpret_cast<const float4*>(p0 + (size_t)z * zstride);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 tq = __ldcg(src + i);
            v[4 * i] += tq.x; v[4 * i + 1] += tq.y; v[4 * i + 2] += tq.z; v[4 * i + 3] += tq.w;
          }
        }
        epi(rr, n0 + c0, v);
      }
    }
  }
}

// Launch on CTA pairs: grid.x = row tiles rounded up to even, cluster (2, 1, 1).  The B tensor maps must have been
// made with a box of bn / 2 rows.
template <int NT, int BKT, int FMT, class Epi>
inline cudaError_t launch_gemm_tc_pair(const TmapSet& tm, int M, int N, int K, const Shape& sh, const Epi& epi, int* err_flag,
                                       cudaStream_t st, float* ws, int* counters) {
  static bool optin_done[kMaxDevices] = {};
  if (cudaError_t e = ensure_smem_optin(gemm_tc_pair_kernel<NT, BKT, FMT, Epi>, optin_done); e != cudaSuccess) return e;
  if (sh.bn % 16) return cudaErrorInvalidValue;
  const int splits = (sh.splits > 1 && ws && counters) ? sh.splits : 1;
  const int mt = (M + BM - 1) / BM;
  dim3 grid((mt + 1) & ~1, (N + sh.bn - 1) / sh.bn, splits);
  int drain = (sh.drain > 0 ? sh.drain : kDrainDefault) * 32 / BKT;
  if (drain < 1) drain = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = dim3(kThreadsMain); cfg.dynamicSmemBytes = (size_t)sh.smem_bytes; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = sh.pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<NT, BKT, FMT, Epi>, tm, M, N, K, sh.bn, sh.stages, drain, epi, err_flag, splits,
                            splits > 1 ? ws : (float*)nullptr, counters);
}

// ---- persistent form on CTA pairs (many-wave GEMMs: the vocabulary projection) ---------------------------
// gemm_tc_persist_kernel with every SM pair walking over 256 x BN tiles: pair p takes pair tiles p, p + pairs, ...
// (row pair fastest); CTA `rank` of the pair owns row tile 2 * (row pair) + rank of each.  Loads, barriers and
// TMEM hand-over as in gemm_tc_pair_kernel; the tensor core may start the next tile once the epilogue warps of
// BOTH CTAs have copied their accumulator rows out (they arrive on the leader's barrier).
inline Shape make_shape_persist_pair(int bn, int nt, int bk, int fmt) {
  Shape s = make_shape_pair(bn, nt, bk, fmt);
  if (nt == 1) {
    const int stg = kEpiWarps * 32 * kPersistStageStride * 4;
    s.stages = (SMEM_BUDGET - stg) / s.stage_bytes;
    if (s.stages > kMaxStages) s.stages = kMaxStages;
    s.smem_bytes = s.stages * s.stage_bytes + stg + 1024 + 256;
  }
  return s;
}

template <int NT, int BKT, int FMT, class Epi>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_persist_pair_kernel(const __grid_constant__ TmapSet tm, int M, int N, int K, int BN, int STAGES, Epi epi,
                            int* __restrict__ err_flag, int stage_stride) {
  constexpr int PC = product_code(NT, FMT);
  constexpr int NP = num_products(PC);
  constexpr int A_BYTES = BM * BKT * 2;
  constexpr int BK = BKT;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - raw);
  const int BH = BN >> 1;
  const int B_BYTES = BH * BK * 2;
  const int STAGE_BYTES = NT * (A_BYTES + B_BYTES);
  const int STG_WARP = 32 * stage_stride * 4;
  const int RING = (stage_stride > 0 ? STAGES * STAGE_BYTES : ring_bytes(STAGES, STAGE_BYTES));
  const int PRE = RING + kEpiWarps * STG_WARP;
  const uint32_t bars = base + PRE;   // full[STAGES], empty[STAGES], accum_full, tmem_free
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + PRE + 8 * (2 * STAGES + 3));
  __shared__ int s_abort;

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int mt = (M + BM - 1) / BM;
  const int mt2 = (mt + 1) >> 1;                       // row pairs
  const int ntile = mt2 * ((N + BN - 1) / BN);        // pair tiles
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int nkb = K / BK;
  const uint32_t accum_full = bars + 8u * (2 * STAGES);
  const uint32_t tmem_free = accum_full + 8u;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(bars + 8u * s, 1); mbar_init(bars + 8u * (STAGES + s), 1); }
    mbar_init(accum_full, 1);
    mbar_init(tmem_free, 2 * kEpiWarps);   // both CTAs' epilogue warps (the leader's copy is the one waited on)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    const bool is_a = lane < NT;
    const int t = is_a ? lane : lane - NT;
    const CUtensorMap* map = reinterpret_cast<const CUtensorMap*>(&tm) + (is_a ? (t < 3 ? t : 0) : 3 + (t < 3 ? t : 0));
    const uint32_t dst_off = is_a ? (uint32_t)(t * A_BYTES) : (uint32_t)(NT * A_BYTES + t * B_BYTES);
    const uint32_t full0 = cluster_map(bars, 0u);
    const uint32_t tx_bytes = 2u * (uint32_t)STAGE_BYTES;
    int s = 0; uint32_t ph = 0;
    pdl_wait();
    bool live = true;
    for (int tile = pair; tile < ntile && live; tile += npairs) {
      const int ycoord = is_a ? ((tile % mt2) * 2 + (int)rank) * BM : (tile / mt2) * BN + (int)rank * BH;
      for (int kb = 0; kb < nkb; ++kb) {
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(bars + 8u * (STAGES + s), ph ^ 1u, &s_abort) ? 1 : 0;
          if (ok && leader) mbar_expect_tx(bars + 8u * s, tx_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { live = false; break; }
        if (lane < 2 * NT) tma_load_2d_pair(base + s * STAGE_BYTES + dst_off, map, kb * BK, ycoord, full0 + 8u * s);
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc(2 * BM, BN, FMT);
      const uint32_t acc1 = tmem_acc + (uint32_t)acc_stride(BN);
      const uint64_t bstep = (uint64_t)(B_BYTES >> 4);
      int s = 0; uint32_t ph = 0;
      bool live = true;
      int it = 0;
      for (int tile = pair; tile < ntile && live; tile += npairs, ++it) {
        if (it > 0) {
          if (!mbar_wait(tmem_free, (uint32_t)((it - 1) & 1), &s_abort)) break;
          tc_fence_after();
        }
        for (int kb = 0; kb < nkb; ++kb) {
          const uint32_t st = base + s * STAGE_BYTES;
          if (!mbar_wait(bars + 8u * s, ph, &s_abort)) { live = false; break; }
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
                umma_f16_pair(acc1, ad, bd, idesc, (kb | ks | p) ? 1u : 0u);
              }
            }
          }
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks)
            umma_f16_pair(tmem_acc, a0 + (uint64_t)(ks * 2), b0 + (uint64_t)(ks * 2), idesc, (kb | ks) ? 1u : 0u);
          umma_commit_pair(bars + 8u * (STAGES + s));
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (live) umma_commit_pair(accum_full);
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
    const uint32_t tmem_free_leader = cluster_map(tmem_free, 0u);
    pdl_wait();
    int it = 0;
    for (int tile = pair; tile < ntile; tile += npairs, ++it) {
      const int m0 = ((tile % mt2) * 2 + (int)rank) * BM, n0 = (tile / mt2) * BN;
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
      if (lane == 0) mbar_arrive_cluster(tmem_free_leader);   // the pair's tensor cores may start the next tile
      const bool last = tile + npairs >= ntile;
      const int slot = (tile / mt2) * kParts + part;
      if constexpr (Epi::kHasPmax) {
        if (stage_stride > 0) {
          float* own = reinterpret_cast<float*>(base_ptr + RING + (warp - 2) * STG_WARP);
          float m = -INFINITY;
#pragma unroll
          for (int c0 = 0; c0 < kChunks; c0 += 2) {
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
        // the last tile's accumulators are complete, so neither tensor core reads a ring any more
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
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem_acc, TMEM_COLS);
  if (threadIdx.x == 0 && s_abort) atomicExch(err_flag, 1);
}

// One cluster of two CTAs per SM pair (at most n_sm / 2 pairs); B tensor maps with a box of bn / 2 rows.
template <int NT, int BKT, int FMT, class Epi>
inline cudaError_t launch_gemm_tc_persist_pair(const TmapSet& tm, int M, int N, int K, const Shape& sh, const Epi& epi, int* err_flag,
                                               cudaStream_t st, int n_sm) {
  if (K % sh.bk || sh.stages < 2 || sh.bn % 16) return cudaErrorInvalidValue;
  static bool optin_done[kMaxDevices] = {};
  if (cudaError_t e = ensure_smem_optin(gemm_tc_persist_pair_kernel<NT, BKT, FMT, Epi>, optin_done); e != cudaSuccess) return e;
  const int mt2 = ((M + BM - 1) / BM + 1) / 2;
  const int tiles = mt2 * ((N + sh.bn - 1) / sh.bn);
  const int pairs = tiles < n_sm / 2 ? tiles : n_sm / 2;
  const int stride = sh.nt == 1 ? kPersistStageStride : 0;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = (size_t)sh.smem_bytes; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = sh.pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_tc_persist_pair_kernel<NT, BKT, FMT, Epi>, tm, M, N, K, sh.bn, sh.stages, epi, err_flag, stride);
}

// How many CTA pairs of the one-tile pair kernel the current device holds at once (0: clusters of two such CTAs
// cannot be scheduled here, e.g. on a partitioned device, and the host must keep to the one-tile kernels).
template <int NT, int BKT, int FMT, class Epi>
inline int max_resident_pairs() {
  static bool optin_done[kMaxDevices] = {};
  if (ensure_smem_optin(gemm_tc_pair_kernel<NT, BKT, FMT, Epi>, optin_done) != cudaSuccess) { cudaGetLastError(); return 0; }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2, 1, 1); cfg.blockDim = dim3(kThreadsMain); cfg.dynamicSmemBytes = (size_t)(SMEM_BUDGET + 1280);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<NT, BKT, FMT, Epi>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

}  // namespace tc
}  // namespace linmt

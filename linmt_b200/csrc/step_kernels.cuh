// step_kernels.cuh -- the non-GEMM kernels of the decoding step loop: embedding gather and
// beam reorder, attention, log-softmax + per-beam top-(k+1), beam selection, finalisation.
// All beam state lives on the device; the host only launches.
#pragma once
#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdint.h>

#include "gemm_tc.cuh"

namespace linmt {

constexpr int kMaxBeam = 31;          // kk = beam + 1 <= 32
constexpr int kStart = 0, kEos = 1, kUnk = 2;  // src/input_file_preprocess.cc:549-567
constexpr float kDeadScore = -1e30f;  // score of a hypothesis created when candidates run out

// ---------------------------------------------------------------------------------------
// Encoder input: x[b] = E_src[ids_rev[b][pos]] (SparseLookupKernel,
// src/deep_rnn_kernel.h:248-255); the sentence is read back to front
// (src/decoder_sentence.cu:68).  Rows past their length get zeros.
// grid = (B), block = 256
static __global__ void enc_embed_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ off,
                                 const int32_t* __restrict__ len, const float* __restrict__ emb, int vocab,
                                 float* __restrict__ x, int Hp, int pos) {
  const int b = blockIdx.x;
  const int S = len[b];
  float4* dst = reinterpret_cast<float4*>(x + (size_t)b * Hp);
  if (pos < S) {
    int tok = ids[off[b] + (S - 1 - pos)];
    if (tok < 0 || tok >= vocab) tok = 0;  // out-of-range ids read <UNK> (src/decoder_sentence.cu:61-62)
    const float4* src = reinterpret_cast<const float4*>(emb + (size_t)tok * Hp);
    for (int i = threadIdx.x; i < Hp / 4; i += blockDim.x) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < Hp / 4; i += blockDim.x) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// ---------------------------------------------------------------------------------------
// Start of a decoder step: gathers every state row through the parent chosen by the last
// beam selection and looks up the new token's embedding.  Replaces SwapDecodingStates +
// TargetCopyPrevStates (src/deep_rnn.h:1842-1872, 2L(k+1)+k+2L cudaMemcpy calls) and the
// embedding lookup of src/node_input_to_hidden.h:243.  At step 0 the source rows are the
// encoder's final states, one per sentence (src/deep_rnn.h:1766-1789).
//   src[a], dst[a]: n_arr state arrays [rows][Hp]; src_per_sentence = 1 at step 0.
// grid = (rows, n_arr + 1), block = 256; blockIdx.y == n_arr is the embedding.
struct PrepArrays {
  const float* src[12];
  float* dst[12];
  int n_arr;
};
static __global__ void dec_prep_kernel(PrepArrays arr, const int32_t* __restrict__ parent, const int32_t* __restrict__ tok,
                                const float* __restrict__ emb, int vocab, float* __restrict__ x, int Hp, int k,
                                int src_per_sentence) {
  const int r = blockIdx.x;
  const int a = blockIdx.y;
  const float4* src;
  float4* dst;
  if (a == arr.n_arr) {
    int t = tok[r];
    if (t < 0 || t >= vocab) t = kUnk;
    src = reinterpret_cast<const float4*>(emb + (size_t)t * Hp);
    dst = reinterpret_cast<float4*>(x + (size_t)r * Hp);
  } else {
    const int sent = r / k;
    const int srow = src_per_sentence ? sent : sent * k + parent[r];
    src = reinterpret_cast<const float4*>(arr.src[a] + (size_t)srow * Hp);
    dst = reinterpret_cast<float4*>(arr.dst[a] + (size_t)r * Hp);
  }
  for (int i = threadIdx.x; i < Hp / 4; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------
// The same step start for the tensor-core path, where states live as bf16 planes inside the
// operand panels: a list of byte-row copy jobs.  kind 0: state row gathered through the parent
// (or, at step 0, the sentence's encoder row); kind 1: embedding row of the slot's token.
// grid = (rows, n_jobs), block = 128
struct GatherJob {
  const unsigned char* src; long long src_stride;   // bytes
  unsigned char* dst; long long dst_stride;
  int row_bytes;   // multiple of 16
  int kind;
};
struct GatherJobs {
  GatherJob j[32];
  int n;
};
constexpr int kGatherJobsPerBlock = 4;   // a full step (768 rows x 10 jobs) is then 2304 blocks: one wave of resident CTAs
static __global__ void row_gather_kernel(GatherJobs jobs, const int32_t* __restrict__ parent, const int32_t* __restrict__ tok,
                                         int vocab, int k, int src_per_sentence) {
  tc::pdl_launch_dependents();   // see gemm_tc.cuh: the next kernel of the step may start its prologue
  tc::pdl_wait();                // nothing below runs before the previous kernel's results are visible
  const int r = blockIdx.x;
  const int j0 = blockIdx.y * kGatherJobsPerBlock;
  const int sent = r / k;
  const long long prow = src_per_sentence ? sent : sent * k + parent[r];
  // every thread moves 16 bytes of up to four jobs at a time: all loads first, then the stores
  const unsigned char* src[kGatherJobsPerBlock];
  unsigned char* dst[kGatherJobsPerBlock];
  int nchunk[kGatherJobsPerBlock];
  int most = 0;
#pragma unroll
  for (int q = 0; q < kGatherJobsPerBlock; ++q) {
    nchunk[q] = 0; src[q] = nullptr; dst[q] = nullptr;
    if (j0 + q < jobs.n) {
      const GatherJob& jb = jobs.j[j0 + q];
      long long srow = prow;
      if (jb.kind == 1) {
        int t = tok[r];
        if (t < 0 || t >= vocab) t = kUnk;
        srow = t;
      }
      src[q] = jb.src + srow * jb.src_stride;
      dst[q] = jb.dst + (long long)r * jb.dst_stride;
      nchunk[q] = jb.row_bytes / 16;
      most = nchunk[q] > most ? nchunk[q] : most;
    }
  }
  for (int c = threadIdx.x; c < most; c += blockDim.x) {
    uint4 v[kGatherJobsPerBlock];
#pragma unroll
    for (int q = 0; q < kGatherJobsPerBlock; ++q)
      if (c < nchunk[q]) v[q] = reinterpret_cast<const uint4*>(src[q])[c];
#pragma unroll
    for (int q = 0; q < kGatherJobsPerBlock; ++q)
      if (c < nchunk[q]) reinterpret_cast<uint4*>(dst[q])[c] = v[q];
  }
}

// Encoder input for the tensor-core path: embedding planes of the token at reversed position
// `pos` into columns [0, Hp) of the layer-0 panel; zeros past the sentence.
// grid = (B, nt), block = 128
static __global__ void enc_embed_planes_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ off,
                                               const int32_t* __restrict__ len, tc::Planes emb, int vocab,
                                               tc::Planes dst, int Hp, int pos) {
  const int b = blockIdx.x, t = blockIdx.y;
  const int S = len[b];
  uint4* d = reinterpret_cast<uint4*>(dst.p[t] + (size_t)b * dst.ld);
  if (pos < S) {
    int tok = ids[off[b] + (S - 1 - pos)];
    if (tok < 0 || tok >= vocab) tok = 0;
    const uint4* src = reinterpret_cast<const uint4*>(emb.p[t] + (size_t)tok * emb.ld);
    for (int i = threadIdx.x; i < Hp / 8; i += blockDim.x) d[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < Hp / 8; i += blockDim.x) d[i] = make_uint4(0, 0, 0, 0);
  }
}

// ---------------------------------------------------------------------------------------
// Block-wide sum in a fixed order (deterministic).
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = blockDim.x >> 5;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// ---------------------------------------------------------------------------------------
// Attention for one decoder row (AttentionNode::ForwardProp, src/layer_attention.h:243-483,
// kernels k12-k20: Sgemm m=1, SigmoidKernel, AlignmentPosKernel, LowerUpperKernel,
// CreateIndicesKernel, LoadInHSKernel, ElemReduceKernelLarge, AlignmentReductionKernel,
// CreateCTKernel).
//   proj [rows][2*Hp]: tanh(W_p h) | W_a^T h      (global_dot: `u` = h_top itself)
//   hs   [B][max_src][Hp]: top encoder state after consuming reversed position p
//   ctx  [rows][Hp] fp32 and/or ctx_planes (bf16 planes, columns [0,Hp) of the panel)
//   rec_align [rows][rec_win] / rec_lo [rows] / rec_vit [rows]: alignment record of this step
//   (may be null).  win = 2D+1 for local attention, max_src for the global modes.
//   ens = 0: one model; the record is the window (rec_win = win) and its first position rec_lo.
//   ens = 1, 2, 3: first / middle / last member of an ensemble; the record is dense over the source
//   (rec_win = max_src, rec_lo = 0), the first member writes it, the others add to it in member order,
//   and the last one takes the vote: the position of the largest summed score, the search starting from
//   "none, 0" (EnsembleFactory::EnsemblesModels, src/decoder.h:1934-1964).
// grid = rows, block = 256, dynamic smem = (win + 8) floats.  The kernel is a chain of L2 round trips, not
// of bytes.  (Three variations were tried and measured no faster: the window's states kept in shared memory
// between the score sweep and the context sweep -- 86 KB per CTA costs the occupancy the halved traffic buys;
// one CTA per group of beams of a sentence reading every state row once for all of them -- a quarter of the
// CTAs, the same chain of round trips in each; and loads issued in batches of eight ahead of the arithmetic --
// the registers cost more occupancy than the batching hides latency.)
// Optional record of the attention centre p_t of every row of a forward (local attention): the parity tests
// use it to tell a window that was cut on the other side of an integer apart from an error.
struct AttTrace {
  float* pt;            // [n][T1][k] by the caller's sentence index, or null
  const int32_t* orig;  // batch slot -> caller's sentence index
  int T1;               // forwards per sentence in the record (longest step count + 1)
  int t;                // this forward
};
// Optional fold of the attention output layer into this kernel.  htilde = tanh(W_c1 ctx + W_c2 h + b) and
// ctx = sum_j a_j hs_j, so W_c1 ctx = sum_j a_j (W_c1 hs_j): with `cs` = the encoder states already multiplied by
// W_c1 (once per batch), the weighted sum IS the first term, `add` carries the row's W_c2 h (computed with the
// attention projections) and the kernel writes the attentional state itself -- a dependent GEMM launch less per
// step.  cs == nullptr: plain context.
struct AttFold {
  const float* cs;      // [B][max_src][Hp] like hs
  const float* add; int ld_add;   // element (row, j) at add[row * ld_add + j]
  const float* bias;    // [Hp]
};
// (six CTAs per SM: 888 resident CTAs hold the 768 rows of a full step in one wave; at five, 28 rows ran as a second wave)
static __global__ void __launch_bounds__(256, 6) attention_kernel(const float* __restrict__ proj, int ldp, const float* __restrict__ u_alt, int ldu,
                                 const float* __restrict__ vp, const float* __restrict__ hs,
                                 const int32_t* __restrict__ src_len, float* __restrict__ ctx, int H, int Hp,
                                 int k, int max_src, int mode, int D, int win, float* __restrict__ rec_align,
                                 int32_t* __restrict__ rec_lo, int32_t* __restrict__ rec_vit, tc::Planes ctx_planes, int nt,
                                 int rec_win, int ens, AttTrace at, AttFold fold) {
  tc::pdl_launch_dependents();   // see gemm_tc.cuh: the next kernel of the step may start its prologue
  tc::pdl_wait();                // nothing below runs before the previous kernel's results are visible
  extern __shared__ float sm[];
  float* e = sm;            // [win]
  float* red = sm + win;    // [8]
  __shared__ float s_pt;
  __shared__ int s_lo, s_hi;
  const int r = blockIdx.x;
  const int sent = r / k;
  const int S = src_len[sent];
  const float* u = u_alt ? (u_alt + (size_t)r * ldu) : (proj + (size_t)r * ldp + Hp);
  const float* hsb = hs + (size_t)sent * max_src * Hp;

  if (mode == 0) {
    float part = 0.f;
    const float* t1 = proj + (size_t)r * ldp;
    for (int j = threadIdx.x; j < H; j += blockDim.x) part = fmaf(vp[j], t1[j], part);
    const float dot = block_sum(part, red);
    if (threadIdx.x == 0) {
      const float sg = (float)(1.0 / (1.0 + exp(-1.0 * (double)dot)));  // SigmoidKernel, deep_rnn_kernel.h:1075-1080
      const float pt = (float)S * sg;
      s_pt = pt;
      s_lo = (0 > (int)pt - D) ? 0 : ((int)pt - D);                       // LowerUpperKernel, :1094-1100
      s_hi = ((S - 1) < (int)pt + D) ? (S - 1) : ((int)pt + D);
      if (at.pt) at.pt[((size_t)at.orig[sent] * at.T1 + at.t) * k + (r - sent * k)] = pt;
    }
  } else if (threadIdx.x == 0) {
    s_pt = 0.f; s_lo = 0; s_hi = S - 1;
  }
  __syncthreads();
  const int lo = s_lo, hi = s_hi;
  const int W = hi - lo + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int w = warp; w < W; w += nw) {
    const float* hrow = hsb + (size_t)(S - 1 - (lo + w)) * Hp;
    float acc = 0.f;
    for (int j = lane * 4; j < Hp; j += 128) {
      const float4 a = *reinterpret_cast<const float4*>(hrow + j);
      const float4 b = *reinterpret_cast<const float4*>(u + j);
      acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) e[w] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    // AlignmentReductionKernel, deep_rnn_kernel.h:1197-1241 (max starts at 0, no renormalisation
    // after the Gaussian), one lane per window position instead of one thread per beam
    float mx = 0.f;
    for (int w = lane; w < W; w += 32) mx = fmaxf(mx, e[w]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int w = lane; w < W; w += 32) { const float ev = expf(e[w] - mx); e[w] = ev; sum += ev; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float sigma_sq = ((float)D * (float)D) / 4.0f;
    const float pt = s_pt;
    float best = 0.f; int besti = 0x7fffffff;
    for (int w = lane; w < W; w += 32) {
      float a = e[w];
      if (mode == 0) {
        const float tmp = expf((-1 * powf(pt - (float)(lo + w), 2.0f)) / (2 * sigma_sq));
        if (0 != sum) a = (a / sum) * tmp;
      } else if (0 != sum) a = a / sum;
      e[w] = a;
      if (a > best) { best = a; besti = lo + w; }  // viterbi vote, src/decoder.h:1948-1962 (first maximum)
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
    }
    if (lane == 0 && rec_lo && ens == 0) { rec_lo[r] = lo; rec_vit[r] = (best > 0.f) ? besti : -1; }
  }
  __syncthreads();
  if (rec_align && ens == 0)
    for (int w = threadIdx.x; w < rec_win; w += blockDim.x) rec_align[(size_t)r * rec_win + w] = (w < W) ? e[w] : 0.f;
  if (rec_align && ens != 0) {
    float* row = rec_align + (size_t)r * rec_win;
    for (int sp = threadIdx.x; sp < rec_win; sp += blockDim.x) {
      const float a = (sp >= lo && sp <= hi) ? e[sp - lo] : 0.f;
      row[sp] = (ens == 1) ? (0.f + a) : (row[sp] + a);
    }
    if (ens == 3) {
      __syncthreads();
      if (warp == 0) {
        float best = 0.f; int besti = 0x7fffffff;
        for (int sp = lane; sp < rec_win; sp += 32) {
          const float a = row[sp];
          if (a > best) { best = a; besti = sp; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
          if (ob > best || (ob == best && oi < besti)) { best = ob; besti = oi; }
        }
        if (lane == 0) { rec_lo[r] = 0; rec_vit[r] = (best > 0.f) ? besti : -1; }
      }
    }
  }
  // context: CreateCTKernel, deep_rnn_kernel.h:1250-1260 (sum over window positions in order)
  float* crow = ctx ? ctx + (size_t)r * Hp : nullptr;
  const float* csb = fold.cs ? fold.cs + (size_t)sent * max_src * Hp : hsb;
  for (int j = threadIdx.x * 4; j < Hp; j += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int w = 0; w < W; ++w) {
      const float a = e[w];
      const float4 h4 = *reinterpret_cast<const float4*>(csb + (size_t)(S - 1 - (lo + w)) * Hp + j);
      acc.x += a * h4.x; acc.y += a * h4.y; acc.z += a * h4.z; acc.w += a * h4.w;
    }
    if (fold.cs) {
      // the attentional state: the sums of TcEpiBiasTanh in its order, (W_c1 ctx + W_c2 h) + b
      const float4 g = *reinterpret_cast<const float4*>(fold.add + (size_t)r * fold.ld_add + j);
      const float4 b = *reinterpret_cast<const float4*>(fold.bias + j);
      acc.x = tc::tanh_fast((acc.x + g.x) + b.x); acc.y = tc::tanh_fast((acc.y + g.y) + b.y);
      acc.z = tc::tanh_fast((acc.z + g.z) + b.z); acc.w = tc::tanh_fast((acc.w + g.w) + b.w);
    }
    if (crow) *reinterpret_cast<float4*>(crow + j) = acc;
    if (ctx_planes.p[0]) {  // tensor-core path: the context goes straight into its operand panel
      const size_t idx = (size_t)r * ctx_planes.ld + j;
      tc::split_store4(ctx_planes, nt, idx, acc.x, acc.y, acc.z, acc.w);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Log-softmax statistics and per-row top-kk of the logits in ONE pass over HBM.
// Replaces MatrixBiasKernel's consumer OutputdistOverflowPreventionKernel
// (src/deep_rnn_kernel.h:352-429, three passes), the V x k device-to-host copy
// (src/decoder.h:1413) and the host scan that keeps the k+1 best per beam
// (src/decoder.h:401-410).  Order: value descending, vocabulary index ascending -- what the
// strict-greater replacement of the reference keeps.  log p = (z - max) - log(sum exp).
// grid = rows, block = 256.
struct TopkOut {
  int32_t* idx;    // [rows][kk]
  float* logp;     // [rows][kk]
  float* eos_logp; // [rows]
  float* row_stats; // [rows][2] = (max, log sum exp(z - max)) of the row, may be null
};
__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

// Refinement of a row whose logits came from a ONE-product (plain fp16) vocabulary GEMM: the row's
// activations and the vocabulary weights as fp16 pairs, from which the few logits that matter are
// recomputed at fp32-class accuracy.  eps_coef * |a|_2 bounds the error of a one-product logit
// (both operands rounded to 11 bits: relative 2^-10 on every term, Cauchy-Schwarz over the row,
// largest weight-row norm of the model folded into eps_coef).
struct TopkRefine {
  const __half* a0; const __half* a1; int lda;   // activations [rows][lda], planes of the fp16 pair
  const __half* b0; const __half* b1; int ldb;   // vocabulary weights [V][ldb]
  const float* bias;                             // [V]
  int K;
  float eps_coef;
};
constexpr float kPairInv = 1.0f / 2048.0f;

// Pass 1 finds the row maximum and, from the 256 per-thread maxima, a threshold that at least
// kk elements reach (the kk-th largest thread maximum).  Pass 2 (the row is L2/L1 resident by
// then) sums exp(z - max) and collects the few elements at or above the threshold, which are
// then ranked exactly.  If more elements than the candidate buffer holds reach the threshold
// (e.g. a row of equal logits) the block falls back to kk exact arg-best sweeps.
constexpr int kTopkCap = 1024;
static __global__ void __launch_bounds__(256, 6) softmax_topk_kernel(const float* __restrict__ logits, int ld, int V, int kk, TopkOut out,
                                                                  int normalise, const float* __restrict__ pmax, int pmax_ld, int n_slots, TopkRefine rf,
                                                                  const __half* __restrict__ logits16) {
  extern __shared__ float s_a[];   // [rf.K] the row's activations in fp32 (refinement only)
  tc::pdl_launch_dependents();   // see gemm_tc.cuh: the next kernel of the step may start its prologue
  tc::pdl_wait();                // nothing below runs before the previous kernel's results are visible
  __shared__ float s_tmax[256];
  __shared__ float s_cv[kTopkCap];
  __shared__ int s_ci[kTopkCap];
  __shared__ float s_red[8];
  __shared__ int s_redi[8];
  __shared__ float s_cd[kTopkCap];   // refinement: change of exp(z - max) per candidate, in buffer order ...
  __shared__ float s_co[kTopkCap];   // ... and in vocabulary order
  __shared__ int s_count;
  __shared__ float s_tau, s_max, s_lse, s_sum, s_eos, s_eos_delta;
  const int r = blockIdx.x, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const float* z = logits + (size_t)r * ld;
  // fp16 logits (refinement mode only: the candidates' values are recomputed, the rest only enter the sum)
  const __half* zh = logits16 ? logits16 + (size_t)r * ld : nullptr;
  auto zat = [&](int i) { return zh ? __half2float(zh[i]) : z[i]; };
  const int V4 = V & ~3;
  // ---- pass 1: maxima (four independent 16-byte loads in flight per thread) -- or, when the GEMM that
  // produced the logits left the maxima of disjoint column blocks of every row (pmax), just those ----
  float m = -INFINITY;
  if (pmax) {
    for (int s = tid; s < n_slots; s += 256) m = fmaxf(m, pmax[(size_t)r * pmax_ld + s]);
  } else if (zh) {
    for (int i = tid; i < V; i += 256) m = fmaxf(m, __half2float(zh[i]));
  } else {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
    int i = tid * 4;
    for (; i + 3 * 1024 < V4; i += 4 * 1024) {
      const float4 q0 = *reinterpret_cast<const float4*>(z + i);
      const float4 q1 = *reinterpret_cast<const float4*>(z + i + 1024);
      const float4 q2 = *reinterpret_cast<const float4*>(z + i + 2048);
      const float4 q3 = *reinterpret_cast<const float4*>(z + i + 3072);
      m0 = fmaxf(fmaxf(m0, q0.x), fmaxf(q0.y, fmaxf(q0.z, q0.w)));
      m1 = fmaxf(fmaxf(m1, q1.x), fmaxf(q1.y, fmaxf(q1.z, q1.w)));
      m2 = fmaxf(fmaxf(m2, q2.x), fmaxf(q2.y, fmaxf(q2.z, q2.w)));
      m3 = fmaxf(fmaxf(m3, q3.x), fmaxf(q3.y, fmaxf(q3.z, q3.w)));
    }
    for (; i < V4; i += 1024) {
      const float4 q = *reinterpret_cast<const float4*>(z + i);
      m0 = fmaxf(fmaxf(m0, q.x), fmaxf(q.y, fmaxf(q.z, q.w)));
    }
    m = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
    for (int i = V4 + tid; i < V; i += 256) m = fmaxf(m, z[i]);
  }
  s_tmax[tid] = m;
  if (tid == 0) s_count = 0;
  __syncthreads();
  if (kk <= 32) {
    // Threshold from 32 group maxima (group = the 8 threads with the same lane): each is an
    // element of the row and the groups are disjoint, so at least kk elements reach the kk-th
    // largest of them; it is a little lower than the kk-th largest thread maximum (a few more
    // candidates to rank) and costs one warp ~100 instructions instead of 256 x 256 compares.
    if (warp == 0) {
      float g = -INFINITY;
#pragma unroll
      for (int w = 0; w < 8; ++w) g = fmaxf(g, s_tmax[w * 32 + lane]);
      float bm = g;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
      int rank = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float o = __shfl_sync(0xffffffffu, g, j);
        rank += (o > g || (o == g && j < lane)) ? 1 : 0;
      }
      if (rank == kk - 1) s_tau = g;
      if (lane == 0) s_max = bm;
    }
  } else {
    int rank = 0;
    float bm = -INFINITY;
    for (int j = 0; j < 256; ++j) {
      const float o = s_tmax[j];
      bm = fmaxf(bm, o);
      rank += (o > m || (o == m && j < tid)) ? 1 : 0;
    }
    if (rank == (kk < 256 ? kk : 256) - 1) s_tau = m;
    if (tid == 0) s_max = bm;
  }
  __syncthreads();
  if (pmax) {
    // The threshold from 32 group maxima admits a few dozen elements.  A tighter one costs little here: the
    // block maxima that reach it are few, each is an element of the row, the blocks are disjoint, and the
    // kk-th largest of them is still reached by at least kk elements.
    const float tau0 = s_tau;
    for (int sl = tid; sl < n_slots; sl += 256) {
      const float v = pmax[(size_t)r * pmax_ld + sl];
      if (v >= tau0) {
        const int pos = atomicAdd(&s_count, 1);
        if (pos < kTopkCap) s_cv[pos] = v;
      }
    }
    __syncthreads();
    const int m2 = s_count;
    if (m2 <= kTopkCap)
      for (int c = tid; c < m2; c += 256) {
        const float v = s_cv[c];
        int rank = 0;
        for (int d = 0; d < m2; ++d) rank += (s_cv[d] > v || (s_cv[d] == v && d < c)) ? 1 : 0;
        if (rank == kk - 1) s_tau = v;
      }
    __syncthreads();
    if (tid == 0) s_count = 0;
    __syncthreads();
  }
  float tau = s_tau;
  const float rmax = s_max;
  if (rf.a0) {
    // Every logit in this row is within eps of its accurate value, so the accurate top-kk all lie at or
    // above (kk-th largest approximate value) - 2 eps, and tau is no larger than that kk-th value.
    float ss = 0.f;
    for (int j = tid; j < rf.K; j += 256) {
      const float a = __half2float(rf.a0[(size_t)r * rf.lda + j]) + __half2float(rf.a1[(size_t)r * rf.lda + j]) * kPairInv;
      s_a[j] = a;
      ss = fmaf(a, a, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += s_red[w];
    tau -= 2.0f * (rf.eps_coef * sqrtf(tot) + 1e-5f);   // + fp16 subnormals and the accumulator's own rounding
    if (zh) tau -= 2.0f * 4.9e-4f * fmaxf(fabsf(rmax), fabsf(tau));   // and the rounding of the stored value (2^-11 relative)
    __syncthreads();
  }
  // ---- pass 2: sum of exponentials, candidates ----
  float ssum = 0.f;
  auto visit = [&](float v, int i) {
    ssum += __expf(v - rmax);  // arguments in [-few, 0]: ~1e-7 relative on the sum of V terms
    if (v >= tau) {
      const int pos = atomicAdd(&s_count, 1);
      if (pos < kTopkCap) { s_cv[pos] = v; s_ci[pos] = i; }
    }
  };
  {
    // four independent 16-byte loads in flight per thread; candidates are rare, so a group of four is
    // first tested as a whole against the threshold
    auto group = [&](const float4& q, int i) {
      ssum += __expf(q.x - rmax) + __expf(q.y - rmax);
      ssum += __expf(q.z - rmax) + __expf(q.w - rmax);
      if (fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)) >= tau) {
        const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v[u] >= tau) {
            const int pos = atomicAdd(&s_count, 1);
            if (pos < kTopkCap) { s_cv[pos] = v[u]; s_ci[pos] = i + u; }
          }
      }
    };
    if (zh) {
      // eight values per 16-byte load, blocks of 2048 columns, from the last one down
      auto group8 = [&](const uint4& q, int i) {
        const __half2* h = reinterpret_cast<const __half2*>(&q);
        const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
        group(make_float4(a.x, a.y, b.x, b.y), i);
        group(make_float4(c.x, c.y, d.x, d.y), i + 4);
      };
      const int V8 = V & ~7;
      const int top8 = V8 & ~2047;
      if (top8 + tid * 8 < V8) group8(*reinterpret_cast<const uint4*>(zh + top8 + tid * 8), top8 + tid * 8);
      int i = top8 - 2048 + tid * 8;
      for (; i - 3 * 2048 >= 0; i -= 4 * 2048) {
        const uint4 q0 = *reinterpret_cast<const uint4*>(zh + i);
        const uint4 q1 = *reinterpret_cast<const uint4*>(zh + i - 2048);
        const uint4 q2 = *reinterpret_cast<const uint4*>(zh + i - 4096);
        const uint4 q3 = *reinterpret_cast<const uint4*>(zh + i - 6144);
        group8(q0, i); group8(q1, i - 2048); group8(q2, i - 4096); group8(q3, i - 6144);
      }
      for (; i >= 0; i -= 2048) group8(*reinterpret_cast<const uint4*>(zh + i), i);
      for (int j = V8 + tid; j < V; j += 256) visit(__half2float(zh[j]), j);
    } else {
    // From the last column block down: the GEMM that wrote the logits walked the column tiles upwards, so the
    // highest columns of every row are the ones still in L2 (all rows are swept at the same time).
    const int top = V4 & ~1023;                       // start of the last, possibly partial, block of 1024
    if (top + tid * 4 < V4) group(*reinterpret_cast<const float4*>(z + top + tid * 4), top + tid * 4);
    int i = top - 1024 + tid * 4;
    for (; i - 3 * 1024 >= 0; i -= 4 * 1024) {
      const float4 q0 = *reinterpret_cast<const float4*>(z + i);
      const float4 q1 = *reinterpret_cast<const float4*>(z + i - 1024);
      const float4 q2 = *reinterpret_cast<const float4*>(z + i - 2048);
      const float4 q3 = *reinterpret_cast<const float4*>(z + i - 3072);
      group(q0, i); group(q1, i - 1024); group(q2, i - 2048); group(q3, i - 3072);
    }
    for (; i >= 0; i -= 1024) group(*reinterpret_cast<const float4*>(z + i), i);
    for (int j = V4 + tid; j < V; j += 256) visit(z[j], j);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
  if (lane == 0) s_red[warp] = ssum;
  __syncthreads();
  if (tid == 0) {
    float bs = 0.f;
    for (int w = 0; w < 8; ++w) bs += s_red[w];
    s_sum = bs;
    s_lse = normalise ? logf(bs) : -rmax;   // normalise = 0: the row already holds log-probabilities
    if (!rf.a0) {
      if (out.eos_logp) out.eos_logp[r] = (zat(kEos) - rmax) - s_lse;
      if (out.row_stats) { out.row_stats[2 * r] = rmax; out.row_stats[2 * r + 1] = s_lse; }
    }
  }
  __syncthreads();
  int n = s_count;
  if (rf.a0 && n > kTopkCap) {
    // More elements than the buffer holds reach the widened threshold (a nearly flat row): pick the kk best
    // of the one-product logits by exact sweeps and make those the candidates.  Their values are refined
    // like any others below; an element within the error bound just beyond the kk-th can be missed here,
    // which on a row this flat is a tie within the tolerance.
    float last_v = INFINITY;
    int last_i = -1;
    for (int round = 0; round < kk; ++round) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int i = tid; i < V; i += 256) {
        const float v = zat(i);
        const bool after = (v < last_v) || (v == last_v && i > last_i);
        if (after && better(v, i, bv, bi)) { bv = v; bi = i; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
      __syncthreads();
      if (lane == 0) { s_red[warp] = bv; s_redi[warp] = bi; }
      __syncthreads();
      bv = s_red[0]; bi = s_redi[0];
      for (int w = 1; w < 8; ++w) if (better(s_red[w], s_redi[w], bv, bi)) { bv = s_red[w]; bi = s_redi[w]; }
      if (tid == 0) { s_cv[round] = bv; s_ci[round] = bi; }
      last_v = bv; last_i = bi;
    }
    __syncthreads();
    n = 0;
    while (n < kk && s_ci[n] != 0x7fffffff) ++n;   // fewer than kk elements in the row
    __syncthreads();
    if (tid == 0) s_count = n;
  }
  if (rf.a0) {
    // accurate values for the candidates (and for EOS, whose log-probability is always reported): one
    // warp per candidate, fp32 FMAs over the two planes of both operands.  Each also yields the term by
    // which the row's sum of exponentials changes when the accurate value replaces the one-product one:
    // on a peaked row the few dominant logits ARE the normaliser, and their fp16-product error would
    // otherwise go straight into every log-probability of the row.
    const int nc = n;
    for (int c = warp; c <= nc; c += 8) {
      const int v = (c < nc) ? s_ci[c] : kEos;
      const __half* w0 = rf.b0 + (size_t)v * rf.ldb;
      const __half* w1 = rf.b1 + (size_t)v * rf.ldb;
      float acc = 0.f;
      for (int j = lane * 4; j < rf.K; j += 128) {
        const uint2 q0 = *reinterpret_cast<const uint2*>(w0 + j);
        const uint2 q1 = *reinterpret_cast<const uint2*>(w1 + j);
        const __half2 h00 = *reinterpret_cast<const __half2*>(&q0.x), h01 = *reinterpret_cast<const __half2*>(&q0.y);
        const __half2 h10 = *reinterpret_cast<const __half2*>(&q1.x), h11 = *reinterpret_cast<const __half2*>(&q1.y);
        const float2 b00 = __half22float2(h00), b01 = __half22float2(h01), b10 = __half22float2(h10), b11 = __half22float2(h11);
        acc = fmaf(s_a[j + 0], fmaf(b10.x, kPairInv, b00.x), acc);
        acc = fmaf(s_a[j + 1], fmaf(b10.y, kPairInv, b00.y), acc);
        acc = fmaf(s_a[j + 2], fmaf(b11.x, kPairInv, b01.x), acc);
        acc = fmaf(s_a[j + 3], fmaf(b11.y, kPairInv, b01.y), acc);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) {
        const float zv = acc + (rf.bias ? rf.bias[v] : 0.f);
        const float za = (c < nc) ? s_cv[c] : zat(kEos);
        const float delta = __expf(zv - rmax) - __expf(za - rmax);
        if (c < nc) { s_cv[c] = zv; s_cd[c] = delta; }
        else { s_eos = zv; s_eos_delta = delta; }
      }
    }
    __syncthreads();
    // the correction is summed in vocabulary order, so the result does not depend on the order in which
    // the candidates happened to enter the buffer
    bool eos_listed = false;
    for (int c = tid; c < nc; c += 256) {
      const int i = s_ci[c];
      int pos = 0;
      for (int d = 0; d < nc; ++d) pos += (s_ci[d] < i) ? 1 : 0;
      s_co[pos] = s_cd[c];
    }
    __syncthreads();
    if (tid == 0) {
      float corr = 0.f;
      for (int c = 0; c < nc; ++c) { corr += s_co[c]; eos_listed = eos_listed || (s_ci[c] == kEos); }
      if (!eos_listed) corr += s_eos_delta;
      const float bs = s_sum + corr;
      s_lse = normalise ? logf(bs > 0.f ? bs : s_sum) : -rmax;
      if (out.eos_logp) out.eos_logp[r] = (s_eos - rmax) - s_lse;
      if (out.row_stats) { out.row_stats[2 * r] = rmax; out.row_stats[2 * r + 1] = s_lse; }
    }
    __syncthreads();
  }
  const float rlse = s_lse;
  if (n <= kTopkCap) {
    // exact ranking of the candidates: value descending, index ascending
    for (int c = tid; c < n; c += 256) {
      const float v = s_cv[c];
      const int i = s_ci[c];
      int rank = 0;
      for (int d = 0; d < n; ++d) rank += better(s_cv[d], s_ci[d], v, i) ? 1 : 0;
      if (rank < kk) {
        out.idx[(size_t)r * kk + rank] = i;
        out.logp[(size_t)r * kk + rank] = (v - rmax) - rlse;
      }
    }
    for (int q = n + tid; q < kk; q += 256) {  // fewer than kk elements in the row
      out.idx[(size_t)r * kk + q] = -1;
      out.logp[(size_t)r * kk + q] = -INFINITY;
    }
    return;
  }
  // ---- fallback: kk sweeps, each picking the best element after the previous pick ----
  float last_v = INFINITY;
  int last_i = -1;
  for (int round = 0; round < kk; ++round) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += 256) {
      const float v = zat(i);
      const bool after = (v < last_v) || (v == last_v && i > last_i);
      if (after && better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    __syncthreads();
    if (lane == 0) { s_red[warp] = bv; s_redi[warp] = bi; }
    __syncthreads();
    bv = s_red[0]; bi = s_redi[0];
    for (int w = 1; w < 8; ++w) if (better(s_red[w], s_redi[w], bv, bi)) { bv = s_red[w]; bi = s_redi[w]; }
    if (tid == 0) {
      const bool valid = bi != 0x7fffffff;
      out.idx[(size_t)r * kk + round] = valid ? bi : -1;
      out.logp[(size_t)r * kk + round] = valid ? ((bv - rmax) - rlse) : -INFINITY;
    }
    last_v = bv; last_i = bi;
  }
}

inline cudaError_t launch_softmax_topk(const float* logits, int ld, int V, int kk, int rows, const TopkOut& out, int normalise,
                                       cudaStream_t st, bool pdl = false, const float* pmax = nullptr, int pmax_ld = 0, int n_slots = 0,
                                       const TopkRefine* refine = nullptr, const __half* logits16 = nullptr) {
  if (n_slots <= 0) pmax = nullptr;
  TopkRefine rf{};
  if (refine) rf = *refine;
  const size_t smem = rf.a0 ? sizeof(float) * (size_t)rf.K : 0;
  return tc::launch_k(pdl, softmax_topk_kernel, dim3(rows), dim3(256), smem, st, logits, ld, V, kk, out, normalise, pmax, pmax_ld, n_slots, rf, refine ? logits16 : (const __half*)nullptr);
}

// ---------------------------------------------------------------------------------------
// Ensemble of up to 8 members for one row: out[v] = log(mean_m softmax(z_m)[v]) (mode 0, the
// reference's rule, src/decoder.h:1913-1921 -- its renormalisation, :1923-1931, is the
// log-softmax the next kernel applies to this row) or mean_m log softmax(z_m)[v] (mode 1).
// Two sweeps over the members' rows (HBM-bound: each row of logits is read twice, the combined row
// written once): running (max, sum of exponentials) per member, then the combination.
// grid = rows, block = 256
struct EnsembleRows {
  const float* logits[8];
  int n;
};
static __global__ void __launch_bounds__(256) ensemble_combine_kernel(EnsembleRows er, int ld, int V, int mode, float* __restrict__ out) {
  tc::pdl_launch_dependents();   // see gemm_tc.cuh: the next kernel of the step may start its prologue
  tc::pdl_wait();                // nothing below runs before the previous kernel's results are visible
  __shared__ float s_m[8][8], s_s[8][8];   // [member][warp] partial (max, sum of exp relative to it)
  __shared__ float s_max[8], s_lse[8];
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int V4 = V & ~3;
  // one sweep per member: running maximum and sum of exponentials relative to it (16-byte loads, two in flight)
  for (int m = 0; m < er.n; ++m) {
    const float* z = er.logits[m] + (size_t)r * ld;
    float mx = -INFINITY, sum = 0.f;
    auto take = [&](float x) {
      if (x > mx) { sum = sum * __expf(mx - x) + 1.0f; mx = x; }
      else sum += __expf(x - mx);
    };
    int i = tid * 4;
    for (; i + 1024 < V4; i += 2048) {
      const float4 q0 = *reinterpret_cast<const float4*>(z + i);
      const float4 q1 = *reinterpret_cast<const float4*>(z + i + 1024);
      take(q0.x); take(q0.y); take(q0.z); take(q0.w);
      take(q1.x); take(q1.y); take(q1.z); take(q1.w);
    }
    for (; i < V4; i += 1024) {
      const float4 q = *reinterpret_cast<const float4*>(z + i);
      take(q.x); take(q.y); take(q.z); take(q.w);
    }
    for (int j = V4 + tid; j < V; j += 256) take(z[j]);
    // combine (max, sum) pairs in a fixed order: lanes by shuffle tree, then the warps one after the other
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o);
      const float os = __shfl_xor_sync(0xffffffffu, sum, o);
      const float nm = fmaxf(mx, om);
      sum = (nm == -INFINITY) ? 0.f : sum * __expf(mx - nm) + os * __expf(om - nm);
      mx = nm;
    }
    if (lane == 0) { s_m[m][warp] = mx; s_s[m][warp] = sum; }
  }
  __syncthreads();
  if (tid < er.n) {
    float mx = s_m[tid][0], sum = s_s[tid][0];
    for (int w = 1; w < 8; ++w) {
      const float om = s_m[tid][w], os = s_s[tid][w];
      const float nm = fmaxf(mx, om);
      sum = (nm == -INFINITY) ? 0.f : sum * __expf(mx - nm) + os * __expf(om - nm);
      mx = nm;
    }
    s_max[tid] = mx; s_lse[tid] = logf(sum);
  }
  __syncthreads();
  // second sweep: the members' probabilities (or log-probabilities) of four classes at a time, accumulated in
  // double like the reference's loop (src/decoder.h:1913-1921)
  float* o = out + (size_t)r * ld;
  const float inv_n = 1.0f / er.n;
  for (int i = tid * 4; i < V4; i += 1024) {
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    for (int m = 0; m < er.n; ++m) {
      const float4 q = *reinterpret_cast<const float4*>(er.logits[m] + (size_t)r * ld + i);
      const float c = s_max[m] + s_lse[m];
      const float l0 = q.x - c, l1 = q.y - c, l2 = q.z - c, l3 = q.w - c;   // (z - max) - lse up to one rounding
      if (mode == 0) { a0 += (double)expf(l0); a1 += (double)expf(l1); a2 += (double)expf(l2); a3 += (double)expf(l3); }
      else { a0 += (double)l0; a1 += (double)l1; a2 += (double)l2; a3 += (double)l3; }
    }
    float4 w;
    if (mode == 0) w = make_float4(logf((float)(a0 / er.n)), logf((float)(a1 / er.n)), logf((float)(a2 / er.n)), logf((float)(a3 / er.n)));
    else w = make_float4((float)(a0 / er.n), (float)(a1 / er.n), (float)(a2 / er.n), (float)(a3 / er.n));
    *reinterpret_cast<float4*>(o + i) = w;
  }
  for (int j = V4 + tid; j < V; j += 256) {
    double acc = 0.0;
    for (int m = 0; m < er.n; ++m) {
      const float lp = er.logits[m][(size_t)r * ld + j] - (s_max[m] + s_lse[m]);
      acc += (mode == 0) ? (double)expf(lp) : (double)lp;
    }
    acc /= er.n;
    o[j] = (mode == 0) ? logf((float)acc) : (float)acc;
  }
  (void)inv_n;
}

// ---------------------------------------------------------------------------------------
// Beam selection for one sentence and one step, all on the device.  Replaces
// Decoder<T>::ExpandHypothesis (src/decoder.h:355-480) and, on a sentence's last step,
// Decoder<T>::FinishCurrentHypotheses (src/decoder.h:502-525).
// Candidate order = (score desc, beam asc, vocab asc), the defined order of the reference's
// global heap.  START is skipped, EOS goes to the finished list without using a slot.
struct BeamState {
  int32_t* tok;        // [R] current token of each slot
  float* score;        // [R]
  int32_t* parent;     // [R] parent slot chosen by the last selection
  int32_t* hist_tok;   // [Tcap][R]
  int32_t* hist_parent;// [Tcap][R]
  int32_t* fin_t;      // [B][fin_cap] step at which EOS was produced
  int32_t* fin_b;      // [B][fin_cap] slot whose history the hypothesis continues
  float* fin_score;    // [B][fin_cap]
  int32_t* fin_n;      // [B]
  int fin_cap;
  int R;
};
struct TraceDev {
  int32_t* cand_tok; float* cand_logp; int32_t* surv_tok; int32_t* surv_parent; float* surv_score; float* final_logp;
  const int32_t* force_tok; const int32_t* force_parent; const float* force_score;
  int Tm;
  float* pt;                 // [n][Tm+1][k] attention centre of every forward (member 0), or null
  float* gold_logp;          // [n][Tm][k] log-probability of the forced token of every slot (scoring)
  const float* logits; int ld_logits; const float* row_stats;   // what gold_logp is computed from
  TopkRefine rf;             // set when the logits are one-product values: the forced token's logit is recomputed accurately
};
// grid = active sentences, block = 256, dynamic smem = k*kk*24 + 8 bytes
static __global__ void __launch_bounds__(256) beam_select_kernel(BeamState bs, const int32_t* __restrict__ cand_idx, const float* __restrict__ cand_logp,
                                   const float* __restrict__ eos_logp, const int32_t* __restrict__ steps,
                                   const int32_t* __restrict__ orig, int t, int k, float penalty, float diversity,
                                   TraceDev tr) {
  tc::pdl_launch_dependents();   // see gemm_tc.cuh: the next kernel of the step may start its prologue
  tc::pdl_wait();                // nothing below runs before the previous kernel's results are visible
  extern __shared__ unsigned char smraw[];
  const int kk = k + 1;
  const int ncap = k * kk;
  float* cs = reinterpret_cast<float*>(smraw);   // candidate score
  int* cb = reinterpret_cast<int*>(cs + ncap);   // beam
  int* cv = cb + ncap;                           // vocab id
  int* order = cv + ncap;                        // sorted position -> candidate
  unsigned long long* key = reinterpret_cast<unsigned long long*>(order + ncap);  // sortable (score, beam, vocab)
  const int sent = blockIdx.x;
  const int T = steps[sent];
  const int r0 = sent * k;
  const int osent = orig[sent];
  if (t > T) return;
  if (t == T) {
    if (threadIdx.x == 0) {
      int n = bs.fin_n[sent];
      for (int b = 0; b < k; ++b) {
        const float lp = eos_logp[r0 + b];
        if (tr.final_logp) tr.final_logp[(size_t)osent * k + b] = lp;
        if (n < bs.fin_cap) {
          bs.fin_t[(size_t)sent * bs.fin_cap + n] = t;
          bs.fin_b[(size_t)sent * bs.fin_cap + n] = b;
          bs.fin_score[(size_t)sent * bs.fin_cap + n] = bs.score[r0 + b] + (lp + penalty);
          ++n;
        }
      }
      bs.fin_n[sent] = n;
    }
    return;
  }
  const int cols = (t == 0) ? 1 : k;
  const int n = cols * kk;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const int b = c / kk, q = c - b * kk;
    const float lp = cand_logp[(size_t)(r0 + b) * kk + q];
    const int v = cand_idx[(size_t)(r0 + b) * kk + q];
    const float rank_penalty = (float)(q + 1) * diversity;
    cs[c] = (lp + bs.score[r0 + b]) - rank_penalty;
    cb[c] = b; cv[c] = v;
    order[c] = c;  // overwritten by the ranking below; keeps every entry valid even for NaN scores
    {
      // one 64-bit key, larger = earlier: score descending, then beam ascending, then vocabulary id ascending
      const unsigned int fb = __float_as_uint(cs[c]);
      const unsigned int ord = (fb & 0x80000000u) ? ~fb : (fb | 0x80000000u);
      const unsigned int low = 0xFFFFFFFFu - (((unsigned int)b << 24) | ((unsigned int)v & 0xFFFFFFu));
      key[c] = ((unsigned long long)ord << 32) | low;
    }
    if (tr.cand_tok) {
      const size_t off = ((((size_t)osent * tr.Tm + t) * k + b) * kk) + q;
      tr.cand_tok[off] = v; tr.cand_logp[off] = lp;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const unsigned long long kc = key[c];
    int pos = 0;
    for (int d = 0; d < n; ++d) pos += (key[d] > kc) ? 1 : 0;
    order[pos] = c;
  }
  __syncthreads();
  // The walk itself is serial (START is skipped, EOS leaves the beam without taking a slot), but it
  // only touches shared memory; every global write happens afterwards, one thread per slot.
  __shared__ int s_ntok[kMaxBeam + 1], s_npar[kMaxBeam + 1];
  __shared__ float s_nscore[kMaxBeam + 1];
  if (threadIdx.x == 0) {
    int ns = 0;
    int nf = bs.fin_n[sent];
    for (int p = 0; p < n && ns < k; ++p) {
      const int c = order[p];
      const int v = cv[c];
      if (v == kStart || v < 0) continue;
      if (v == kEos) {
        if (nf < bs.fin_cap) {
          bs.fin_t[(size_t)sent * bs.fin_cap + nf] = t;
          bs.fin_b[(size_t)sent * bs.fin_cap + nf] = cb[c];
          bs.fin_score[(size_t)sent * bs.fin_cap + nf] = cs[c] + penalty;
          ++nf;
        }
        continue;
      }
      s_ntok[ns] = v; s_npar[ns] = cb[c]; s_nscore[ns] = cs[c] + penalty;
      ++ns;
    }
    for (; ns < k; ++ns) { s_ntok[ns] = kUnk; s_npar[ns] = 0; s_nscore[ns] = kDeadScore; }
    bs.fin_n[sent] = nf;
  }
  // Scoring (force-decoding): log-probability of the forced token of every slot under its parent's row.
  // With one-product logits the token's logit is recomputed from both planes of both operands, like the
  // candidates in the softmax kernel; one warp per slot.
  __shared__ float s_gold[kMaxBeam + 1];
  if (tr.force_tok && tr.gold_logp && tr.logits) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = warp; b < k; b += (int)(blockDim.x >> 5)) {
      const size_t off = ((size_t)osent * tr.Tm + t) * k + b;
      const int npar = tr.force_parent[off];
      const int prow = r0 + (npar >= 0 && npar < k ? npar : 0);
      const int gt = tr.force_tok[off] >= 0 ? tr.force_tok[off] : 0;
      float zv = 0.f;
      if (tr.rf.a0) {
        const __half* a0 = tr.rf.a0 + (size_t)prow * tr.rf.lda;
        const __half* a1 = tr.rf.a1 + (size_t)prow * tr.rf.lda;
        const __half* w0 = tr.rf.b0 + (size_t)gt * tr.rf.ldb;
        const __half* w1 = tr.rf.b1 + (size_t)gt * tr.rf.ldb;
        float acc = 0.f;
        for (int j = lane; j < tr.rf.K; j += 32) {
          const float a = fmaf(__half2float(a1[j]), kPairInv, __half2float(a0[j]));
          const float w = fmaf(__half2float(w1[j]), kPairInv, __half2float(w0[j]));
          acc = fmaf(a, w, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        zv = acc + (tr.rf.bias ? tr.rf.bias[gt] : 0.f);
      } else if (lane == 0) {
        zv = tr.logits[(size_t)prow * tr.ld_logits + gt];
      }
      if (lane == 0) s_gold[b] = (zv - tr.row_stats[2 * prow]) - tr.row_stats[2 * prow + 1];
    }
  }
  __syncthreads();
  if (threadIdx.x < k) {
    const int b = threadIdx.x;
    int ntok = s_ntok[b], npar = s_npar[b];
    float nscore = s_nscore[b];
    const size_t off = ((size_t)osent * tr.Tm + t) * k + b;
    if (tr.surv_tok) { tr.surv_tok[off] = ntok; tr.surv_parent[off] = npar; tr.surv_score[off] = nscore; }
    if (tr.force_tok) {
      ntok = tr.force_tok[off]; npar = tr.force_parent[off]; nscore = tr.force_score[off];
      if (tr.gold_logp && tr.logits) tr.gold_logp[off] = s_gold[b];
    }
    bs.tok[r0 + b] = ntok; bs.parent[r0 + b] = npar; bs.score[r0 + b] = nscore;
    bs.hist_tok[(size_t)t * bs.R + r0 + b] = ntok;
    bs.hist_parent[(size_t)t * bs.R + r0 + b] = npar;
  }
}

// ---------------------------------------------------------------------------------------
// Final scoring and n-best extraction for one sentence.  Replaces
// Decoder<T>::ObtainOneBestHypothesis (src/decoder.h:703-859) up to the numeric result:
// length normalisation (:708-713), coverage penalty (:716-759), minimum-ratio filter
// (:762-765), n-best with strictly-greater replacement (:766-773), then the hypothesis is
// rebuilt from the back-pointers.
struct FinalizeArgs {
  BeamState bs;
  const int32_t* steps;     // [B]
  const int32_t* src_len;   // [B]
  const int32_t* orig;      // [B] caller's sentence index
  const float* rec_align;   // [Tcap][R][win] or null
  const int32_t* rec_lo;    // [Tcap][R]
  const int32_t* rec_vit;   // [Tcap][R]
  float* fin_final;         // [B][fin_cap] scratch: final score, -inf if filtered
  int win;
  int k;
  int nbest;
  int max_len;
  int max_src;
  float lp_alpha, cp_beta, min_ratio;
  int32_t* out_tok;   // [n][nbest][max_len]
  int32_t* out_len;   // [n][nbest]
  float* out_score;   // [n][nbest]
  int32_t* out_vit;   // [n][nbest][max_len] or null
  float* out_align;   // [n][nbest][max_len][max_src] or null
};
// grid = sentences, block = 128, dynamic smem = 4 warps * (max_src floats + max_len ints)
static __global__ void __launch_bounds__(128) finalize_kernel(FinalizeArgs a) {
  extern __shared__ unsigned char smraw[];
  const int sent = blockIdx.x;
  const int S = a.src_len[sent];
  const int k = a.k, R = a.bs.R;
  const int nf = a.bs.fin_n[sent];
  const int r0 = sent * k;
  const int32_t* ft = a.bs.fin_t + (size_t)sent * a.bs.fin_cap;
  const int32_t* fb = a.bs.fin_b + (size_t)sent * a.bs.fin_cap;
  const float* fs = a.bs.fin_score + (size_t)sent * a.bs.fin_cap;
  float* ff = a.fin_final + (size_t)sent * a.bs.fin_cap;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* cov = reinterpret_cast<float*>(smraw) + warp * a.max_src;
  int* path = reinterpret_cast<int*>(reinterpret_cast<float*>(smraw) + 4 * a.max_src) + warp * a.max_len;
  const bool tracked = a.rec_align != nullptr;

  if (!tracked || a.cp_beta == 0.f) {
    for (int q = threadIdx.x; q < nf; q += blockDim.x) {
      const int n = ft[q] + 2;
      float sc = fs[q];
      if (0 != a.lp_alpha) {
        const float lp = powf((float)(5 + n), a.lp_alpha) / powf((float)(5 + 1), a.lp_alpha);
        sc /= lp;
      }
      if (0 != a.cp_beta) {
        // alignments are all zero when they are not tracked: every position becomes the
        // uniform row (0 + 0.01) / sum; same loops as the reference, in fp32
        float sum = 0.f;
        const float one = (float)(0.0f + 0.01);
        for (int s = 0; s < S; ++s) sum += one;
        const float u = one / sum;
        float c1 = 0.f;
        for (int j = 1; j < n - 1; ++j) c1 += u;
        float cp = 0.f;
        const float lg = logf(fminf(c1, 1.0f));
        for (int s = 0; s < S; ++s) cp += lg;
        cp *= a.cp_beta;
        if (cp < -20) cp = -20;
        sc += cp;
      }
      const float ratio = ((float)n) / S;
      ff[q] = (ratio > a.min_ratio) ? sc : -INFINITY;
    }
  } else {
    // tracked alignments: one warp per hypothesis, lanes over source positions
    for (int q = warp; q < nf; q += 4) {
      const int t = ft[q];
      const int n = t + 2;
      float sc = fs[q];
      if (0 != a.lp_alpha) {
        const float lp = powf((float)(5 + n), a.lp_alpha) / powf((float)(5 + 1), a.lp_alpha);
        sc /= lp;
      }
      // path[p] = slot that ran the forward producing position p (p = 1 .. t+1)
      if (lane == 0) {
        int slot = fb[q];
        path[t + 1] = slot;
        for (int tt = t - 1; tt >= 0; --tt) {
          const int par = a.bs.hist_parent[(size_t)tt * R + r0 + slot];
          path[tt + 1] = par;
          slot = par;
        }
      }
      __syncwarp();
      for (int s = lane; s < S; s += 32) cov[s] = 0.f;
      for (int p = 2; p <= n - 1; ++p) {
        const int step = p - 1;
        const size_t row = (size_t)step * R + r0 + path[p];
        const int lo = a.rec_lo[row];
        float part = 0.f;
        for (int s = lane; s < S; s += 32) {
          const int w = s - lo;
          const float v = ((w >= 0 && w < a.win) ? a.rec_align[row * a.win + w] : 0.f) + 0.01f;
          part += v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        for (int s = lane; s < S; s += 32) {
          const int w = s - lo;
          const float v = ((w >= 0 && w < a.win) ? a.rec_align[row * a.win + w] : 0.f) + 0.01f;
          cov[s] += v / part;
        }
      }
      __syncwarp();
      float cp = 0.f;
      for (int s = lane; s < S; s += 32) cp += logf(fminf(cov[s], 1.0f));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cp += __shfl_xor_sync(0xffffffffu, cp, o);
      cp *= a.cp_beta;
      if (cp < -20) cp = -20;
      sc += cp;
      const float ratio = ((float)n) / S;
      if (lane == 0) ff[q] = (ratio > a.min_ratio) ? sc : -INFINITY;
      __syncwarp();
    }
  }
  __syncthreads();
  // n-best in creation order with strictly-greater replacement, then descending
  __shared__ int s_best[32];
  __shared__ int s_nb;
  if (threadIdx.x == 0) {
    int nb = 0;
    for (int q = 0; q < nf; ++q) {
      const float sc = ff[q];
      if (sc == -INFINITY) continue;
      if (nb < a.nbest) s_best[nb++] = q;
      else {
        int worst = 0;
        for (int z = 1; z < nb; ++z)
          if (ff[s_best[z]] < ff[s_best[worst]] || (ff[s_best[z]] == ff[s_best[worst]] && s_best[z] > s_best[worst])) worst = z;
        if (ff[s_best[worst]] < sc) s_best[worst] = q;
      }
    }
    for (int i = 1; i < nb; ++i) {  // insertion sort: score desc, creation order asc
      const int q = s_best[i];
      int j = i - 1;
      while (j >= 0 && (ff[s_best[j]] < ff[q] || (ff[s_best[j]] == ff[q] && s_best[j] > q))) { s_best[j + 1] = s_best[j]; --j; }
      s_best[j + 1] = q;
    }
    s_nb = nb;
  }
  __syncthreads();
  const int osent = a.orig[sent];
  for (int q = warp; q < a.nbest; q += 4) {
    const size_t ob = (size_t)osent * a.nbest + q;
    // positions past the hypothesis (all of them when fewer than nbest passed the filter) read START / "no
    // alignment", so that a result does not carry what an earlier decode left in the buffer
    const int n_used = (q >= s_nb) ? 0 : ft[s_best[q]] + 2;
    for (int j = n_used + lane; j < a.max_len; j += 32) {
      a.out_tok[ob * a.max_len + j] = kStart;
      if (a.out_vit) a.out_vit[ob * a.max_len + j] = -20;
    }
    if (a.out_align)
      for (size_t j = (size_t)n_used * a.max_src + lane; j < (size_t)a.max_len * a.max_src; j += 32)
        a.out_align[ob * a.max_len * a.max_src + j] = 0.f;
    if (q >= s_nb) {
      if (lane == 0) { a.out_len[ob] = 0; a.out_score[ob] = 0.f; }
      continue;
    }
    const int h = s_best[q];
    const int t = ft[h];
    const int n = t + 2;
    if (lane == 0) {
      a.out_len[ob] = n;
      a.out_score[ob] = ff[h];
      int32_t* ot = a.out_tok + ob * a.max_len;
      int32_t* ov = a.out_vit ? a.out_vit + ob * a.max_len : nullptr;
      ot[0] = kStart; ot[t + 1] = kEos;
      int slot = fb[h];
      path[t + 1] = slot;
      if (ov) { ov[0] = -20; ov[t + 1] = a.rec_vit ? a.rec_vit[(size_t)t * R + r0 + slot] : -1; }
      for (int tt = t - 1; tt >= 0; --tt) {
        ot[tt + 1] = a.bs.hist_tok[(size_t)tt * R + r0 + slot];
        const int par = a.bs.hist_parent[(size_t)tt * R + r0 + slot];
        if (ov) ov[tt + 1] = a.rec_vit ? a.rec_vit[(size_t)tt * R + r0 + par] : -1;
        path[tt + 1] = par;
        slot = par;
      }
    }
    __syncwarp();
    if (a.out_align && tracked) {
      float* oa = a.out_align + ob * a.max_len * a.max_src;
      for (int p = 0; p < n; ++p) {
        float part = 0.f;
        const bool norm = (a.cp_beta != 0.f) && p >= 2;
        size_t row = 0; int lo = 0;
        if (p >= 1) { row = (size_t)(p - 1) * R + r0 + path[p]; lo = a.rec_lo[row]; }
        if (norm) {
          for (int s = lane; s < S; s += 32) {
            const int w = s - lo;
            part += ((w >= 0 && w < a.win) ? a.rec_align[row * a.win + w] : 0.f) + 0.01f;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        }
        for (int s = lane; s < a.max_src; s += 32) {
          float v = 0.f;
          if (p >= 1 && s < S) {
            const int w = s - lo;
            v = (w >= 0 && w < a.win) ? a.rec_align[row * a.win + w] : 0.f;
            if (norm) v = (v + 0.01f) / part;
          }
          oa[(size_t)p * a.max_src + s] = v;
        }
      }
    }
    __syncwarp();
  }
}

}  // namespace linmt

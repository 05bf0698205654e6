// gemm_simt.cuh -- fp32 CUDA-core GEMM with fused epilogues.
//
// C[M][N] = A[M][K] . Wt[N][K]^T, both operands K-contiguous (Wt rows ldw apart).  A may be the concatenation
// along K of up to three row-major buffers (x | h_prev | htilde_prev), which is how one
// launch replaces the reference's 8 or 12 separate cublasSgemm calls per LSTM node
// (src/node_input_to_hidden.h:297-556, src/node_hidden_to_hidden.h:248-386).
// Exact fp32 (FFMA) arithmetic: this is the path used when fp32-exact parity is wanted and
// the check against which the tensor-core kernels are validated.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace linmt {

struct ASegs {
  const float* ptr[3];  // row-major, leading dimension ld[i]
  int ld[3];
  int nseg;
  int seg_k;  // K extent of every segment (multiple of 16)
};

__device__ __forceinline__ float sigmoidf_ref(float x) { return 1.0f / (1.0f + expf(-1.0f * x)); }

// ---- epilogues: called once per (row, group of 4 consecutive columns) -------------------

// LSTM cell update.  Columns are gate-interleaved: column 4*j+g holds gate g of hidden unit
// j with g = 0:i 1:f 2:c~ 3:o.  Replaces ForwardSigmoidKernel/ForwardTanhKernel/
// ForwardCTKernel/ForwardHTKernel (src/deep_rnn_kernel.cu:78-136, src/deep_rnn_kernel.h:63-99)
// and, through row_len/pos, the encoder's per-sentence length handling.
struct EpiLstm {
  const float* bias;    // [N] interleaved
  const float* c_prev;  // [M][ld]
  const float* h_prev;  // [M][ld], only read for rows that are past their length
  float* c_out;         // [M][ld]
  float* h_out;         // [M][ld]
  float* h_out2;        // optional second copy of h (encoder top states), element (row, j) at
  long long h2_row_stride;  //   h_out2[row * h2_row_stride + j]
  const int* row_len;   // optional: row is active iff pos < row_len[row]
  int pos;
  int ld;
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    const int j = col0 >> 2;
    const size_t idx = (size_t)row * ld + j;
    const bool active = (row_len == nullptr) || (pos < row_len[row]);
    float c, h;
    if (active) {
      const float4 b = *reinterpret_cast<const float4*>(bias + col0);
      const float gi = sigmoidf_ref(v[0] + b.x);
      const float gf = sigmoidf_ref(v[1] + b.y);
      const float gg = tanhf(v[2] + b.z);
      const float go = sigmoidf_ref(v[3] + b.w);
      c = gf * c_prev[idx] + gi * gg;
      h = go * tanhf(c);
      if (h_out2) h_out2[(size_t)row * h2_row_stride + j] = h;
    } else {
      c = c_prev[idx];
      h = h_prev[idx];
    }
    c_out[idx] = c;
    h_out[idx] = h;
  }
};

// out = tanh(acc + bias): the attentional hidden state
// (TanhAttentionForwardKernel, src/deep_rnn_kernel.h:1281-1287).
struct EpiBiasTanh {
  const float* bias;
  float* out;
  int ld;
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    const float4 b = *reinterpret_cast<const float4*>(bias + col0);
    float4 o;
    o.x = tanhf(v[0] + b.x); o.y = tanhf(v[1] + b.y); o.z = tanhf(v[2] + b.z); o.w = tanhf(v[3] + b.w);
    *reinterpret_cast<float4*>(out + (size_t)row * ld + col0) = o;
  }
};

// Attention projections in one product: columns < split get tanh (W_p h, TanhKernel
// src/deep_rnn_kernel.cu:277-289), the rest are plain (W_a^T h, src/layer_attention.h:327).
struct EpiAttnProj {
  float* out;
  int ld;
  int split;
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    float4 o;
    if (col0 < split) { o.x = tanhf(v[0]); o.y = tanhf(v[1]); o.z = tanhf(v[2]); o.w = tanhf(v[3]); }
    else { o.x = v[0]; o.y = v[1]; o.z = v[2]; o.w = v[3]; }
    *reinterpret_cast<float4*>(out + (size_t)row * ld + col0) = o;
  }
};

// out = acc + bias: the logits (MatrixBiasKernel, src/deep_rnn_kernel.h:524-530).
struct EpiBias {
  const float* bias;  // may be null
  float* out;
  int ld;
  __device__ __forceinline__ void operator()(int row, int col0, const float* v) const {
    float4 o = make_float4(v[0], v[1], v[2], v[3]);
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + col0);
      o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)row * ld + col0) = o;
  }
};

// ---- kernel -----------------------------------------------------------------------------
// BM x BN block tile, BK = 16, 256 threads; each thread owns RM x CN groups of 4x4 outputs
// (rows ty*4 + i*(BM/RM), columns tx*4 + j*(BN/CN)).
template <int BM, int BN, class Epi>
__global__ void __launch_bounds__(256) gemm_simt_kernel(ASegs a, const float* __restrict__ wt, int ldw, int M, int N, int K, Epi epi) {
  constexpr int BK = 16;
  constexpr int TXN = 16;           // threads along N
  constexpr int TYN = 16;           // threads along M
  constexpr int CN = BN / (TXN * 4);
  constexpr int RM = BM / (TYN * 4);
  constexpr int PADM = BM + 4, PADN = BN + 4;
  __shared__ __align__(16) float As[2][BK][PADM];
  __shared__ __align__(16) float Bs[2][BK][PADN];

  const int tid = threadIdx.x;
  const int tx = tid % TXN, ty = tid / TXN;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;  // M fastest: the CTAs sharing a weight tile run together

  constexpr int A_F4 = BM * BK / 4 / 256;  // float4 loads per thread
  constexpr int B_F4 = BN * BK / 4 / 256;
  float4 ra[A_F4], rb[B_F4];

  auto load_tiles = [&](int kt) {
    const int k0 = kt * BK;
    const int seg = k0 / a.seg_k;
    const int ks = k0 - seg * a.seg_k;
    const float* ap = a.ptr[seg];
    const int lda = a.ld[seg];
#pragma unroll
    for (int i = 0; i < A_F4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 2, kq = idx & 3;
      const int gr = m0 + row;
      ra[i] = (gr < M) ? *reinterpret_cast<const float4*>(ap + (size_t)gr * lda + ks + kq * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < B_F4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 2, kq = idx & 3;
      rb[i] = *reinterpret_cast<const float4*>(wt + (size_t)(n0 + row) * ldw + k0 + kq * 4);
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_F4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 2, kq = idx & 3;
      As[buf][kq * 4 + 0][row] = ra[i].x; As[buf][kq * 4 + 1][row] = ra[i].y;
      As[buf][kq * 4 + 2][row] = ra[i].z; As[buf][kq * 4 + 3][row] = ra[i].w;
    }
#pragma unroll
    for (int i = 0; i < B_F4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 2, kq = idx & 3;
      Bs[buf][kq * 4 + 0][row] = rb[i].x; Bs[buf][kq * 4 + 1][row] = rb[i].y;
      Bs[buf][kq * 4 + 2][row] = rb[i].z; Bs[buf][kq * 4 + 3][row] = rb[i].w;
    }
  };

  float acc[RM * 4][CN * 4];
#pragma unroll
  for (int i = 0; i < RM * 4; ++i)
#pragma unroll
    for (int j = 0; j < CN * 4; ++j) acc[i][j] = 0.f;

  const int nkt = K / BK;
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  for (int kt = 0; kt < nkt; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < nkt) load_tiles(kt + 1);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[RM * 4], bv[CN * 4];
#pragma unroll
      for (int i = 0; i < RM; ++i) {
        const float4 t = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4 + i * (BM / RM)]);
        av[i * 4 + 0] = t.x; av[i * 4 + 1] = t.y; av[i * 4 + 2] = t.z; av[i * 4 + 3] = t.w;
      }
#pragma unroll
      for (int j = 0; j < CN; ++j) {
        const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4 + j * (BN / CN)]);
        bv[j * 4 + 0] = t.x; bv[j * 4 + 1] = t.y; bv[j * 4 + 2] = t.z; bv[j * 4 + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < RM * 4; ++i)
#pragma unroll
        for (int j = 0; j < CN * 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kt + 1 < nkt) {
      store_tiles(buf ^ 1);
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int row = m0 + ty * 4 + i * (BM / RM) + ii;
      if (row < M) {
#pragma unroll
        for (int j = 0; j < CN; ++j) {
          const int col0 = n0 + tx * 4 + j * (BN / CN);
          epi(row, col0, &acc[i * 4 + ii][j * 4]);
        }
      }
    }
}

template <int BM, int BN, class Epi>
inline cudaError_t launch_gemm_simt(const ASegs& a, const float* wt, int ldw, int M, int N, int K, const Epi& epi, cudaStream_t st) {
  dim3 grid((M + BM - 1) / BM, N / BN);
  gemm_simt_kernel<BM, BN, Epi><<<grid, 256, 0, st>>>(a, wt, ldw, M, N, K, epi);
  return cudaGetLastError();
}

// Picks the tile so that the grid covers the 148 SMs: large tiles only when they still give
// at least one CTA per SM.
template <class Epi>
inline cudaError_t gemm_simt(const ASegs& a, const float* wt, int ldw, int M, int N, int K, const Epi& epi, cudaStream_t st) {
  const long big = (long)(N / 128) * ((M + 127) / 128);
  if (N % 128 == 0 && big >= 148) return launch_gemm_simt<128, 128, Epi>(a, wt, ldw, M, N, K, epi, st);
  return launch_gemm_simt<64, 64, Epi>(a, wt, ldw, M, N, K, epi, st);
}

}  // namespace linmt

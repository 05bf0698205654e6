// linmt_oracle.cpp -- CPU restatement of LiNMT's beam-search decoding math.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA engine: it may be
// loaded by the tests, by the smoke check and by the benchmark's CPU-baseline legs, and by
// nothing else.  The product library never links, loads or calls it.
//
// PARITY UNPINNED: the reference project ships no tests, golden vectors or trained model,
// and it cannot be built without Boost and a GPU, so this restatement is pinned by source
// reading only (each function cites the reference file:line it follows) and by an
// independent numpy/float64 restatement kept next to it.
//
// Arithmetic is IEEE fp32 like the reference (src/utility_cu.h:42 `typedef float
// precision`); every dense product is a plain k-ascending sum per output element, so the
// result does not depend on how rows are grouped (one sentence at a time == batched).
//
// Layout of a weight blob = the reference's device memory after LoadWeights
// (src/deep_rnn.h:1878-1969): every rows x cols matrix is column-major
// (src/utility_cu.h:37 IDX2C), i.e. a weight "out x in" is stored [in][out].
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------------------------------
// bf16 rounding (round-to-nearest-even) used by the reduced-precision mode.
inline float bf16_round(float x) {
  uint32_t u;
  std::memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  uint32_t r = 0x7fffu + ((u >> 16) & 1u);
  u = (u + r) & 0xffff0000u;
  float y;
  std::memcpy(&y, &u, 4);
  return y;
}

// ---------------------------------------------------------------------------------------
// Dense product Y[r][n] = sum_k X[r][k] * W[k][n], k ascending, one fused multiply-add per
// term.  Stands in for the reference's cublasSgemm calls (src/utility_cu.h:153-157), which
// compute the same sums in an unspecified order.
#if defined(__AVX512F__)
#define VW 16
#define NVEC 4
#define RBLK 6
#else
#define VW 8
#define NVEC 2
#define RBLK 4
#endif
typedef float vf __attribute__((vector_size(VW * 4)));

static inline vf vload(const float* p) { vf v; std::memcpy(&v, p, sizeof(vf)); return v; }
static inline void vstore(float* p, vf v) { std::memcpy(p, &v, sizeof(vf)); }
static inline vf vsplat(float a) {
  vf v;
  for (int i = 0; i < VW; ++i) v[i] = a;
  return v;
}
// a * b + c on vector types contracts to one fused multiply-add per lane (-ffp-contract=fast,
// the GNU default); the scalar tails use fmaf so every path rounds identically.
static inline vf vfma(vf a, vf b, vf c) { return a * b + c; }

template <int RB>
static void gemm_block(float* Y, const float* X, const float* W, int K, int N, int ldx, int ldy,
                       int r0, int n0) {
  vf acc[RB][NVEC];
  for (int r = 0; r < RB; ++r)
    for (int v = 0; v < NVEC; ++v) acc[r][v] = vsplat(0.f);
  for (int k = 0; k < K; ++k) {
    const float* wrow = W + (size_t)k * N + n0;
    vf w[NVEC];
    for (int v = 0; v < NVEC; ++v) w[v] = vload(wrow + v * VW);
    for (int r = 0; r < RB; ++r) {
      vf a = vsplat(X[(size_t)(r0 + r) * ldx + k]);
      for (int v = 0; v < NVEC; ++v) acc[r][v] = vfma(a, w[v], acc[r][v]);
    }
  }
  for (int r = 0; r < RB; ++r)
    for (int v = 0; v < NVEC; ++v) vstore(Y + (size_t)(r0 + r) * ldy + n0 + v * VW, acc[r][v]);
}

#ifdef LINMT_ORACLE_EIGEN
}  // namespace
// Baseline-timing build only: the dense products go through the Eigen headers the reference project ships
// (package/eigen.tar.gz, Eigen 3.2.92), the library its host code is written with (src/decoder.h:128-199),
// with Eigen's own OpenMP threading.  Eigen blocks and reorders the sums, so this build's numbers agree with
// the canonical build only to fp32 rounding: it is timed beside the GPU, never used as the checker.
#include <Eigen/Dense>
namespace {
static void gemm(float* Y, const float* X, const float* W, int R, int K, int N, int ldx, int ldy) {
  typedef Eigen::Matrix<float, Eigen::Dynamic, Eigen::Dynamic, Eigen::RowMajor> Mat;
  Eigen::Map<const Mat, 0, Eigen::OuterStride<> > x(X, R, K, Eigen::OuterStride<>(ldx));
  Eigen::Map<const Mat> w(W, K, N);
  Eigen::Map<Mat, 0, Eigen::OuterStride<> > y(Y, R, N, Eigen::OuterStride<>(ldy));
  y.noalias() = x * w;
}
#else
static void gemm(float* Y, const float* X, const float* W, int R, int K, int N, int ldx, int ldy) {
  const int CB = VW * NVEC;
  const int ncb = N / CB;
#pragma omp parallel for schedule(dynamic, 1)
  for (int cb = 0; cb < ncb; ++cb) {
    int n0 = cb * CB;
    int r0 = 0;
    for (; r0 + RBLK <= R; r0 += RBLK) gemm_block<RBLK>(Y, X, W, K, N, ldx, ldy, r0, n0);
    for (; r0 < R; ++r0) gemm_block<1>(Y, X, W, K, N, ldx, ldy, r0, n0);
  }
  // column tail
  const int nt = ncb * CB;
  if (nt < N) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; ++r) {
      for (int n = nt; n < N; ++n) {
        float acc = 0.f;
        for (int k = 0; k < K; ++k) acc = __builtin_fmaf(X[(size_t)r * ldx + k], W[(size_t)k * N + n], acc);
        Y[(size_t)r * ldy + n] = acc;
      }
    }
  }
}
#endif

// ---------------------------------------------------------------------------------------
// Model view over a weight blob.
struct LstmW {
  const float *Whi, *bi, *Whf, *bf, *Whc, *bc, *Who, *bo, *emb, *Mi, *Mf, *Mo, *Mc;
  const float *Qi, *Qf, *Qo, *Qc;
};
struct Model {
  int L, H, V, Vs, feed;
  std::vector<LstmW> src, tgt;
  const float *Wa, *Wp, *vp, *bout, *Wc1, *Wc2, *D, *bd;
  std::vector<float> rounded;  // bf16-rounded copy of the blob when precision = 1
};

// Order of matrices: src/layer_input_to_hidden.h:1378-1423,
// src/layer_hidden_to_hidden.h:953-979, src/layer_attention.h:1246-1260,
// src/layer_loss.h:1191-1196, sequence src/deep_rnn.h:1878-1969.
static size_t blob_floats(int L, int H, int V, int Vs, int feed) {
  size_t hh = (size_t)H * H, n = 0;
  n += 8 * hh + 4 * (size_t)H + (size_t)H * Vs;
  n += (size_t)(L - 1) * (8 * hh + 4 * (size_t)H);
  n += 8 * hh + 4 * (size_t)H + (size_t)H * V + (feed ? 4 * hh : 0);
  n += (size_t)(L - 1) * (8 * hh + 4 * (size_t)H);
  n += 4 * hh + 2 * (size_t)H;
  n += (size_t)V * H + V;
  return n;
}

static bool parse_model(Model& m, const int32_t* desc, const float* blob, size_t n_floats, int precision) {
  m.L = desc[0]; m.H = desc[1]; m.V = desc[2]; m.Vs = desc[3]; m.feed = desc[4];
  if (m.L < 1 || m.H < 1 || m.V < 3 || m.Vs < 1) return false;
  if (blob_floats(m.L, m.H, m.V, m.Vs, m.feed) != n_floats) return false;
  const float* p = blob;
  const size_t hh = (size_t)m.H * m.H;
  const int H = m.H;
  std::vector<std::pair<size_t, size_t>> mats;  // (offset, size) of GEMM operand matrices
  auto take = [&](size_t n, bool is_mat) {
    const float* q = p;
    if (is_mat) mats.push_back({(size_t)(p - blob), n});
    p += n;
    return q;
  };
  auto lstm = [&](LstmW& w, bool first, int vocab, bool feed) {
    w.Whi = take(hh, true); w.bi = take(H, false);
    w.Whf = take(hh, true); w.bf = take(H, false);
    w.Whc = take(hh, true); w.bc = take(H, false);
    w.Who = take(hh, true); w.bo = take(H, false);
    w.emb = first ? take((size_t)H * vocab, true) : nullptr;
    w.Mi = take(hh, true); w.Mf = take(hh, true); w.Mo = take(hh, true); w.Mc = take(hh, true);
    w.Qi = w.Qf = w.Qo = w.Qc = nullptr;
    if (feed) { w.Qi = take(hh, true); w.Qf = take(hh, true); w.Qo = take(hh, true); w.Qc = take(hh, true); }
  };
  m.src.resize(m.L); m.tgt.resize(m.L);
  for (int l = 0; l < m.L; ++l) lstm(m.src[l], l == 0, m.Vs, false);
  for (int l = 0; l < m.L; ++l) lstm(m.tgt[l], l == 0, m.V, l == 0 && m.feed);
  m.Wa = take(hh, true); m.Wp = take(hh, true); m.vp = take(H, false); m.bout = take(H, false);
  m.Wc1 = take(hh, true); m.Wc2 = take(hh, true);
  m.D = take((size_t)m.V * H, true); m.bd = take(m.V, false);
  if ((size_t)(p - blob) != n_floats) return false;
  if (precision == 1) {
    // Reduced-precision mode: every matrix that feeds a dense product (and the embedding
    // tables) is rounded to bf16; biases and v_p stay fp32.
    m.rounded.assign(blob, blob + n_floats);
    for (auto& mm : mats) {
      float* q = m.rounded.data() + mm.first;
#pragma omp parallel for schedule(static)
      for (size_t i = 0; i < mm.second; ++i) q[i] = bf16_round(q[i]);
    }
    const ptrdiff_t shift = m.rounded.data() - blob;
    auto fix = [&](const float*& q) { if (q) q += shift; };
    for (auto* vec : {&m.src, &m.tgt})
      for (auto& w : *vec) {
        fix(w.Whi); fix(w.bi); fix(w.Whf); fix(w.bf); fix(w.Whc); fix(w.bc); fix(w.Who); fix(w.bo);
        fix(w.emb); fix(w.Mi); fix(w.Mf); fix(w.Mo); fix(w.Mc); fix(w.Qi); fix(w.Qf); fix(w.Qo); fix(w.Qc);
      }
    fix(m.Wa); fix(m.Wp); fix(m.vp); fix(m.bout); fix(m.Wc1); fix(m.Wc2); fix(m.D); fix(m.bd);
  }
  return true;
}

struct Opts {
  int32_t beam, nbest, attention_mode, attention_d, print_info, precision, ensemble_mode, max_len;
  int32_t max_src, group, threads, reserved;
  float penalty, diversity, lp_alpha, cp_beta, min_ratio;
};

// ---------------------------------------------------------------------------------------
// One LSTM node forward for R rows.
//   src/node_input_to_hidden.h:218-636 (layer 1: M x + W h' [+ Q htilde'] + b)
//   src/node_hidden_to_hidden.h:194-443 (layers >= 2: M h_below + W h' + b)
// Gate kernels: src/deep_rnn_kernel.cu:78-136, src/deep_rnn_kernel.h:63-99.  The "Feed"
// sigmoid is a template whose literals are double (deep_rnn_kernel.h:63-71), the non-feed
// float overload uses expf (deep_rnn_kernel.cu:78-85); both are restated as written.
struct Scratch {
  std::vector<float> t1, t2, t3, gi, gf, gg, go;
  void need(size_t n) {
    if (t1.size() < n) { t1.resize(n); t2.resize(n); t3.resize(n); gi.resize(n); gf.resize(n); gg.resize(n); go.resize(n); }
  }
};

static void lstm_forward(const LstmW& w, int H, int R, const float* x, const float* hprev, const float* cprev,
                         const float* htilde, float* h, float* c, Scratch& s, bool bf16) {
  const size_t n = (size_t)R * H;
  s.need(n);
  const float* Ms[4] = {w.Mi, w.Mf, w.Mc, w.Mo};
  const float* Ws[4] = {w.Whi, w.Whf, w.Whc, w.Who};
  const float* Qs[4] = {w.Qi, w.Qf, w.Qc, w.Qo};
  const float* bs[4] = {w.bi, w.bf, w.bc, w.bo};
  float* outs[4] = {s.gi.data(), s.gf.data(), s.gg.data(), s.go.data()};
  for (int g = 0; g < 4; ++g) {
    gemm(s.t1.data(), x, Ms[g], R, H, H, H, H);
    gemm(s.t2.data(), hprev, Ws[g], R, H, H, H, H);
    if (htilde) gemm(s.t3.data(), htilde, Qs[g], R, H, H, H, H);
    float* o = outs[g];
    const float* b = bs[g];
#pragma omp parallel for schedule(static)
    for (int r = 0; r < R; ++r) {
      for (int j = 0; j < H; ++j) {
        size_t idx = (size_t)r * H + j;
        if (htilde) {
          float v = s.t1[idx] + s.t2[idx] + s.t3[idx] + b[j];
          if (g == 2) o[idx] = tanhf(v);
          else o[idx] = (float)(1.0 / (1.0 + std::exp(-1.0 * (double)v)));
        } else {
          float v = s.t1[idx] + s.t2[idx] + b[j];
          if (g == 2) o[idx] = tanhf(v);
          else o[idx] = 1.0f / (1.0f + expf(-1.0f * v));
        }
      }
    }
  }
#pragma omp parallel for schedule(static)
  for (size_t idx = 0; idx < n; ++idx) {
    float cv = s.gf[idx] * cprev[idx] + s.gi[idx] * s.gg[idx];  // ForwardCTKernel, deep_rnn_kernel.h:92-99
    c[idx] = cv;
    float hv = s.go[idx] * tanhf(cv);                           // ForwardHTKernel, deep_rnn_kernel.cu:121-128
    h[idx] = bf16 ? bf16_round(hv) : hv;
  }
}

// ---------------------------------------------------------------------------------------
// Softmax over the vocabulary, restating OutputdistOverflowPreventionKernel
// (src/deep_rnn_kernel.h:352-429): 256 strided partial maxima / sums followed by a
// halving tree, all in fp32, then a divide.
static void softmax_ref(float* p, const float* z, int V) {
  const int TH = 256;
  float buf[TH];
  for (int t = 0; t < TH; ++t) {
    float m = -FLT_MAX;
    for (int i = t; i < V; i += TH) if (m < z[i]) m = z[i];
    buf[t] = m;
  }
  for (int stride = TH / 2; stride > 0; stride >>= 1)
    for (int t = 0; t < stride; ++t) buf[t] = (buf[t] > buf[stride + t]) ? buf[t] : buf[stride + t];
  const float mx = buf[0];
  for (int t = 0; t < TH; ++t) {
    float sum = 0.f;
    for (int i = t; i < V; i += TH) { float e = expf(z[i] - mx); sum += e; p[i] = e; }
    buf[t] = sum;
  }
  for (int stride = TH / 2; stride > 0; stride >>= 1)
    for (int t = 0; t < stride; ++t) buf[t] += buf[stride + t];
  const float sum = buf[0];
  for (int i = 0; i < V; ++i) p[i] = p[i] / sum;
}

// ---------------------------------------------------------------------------------------
// State of one model for one group of sentences (rows = group * beam).
struct ModelRun {
  const Model* m;
  int G, k, R, H, max_src;
  std::vector<int> S;                     // source length per sentence
  std::vector<float> HS;                  // [G][max_src][H] top-layer encoder states by encoder step
  std::vector<std::vector<float>> h, c;   // [L] x [R][H] current states
  std::vector<std::vector<float>> hp, cp; // previous states
  std::vector<float> htilde, htilde_prev; // [R][H]
  std::vector<float> x, tanh1, u, ctx, cat_t1, cat_t2, logits, probs;
  std::vector<float> align;               // [R][max_src] dense alignments of this step
  std::vector<float> pt;                  // [R]
  Scratch scratch;
};

// Encoder: src/deep_rnn.h:1572-1721.  The sentence arrives reversed
// (src/decoder_sentence.cu:68); zero initial states; minibatch 1 per sentence in the
// reference -- here the sentences of a group advance together, each row independent.
static void run_encoder(ModelRun& st, const std::vector<std::vector<int>>& rev_ids, bool bf16,
                        std::vector<std::vector<float>>& fin_h, std::vector<std::vector<float>>& fin_c) {
  const Model& m = *st.m;
  const int G = st.G, H = st.H, L = m.L;
  int Smax = 0;
  for (int i = 0; i < G; ++i) Smax = std::max(Smax, st.S[i]);
  fin_h.assign(L, std::vector<float>((size_t)G * H, 0.f));
  fin_c.assign(L, std::vector<float>((size_t)G * H, 0.f));
  std::vector<float> xa, ha, ca, ho, co;
  std::vector<int> act;
  for (int pos = 0; pos < Smax; ++pos) {
    act.clear();
    for (int i = 0; i < G; ++i) if (pos < st.S[i]) act.push_back(i);
    const int A = (int)act.size();
    xa.resize((size_t)A * H); ha.resize((size_t)A * H); ca.resize((size_t)A * H);
    ho.resize((size_t)A * H); co.resize((size_t)A * H);
    for (int a = 0; a < A; ++a) {
      int tok = rev_ids[act[a]][pos];
      const float* e = m.src[0].emb + (size_t)tok * H;  // SparseLookupKernel, deep_rnn_kernel.h:248-255
      for (int j = 0; j < H; ++j) xa[(size_t)a * H + j] = bf16 ? bf16_round(e[j]) : e[j];
    }
    for (int l = 0; l < L; ++l) {
      for (int a = 0; a < A; ++a) {
        std::memcpy(&ha[(size_t)a * H], &fin_h[l][(size_t)act[a] * H], H * 4);
        std::memcpy(&ca[(size_t)a * H], &fin_c[l][(size_t)act[a] * H], H * 4);
      }
      lstm_forward(m.src[l], H, A, xa.data(), ha.data(), ca.data(), nullptr, ho.data(), co.data(), st.scratch, bf16);
      for (int a = 0; a < A; ++a) {
        std::memcpy(&fin_h[l][(size_t)act[a] * H], &ho[(size_t)a * H], H * 4);
        std::memcpy(&fin_c[l][(size_t)act[a] * H], &co[(size_t)a * H], H * 4);
      }
      xa = ho;  // input of the layer above
    }
    for (int a = 0; a < A; ++a)  // top-layer state of this encoder step, deep_rnn.h:1597-1606
      std::memcpy(&st.HS[((size_t)act[a] * st.max_src + pos) * H], &xa[(size_t)a * H], H * 4);
  }
}

// One decoder forward for the first `rows` rows: src/deep_rnn.h:1754-1836 (LSTM stack),
// src/layer_attention.h:243-483 (attention), src/layer_loss.h:797-883 (softmax).
static void run_forward(ModelRun& st, int rows, int step, const int* tok, const Opts& o, bool want_align) {
  const Model& m = *st.m;
  const int H = st.H, L = m.L, k = st.k, V = m.V;
  const bool bf16 = o.precision == 1;
  for (int r = 0; r < rows; ++r) {
    const float* e = m.tgt[0].emb + (size_t)tok[r] * H;
    for (int j = 0; j < H; ++j) st.x[(size_t)r * H + j] = bf16 ? bf16_round(e[j]) : e[j];
  }
  const float* below = st.x.data();
  for (int l = 0; l < L; ++l) {
    const float* ht = (l == 0 && m.feed && step != 0) ? st.htilde_prev.data() : nullptr;  // node_input_to_hidden.h:325
    lstm_forward(m.tgt[l], H, rows, below, st.hp[l].data(), st.cp[l].data(), ht, st.h[l].data(), st.c[l].data(),
                 st.scratch, bf16);
    below = st.h[l].data();
  }
  const float* htop = st.h[L - 1].data();
  // --- attention ---
  const int D = o.attention_d;
  const float sigma_sq = ((float)D * (float)D) / 4.0f;  // src/layer_attention.h:226 (sigma = D/2)
  if (o.attention_mode == 0) gemm(st.tanh1.data(), htop, m.Wp, rows, H, H, H, H);   // layer_attention.h:272
  if (o.attention_mode != 2) {
    // u = W_a^T h_t (layer_attention.h:327, CUBLAS_OP_T): u[j] = sum_i W_a[i,j] h[i]; W_a[i,j] sits at j*H+i.
    // With W stored [in][out] the transposed product reads it as [out][in]: build it by rows.
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
      for (int j = 0; j < H; ++j) {
        const float* col = m.Wa + (size_t)j * H;
        float acc = 0.f;
        for (int i = 0; i < H; ++i) acc = __builtin_fmaf(col[i], htop[(size_t)r * H + i], acc);
        st.u[(size_t)r * H + j] = acc;
      }
  }
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const int sent = r / k;
    const int S = st.S[sent];
    const float* hs_base = &st.HS[(size_t)sent * st.max_src * H];
    const float* uu = (o.attention_mode == 2) ? &htop[(size_t)r * H] : &st.u[(size_t)r * H];
    float* ctx = &st.ctx[(size_t)r * H];
    float* al = &st.align[(size_t)r * st.max_src];
    for (int s = 0; s < st.max_src; ++s) al[s] = 0.f;
    int lo = 0, hi = S - 1;
    float pt = 0.f;
    if (o.attention_mode == 0) {
      // p_t = S * sigmoid(v_p . tanh(W_p h_t)): TanhKernel (deep_rnn_kernel.cu:277-289), Sgemm m=1
      // (layer_attention.h:282), SigmoidKernel in double (deep_rnn_kernel.h:1075-1080),
      // AlignmentPosKernel (deep_rnn_kernel.h:1085-1090).
      float dot = 0.f;
      for (int j = 0; j < H; ++j) dot = __builtin_fmaf(m.vp[j], tanhf(st.tanh1[(size_t)r * H + j]), dot);
      float sg = (float)(1.0 / (1.0 + std::exp(-1.0 * (double)dot)));
      pt = (float)S * sg;
      // LowerUpperKernel, deep_rnn_kernel.h:1094-1100
      lo = (0 > (int)pt - D) ? 0 : ((int)pt - D);
      hi = ((S - 1) < (int)pt + D) ? (S - 1) : ((int)pt + D);
    }
    st.pt[r] = pt;
    // positions lo..hi; at most 2D+1 of them in local mode (CreateIndicesKernel,
    // deep_rnn_kernel.cu:294-316); position s reads encoder step S-1-s (LoadInHSKernel,
    // deep_rnn_kernel.h:1141-1164).
    const int W = hi - lo + 1;
    std::vector<float> e(W > 0 ? W : 0);
    for (int w = 0; w < W; ++w) {
      const float* hs = hs_base + (size_t)(S - 1 - (lo + w)) * H;
      float acc = 0.f;  // ElemReduceKernelLarge, deep_rnn_kernel.h:1308-1342 (order unspecified there)
      for (int j = 0; j < H; ++j) acc = __builtin_fmaf(hs[j], uu[j], acc);
      e[w] = acc;
    }
    // AlignmentReductionKernel, deep_rnn_kernel.h:1197-1241: max starts at 0.
    float mx = 0.f;
    for (int w = 0; w < W; ++w) if (e[w] > mx) mx = e[w];
    float sum = 0.f;
    for (int w = 0; w < W; ++w) { e[w] = expf(e[w] - mx); sum += e[w]; }
    for (int w = 0; w < W; ++w) {
      float a = e[w];
      if (o.attention_mode == 0) {
        float tmp = expf((-1 * powf(pt - (float)(lo + w), 2.0f)) / (2 * sigma_sq));
        if (0 != sum) a = (a / sum) * tmp;
      } else {
        if (0 != sum) a = a / sum;
      }
      e[w] = a;
      if (want_align) al[lo + w] = a;
    }
    // CreateCTKernel, deep_rnn_kernel.h:1250-1260
    for (int j = 0; j < H; ++j) {
      float acc = 0.f;
      for (int w = 0; w < W; ++w) acc += e[w] * hs_base[(size_t)(S - 1 - (lo + w)) * H + j];
      ctx[j] = bf16 ? bf16_round(acc) : acc;
    }
  }
  // htilde = tanh(W_c1 ctx + W_c2 h_t + b_out): layer_attention.h:441-461,
  // TanhAttentionForwardKernel deep_rnn_kernel.h:1281-1287
  gemm(st.cat_t1.data(), st.ctx.data(), m.Wc1, rows, H, H, H, H);
  gemm(st.cat_t2.data(), htop, m.Wc2, rows, H, H, H, H);
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r)
    for (int j = 0; j < H; ++j) {
      size_t idx = (size_t)r * H + j;
      float v = tanhf(st.cat_t1[idx] + st.cat_t2[idx] + m.bout[j]);
      st.htilde[idx] = bf16 ? bf16_round(v) : v;
    }
  // logits and softmax: layer_loss.h:820 (Sgemm), :827 MatrixBiasKernel, :868 softmax kernel
  gemm(st.logits.data(), st.htilde.data(), m.D, rows, H, V, H, V);
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    float* z = &st.logits[(size_t)r * V];
    for (int v = 0; v < V; ++v) z[v] = z[v] + m.bd[v];
    softmax_ref(&st.probs[(size_t)r * V], z, V);
  }
}

struct Cand { float p; int v; };
struct GCand { float score; int beam; int v; };

struct Hyp {
  std::vector<int> tok;     // START ... EOS
  std::vector<int> vit;     // viterbi alignment per position (position 0 = -20)
  std::vector<float> align; // [len][S] (empty rows = zeros) when alignments are tracked
  float score;
};

}  // namespace

extern "C" {

size_t linmt_oracle_blob_floats(int L, int H, int V, int Vs, int feed) { return blob_floats(L, H, V, Vs, feed); }

int linmt_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Plain dense product for kernel-level checks: Y[R][N] = X[R][K] . W[K][N].
void linmt_oracle_gemm(float* Y, const float* X, const float* W, int R, int K, int N) { gemm(Y, X, W, R, K, N, K, N); }

// Per-row top-(k+1) of a probability row under the canonical rule (value descending,
// index ascending), i.e. what the strict-greater replacement scan of src/decoder.h:401-410
// keeps.  Exposed for kernel-level checks.
void linmt_oracle_softmax_topk(const float* logits, int R, int V, int kk, int32_t* idx, float* logp) {
  std::vector<float> p(V);
  for (int r = 0; r < R; ++r) {
    softmax_ref(p.data(), logits + (size_t)r * V, V);
    std::vector<Cand> top;
    for (int v = 0; v < V; ++v) {
      if ((int)top.size() < kk) top.push_back({p[v], v});
      else {
        int worst = 0;
        for (int i = 1; i < kk; ++i)
          if (top[i].p < top[worst].p || (top[i].p == top[worst].p && top[i].v > top[worst].v)) worst = i;
        if (p[v] > top[worst].p) top[worst] = {p[v], v};
      }
    }
    std::sort(top.begin(), top.end(), [](const Cand& a, const Cand& b) { return a.p > b.p || (a.p == b.p && a.v < b.v); });
    for (int i = 0; i < kk; ++i) {
      idx[(size_t)r * kk + i] = i < (int)top.size() ? top[i].v : -1;
      logp[(size_t)r * kk + i] = i < (int)top.size() ? std::log(top[i].p) : 0.f;
    }
  }
}

// Whole decode of n_sent sentences with n_models ensemble members.
//   desc            [5] = L, H, V, Vs, feed_input (shared by the members)
//   src_ids/src_off natural-order source ids, sentence i = src_ids[src_off[i]..src_off[i+1])
//   steps           T_i: number of beam expansions; one more forward appends EOS
//                   (src/decoder.h:1806, 1829-1836)
// Outputs (row length max_len = max T_i + 2; hypotheses include START and EOS):
//   out_tok [n_sent][nbest][max_len], out_len [n_sent][nbest] (0 = no hypothesis),
//   out_score [n_sent][nbest], out_vit [n_sent][nbest][max_len],
//   out_align nullable [n_sent][nbest][max_len][max_src]
// Trace (any may be null), Tm = max T_i, k = beam:
//   tr_cand_tok/tr_cand_logp [n_sent][Tm][k][k+1]  per-beam top-(k+1) and logf(p)
//   tr_surv_tok/tr_surv_parent/tr_surv_score [n_sent][Tm][k]
//   tr_final_logp [n_sent][k]  logf(p[EOS]) at the extra forward
//   tr_logp_full  [n_sent][Tm+1][k][V] logf(p) of every forward (small models only)
//   tr_pt         [n_models][n_sent][Tm+1][k] attention centre p_t of every member at every forward
int linmt_oracle_decode(int n_models, const int32_t* desc, const float* const* blobs, size_t blob_n,
                        const void* opts_raw, int n_sent, const int32_t* src_ids, const int32_t* src_off,
                        const int32_t* steps, int32_t* out_tok, int32_t* out_len, float* out_score,
                        int32_t* out_vit, float* out_align, int32_t* tr_cand_tok, float* tr_cand_logp,
                        int32_t* tr_surv_tok, int32_t* tr_surv_parent, float* tr_surv_score,
                        float* tr_final_logp, float* tr_logp_full, float* tr_pt) {
  Opts o;
  std::memcpy(&o, opts_raw, sizeof(Opts));
#ifdef _OPENMP
  if (o.threads > 0) omp_set_num_threads(o.threads);
#endif
  std::vector<Model> models(n_models);
  for (int mi = 0; mi < n_models; ++mi)
    if (!parse_model(models[mi], desc, blobs[mi], blob_n, o.precision)) return 1;
  const int H = desc[1], V = desc[2], L = desc[0];
  int k = o.beam;
  {  // beam clamp, src/decoder.h:1549-1551
    int lim = (int)std::sqrt((double)V);
    if (k > lim) k = lim;
  }
  if (k < 1) return 2;
  const int kk = k + 1;
  const int START = 0, EOS = 1;
  int Tm = 0;
  for (int i = 0; i < n_sent; ++i) Tm = std::max(Tm, steps[i]);
  const int max_len = o.max_len;
  if (max_len < Tm + 2) return 3;
  const int max_src = o.max_src;
  const bool track = o.print_info != 0;
  const bool bf16 = o.precision == 1;

  const int group = o.group > 0 ? o.group : n_sent;
  for (int g0 = 0; g0 < n_sent; g0 += group) {
    const int G = std::min(group, n_sent - g0);
    // order the group's sentences by step count, longest first, so the rows still decoding
    // at any step are a prefix
    std::vector<int> order(G);
    for (int i = 0; i < G; ++i) order[i] = g0 + i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return steps[a] > steps[b]; });
    std::vector<std::vector<int>> rev(G);
    std::vector<int> S(G), T(G);
    for (int i = 0; i < G; ++i) {
      int s = order[i];
      S[i] = src_off[s + 1] - src_off[s];
      if (S[i] < 1 || S[i] > max_src) return 4;
      T[i] = steps[s];
      rev[i].assign(src_ids + src_off[s], src_ids + src_off[s + 1]);
      std::reverse(rev[i].begin(), rev[i].end());  // src/decoder_sentence.cu:68
    }
    const int R = G * k;
    std::vector<ModelRun> runs(n_models);
    for (int mi = 0; mi < n_models; ++mi) {
      ModelRun& st = runs[mi];
      st.m = &models[mi]; st.G = G; st.k = k; st.R = R; st.H = H; st.max_src = max_src; st.S = S;
      st.HS.assign((size_t)G * max_src * H, 0.f);
      st.h.assign(L, std::vector<float>((size_t)R * H)); st.c = st.h; st.hp = st.h; st.cp = st.h;
      st.htilde.assign((size_t)R * H, 0.f); st.htilde_prev = st.htilde;
      st.x.resize((size_t)R * H); st.tanh1.resize((size_t)R * H); st.u.resize((size_t)R * H);
      st.ctx.resize((size_t)R * H); st.cat_t1.resize((size_t)R * H); st.cat_t2.resize((size_t)R * H);
      st.logits.resize((size_t)R * V); st.probs.resize((size_t)R * V);
      st.align.assign((size_t)R * max_src, 0.f); st.pt.resize(R);
      std::vector<std::vector<float>> fh, fc;
      run_encoder(st, rev, bf16, fh, fc);
      // decoder start: layer l copies encoder layer l's final (h, c) into every beam row
      // (src/deep_rnn.h:1766-1789, src/layer_input_to_hidden.h:1536-1545)
      for (int l = 0; l < L; ++l)
        for (int r = 0; r < R; ++r) {
          std::memcpy(&st.hp[l][(size_t)r * H], &fh[l][(size_t)(r / k) * H], H * 4);
          std::memcpy(&st.cp[l][(size_t)r * H], &fc[l][(size_t)(r / k) * H], H * 4);
        }
    }
    // beam state per sentence (src/decoder.h:334-350)
    std::vector<int> tok(R, START);
    std::vector<float> score(R, 0.f);
    std::vector<std::vector<int>> htok(R, std::vector<int>(max_len, START));
    std::vector<std::vector<int>> hvit(R, std::vector<int>(max_len, -20));
    std::vector<std::vector<float>> halign;  // [R][max_len*max_src] when tracked
    if (track) halign.assign(R, std::vector<float>((size_t)max_len * max_src, 0.f));
    std::vector<std::vector<Hyp>> finished(G);
    std::vector<float> pbar((size_t)R * V);
    std::vector<float> abar((size_t)R * max_src, 0.f);
    std::vector<int> vit(R, -1);

    for (int t = 0; t <= Tm; ++t) {
      int n_act = 0;
      for (int i = 0; i < G; ++i) if (T[i] >= t) ++n_act;
      if (n_act == 0) break;
      const int rows = n_act * k;
      for (int mi = 0; mi < n_models; ++mi) run_forward(runs[mi], rows, t, tok.data(), o, track);
      // ensemble: src/decoder.h:1910-1931 (mean of probabilities in double, renormalised
      // per beam); mode 1 is the mean of log-probabilities without renormalisation.
#pragma omp parallel for schedule(static)
      for (int r = 0; r < rows; ++r) {
        float* pb = &pbar[(size_t)r * V];
        if (o.ensemble_mode == 0) {
          for (int v = 0; v < V; ++v) {
            double s = 0;
            for (int mi = 0; mi < n_models; ++mi) s += runs[mi].probs[(size_t)r * V + v];
            pb[v] = (float)(s / n_models);
          }
          float norm = 0.f;
          for (int v = 0; v < V; ++v) norm += pb[v];
          for (int v = 0; v < V; ++v) pb[v] = pb[v] / norm;
        } else {
          for (int v = 0; v < V; ++v) {
            double s = 0;
            for (int mi = 0; mi < n_models; ++mi) s += (double)std::log(runs[mi].probs[(size_t)r * V + v]);
            pb[v] = (float)std::exp(s / n_models);
          }
        }
        if (track) {  // src/decoder.h:1934-1964: summed alignments, arg-max with max starting at 0
          float* ab = &abar[(size_t)r * max_src];
          for (int s = 0; s < max_src; ++s) {
            float a = 0.f;
            for (int mi = 0; mi < n_models; ++mi) a += runs[mi].align[(size_t)r * max_src + s];
            ab[s] = a;
          }
          float mv = 0.f; int mj = -1;
          for (int s = 0; s < max_src; ++s) if (ab[s] > mv) { mv = ab[s]; mj = s; }
          vit[r] = mj;
        }
      }
      if (tr_pt)
        for (int mi = 0; mi < n_models; ++mi)
          for (int i = 0; i < n_act; ++i)
            for (int b = 0; b < k; ++b)
              tr_pt[(((size_t)mi * n_sent + order[i]) * (Tm + 1) + t) * k + b] = runs[mi].pt[i * k + b];
      if (tr_logp_full) {
        for (int i = 0; i < n_act; ++i)
          for (int b = 0; b < k; ++b) {
            float* dst = tr_logp_full + (((size_t)order[i] * (Tm + 1) + t) * k + b) * V;
            const float* pb = &pbar[(size_t)(i * k + b) * V];
            for (int v = 0; v < V; ++v) dst[v] = std::log(pb[v]);
          }
      }
      std::vector<int> parent(R, 0);
      for (int i = 0; i < n_act; ++i) {
        const int sent = order[i];
        const int r0 = i * k;
        if (t == T[i]) {
          // FinishCurrentHypotheses, src/decoder.h:502-525
          for (int b = 0; b < k; ++b) {
            const int r = r0 + b;
            float lp = std::log(pbar[(size_t)r * V + EOS]);
            if (tr_final_logp) tr_final_logp[(size_t)sent * k + b] = lp;
            score[r] += lp + o.penalty;
            Hyp h;
            h.tok.assign(htok[r].begin(), htok[r].begin() + t + 2);
            h.tok[t + 1] = EOS;
            h.vit.assign(hvit[r].begin(), hvit[r].begin() + t + 2);
            h.vit[t + 1] = vit[r];
            if (track) {
              h.align.assign(halign[r].begin(), halign[r].begin() + (size_t)(t + 2) * max_src);
              std::memcpy(&h.align[(size_t)(t + 1) * max_src], &abar[(size_t)r * max_src], max_src * 4);
            }
            h.score = score[r];
            finished[i].push_back(std::move(h));
          }
          continue;
        }
        // ExpandHypothesis, src/decoder.h:355-480
        const int cols = (t == 0) ? 1 : k;
        std::vector<GCand> cand;
        for (int b = 0; b < cols; ++b) {
          const float* pb = &pbar[(size_t)(r0 + b) * V];
          std::vector<Cand> top;
          top.reserve(kk);
          for (int v = 0; v < V; ++v) {
            if ((int)top.size() < kk) top.push_back({pb[v], v});
            else {
              int worst = 0;
              for (int q = 1; q < kk; ++q)
                if (top[q].p < top[worst].p || (top[q].p == top[worst].p && top[q].v > top[worst].v)) worst = q;
              if (pb[v] > top[worst].p) top[worst] = {pb[v], v};
            }
          }
          std::sort(top.begin(), top.end(),
                    [](const Cand& a, const Cand& c) { return a.p > c.p || (a.p == c.p && a.v < c.v); });
          for (int q = 0; q < (int)top.size(); ++q) {
            float lp = std::log(top[q].p);
            float rank_penalty = (float)(q + 1) * o.diversity;
            float sc = lp + score[r0 + b] - rank_penalty;
            cand.push_back({sc, b, top[q].v});
            if (tr_cand_tok && t < Tm) {
              size_t off = ((((size_t)sent * Tm + t) * k + b) * kk) + q;
              tr_cand_tok[off] = top[q].v;
              tr_cand_logp[off] = lp;
            }
          }
        }
        // canonical pop order of the global heap: score desc, beam asc, vocab asc
        std::sort(cand.begin(), cand.end(), [](const GCand& a, const GCand& c) {
          if (a.score != c.score) return a.score > c.score;
          if (a.beam != c.beam) return a.beam < c.beam;
          return a.v < c.v;
        });
        std::vector<int> ntok(k), npar(k);
        std::vector<float> nscore(k);
        int ns = 0;
        for (size_t ci = 0; ci < cand.size() && ns < k; ++ci) {
          const GCand& cd = cand[ci];
          if (cd.v == START) continue;
          const int rb = r0 + cd.beam;
          if (cd.v == EOS) {
            Hyp h;
            h.tok.assign(htok[rb].begin(), htok[rb].begin() + t + 2);
            h.tok[t + 1] = EOS;
            h.vit.assign(hvit[rb].begin(), hvit[rb].begin() + t + 2);
            h.vit[t + 1] = vit[rb];
            if (track) {
              h.align.assign(halign[rb].begin(), halign[rb].begin() + (size_t)(t + 2) * max_src);
              std::memcpy(&h.align[(size_t)(t + 1) * max_src], &abar[(size_t)rb * max_src], max_src * 4);
            }
            h.score = cd.score + o.penalty;
            finished[i].push_back(std::move(h));
            continue;
          }
          ntok[ns] = cd.v; npar[ns] = cd.beam; nscore[ns] = cd.score + o.penalty;
          ++ns;
        }
        // The reference pops an empty heap here (undefined); the defined rule is a dead
        // hypothesis: token UNK(2) from beam 0 with score -1e30.
        for (; ns < k; ++ns) { ntok[ns] = 2; npar[ns] = 0; nscore[ns] = -1e30f; }
        std::vector<std::vector<int>> t_tok(k), t_vit(k);
        std::vector<std::vector<float>> t_al(k);
        for (int b = 0; b < k; ++b) {
          const int rb = r0 + npar[b];
          t_tok[b] = htok[rb]; t_tok[b][t + 1] = ntok[b];
          t_vit[b] = hvit[rb]; t_vit[b][t + 1] = vit[rb];
          if (track) {
            t_al[b] = halign[rb];
            std::memcpy(&t_al[b][(size_t)(t + 1) * max_src], &abar[(size_t)rb * max_src], max_src * 4);
          }
        }
        for (int b = 0; b < k; ++b) {
          const int r = r0 + b;
          htok[r].swap(t_tok[b]); hvit[r].swap(t_vit[b]);
          if (track) halign[r].swap(t_al[b]);
          tok[r] = ntok[b]; score[r] = nscore[b]; parent[r] = npar[b];
          if (tr_surv_tok) {
            size_t off = ((size_t)sent * Tm + t) * k + b;
            tr_surv_tok[off] = ntok[b]; tr_surv_parent[off] = npar[b]; tr_surv_score[off] = nscore[b];
          }
        }
      }
      // SwapDecodingStates + TargetCopyPrevStates, src/deep_rnn.h:1842-1872
      for (int mi = 0; mi < n_models; ++mi) {
        ModelRun& st = runs[mi];
        for (int l = 0; l < L; ++l)
          for (int r = 0; r < rows; ++r) {
            const int srcr = (r / k) * k + parent[r];
            std::memcpy(&st.hp[l][(size_t)r * H], &st.h[l][(size_t)srcr * H], H * 4);
            std::memcpy(&st.cp[l][(size_t)r * H], &st.c[l][(size_t)srcr * H], H * 4);
          }
        for (int r = 0; r < rows; ++r) {
          const int srcr = (r / k) * k + parent[r];
          std::memcpy(&st.htilde_prev[(size_t)r * H], &st.htilde[(size_t)srcr * H], H * 4);
        }
      }
    }

    // ObtainOneBestHypothesis, src/decoder.h:703-859
    for (int i = 0; i < G; ++i) {
      const int sent = order[i];
      const int Sl = S[i];
      std::vector<Hyp>& hy = finished[i];
      if (0 != o.lp_alpha)
        for (auto& h : hy) {
          float lp = powf((float)(5 + (int)h.tok.size()), o.lp_alpha) / powf((float)(5 + 1), o.lp_alpha);
          h.score /= lp;
        }
      if (0 != o.cp_beta)
        for (auto& h : hy) {
          const int n = (int)h.tok.size();
          std::vector<float> al((size_t)n * Sl, 0.f);
          if (track)
            for (int p = 0; p < n; ++p)
              for (int s = 0; s < Sl; ++s) al[(size_t)p * Sl + s] = h.align[(size_t)p * max_src + s];
          for (int j = 1; j < n - 1; ++j) {
            float sum = 0.f;
            for (int s = 0; s < Sl; ++s) { al[(size_t)(j + 1) * Sl + s] += 0.01; sum += al[(size_t)(j + 1) * Sl + s]; }
            for (int s = 0; s < Sl; ++s) al[(size_t)(j + 1) * Sl + s] /= sum;
          }
          float cp = 0.f;
          for (int s = 0; s < Sl; ++s) {
            float sum = 0.f;
            for (int j = 1; j < n - 1; ++j) sum += al[(size_t)(j + 1) * Sl + s];
            cp += std::log(std::min(sum, 1.0f));
          }
          cp *= o.cp_beta;
          if (cp < -20) cp = -20;
          h.score += cp;
          if (track)
            for (int p = 0; p < n; ++p)
              for (int s = 0; s < Sl; ++s) h.align[(size_t)p * max_src + s] = al[(size_t)p * Sl + s];
        }
      // n-best with strictly-greater replacement; canonical tie order = creation order
      std::vector<int> best;
      for (int q = 0; q < (int)hy.size(); ++q) {
        float ratio = ((float)hy[q].tok.size()) / Sl;
        if (!(ratio > o.min_ratio)) continue;
        if ((int)best.size() < o.nbest) best.push_back(q);
        else {
          int worst = 0;
          for (int z = 1; z < (int)best.size(); ++z)
            if (hy[best[z]].score < hy[best[worst]].score ||
                (hy[best[z]].score == hy[best[worst]].score && best[z] > best[worst])) worst = z;
          if (hy[best[worst]].score < hy[q].score) best[worst] = q;
        }
      }
      std::sort(best.begin(), best.end(), [&](int a, int b) {
        if (hy[a].score != hy[b].score) return hy[a].score > hy[b].score;
        return a < b;
      });
      for (int q = 0; q < o.nbest; ++q) {
        size_t ob = (size_t)sent * o.nbest + q;
        if (q >= (int)best.size()) { out_len[ob] = 0; out_score[ob] = 0.f; continue; }
        const Hyp& h = hy[best[q]];
        out_len[ob] = (int)h.tok.size();
        out_score[ob] = h.score;
        for (int p = 0; p < (int)h.tok.size(); ++p) {
          out_tok[ob * max_len + p] = h.tok[p];
          if (out_vit) out_vit[ob * max_len + p] = h.vit[p];
        }
        if (out_align && track)
          std::memcpy(out_align + ob * max_len * max_src, h.align.data(), h.align.size() * 4);
      }
    }
  }
  return 0;
}

}  // extern "C"

// engine.cu -- decoding engine: weight packing, device state, encoder, step loop, C ABI.
//
// Host code launches kernels on one stream and never waits inside the step loop: beam
// state, back-pointers, finished hypotheses and alignment records all stay on the device
// (the reference copies V x k probabilities to the host and walks heaps there every step,
// src/decoder.h:1396-1436, 355-480).
#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <chrono>
#include <mutex>
#include <numeric>
#include <thread>

#include "gemm_simt.cuh"
#include "step_kernels.cuh"

namespace linmt {

#define CK(call)                                                                              \
  do {                                                                                        \
    cudaError_t e_ = (call);                                                                  \
    if (e_ != cudaSuccess) {                                                                  \
      char b_[512];                                                                           \
      snprintf(b_, sizeof b_, "CUDA error %s at %s:%d: %s", cudaGetErrorName(e_), __FILE__, __LINE__, cudaGetErrorString(e_)); \
      return fail(LINMT_ECUDA, b_);                                                           \
    }                                                                                         \
  } while (0)

#define LAUNCHED() (++stats.kernel_launches)

template <class T>
int Engine::dalloc(T** p, size_t count) {
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T));
  if (e != cudaSuccess) {
    err = std::string("cudaMalloc failed: ") + cudaGetErrorString(e);
    return LINMT_ENOMEM;
  }
  allocs_.push_back(q);
  *p = static_cast<T*>(q);
  return LINMT_OK;
}
// Replaces *p by a fresh allocation of `count` elements and frees the old one.
template <class T>
int Engine::regrow(T** p, size_t count) {
  if (*p) {
    auto it = std::find(allocs_.begin(), allocs_.end(), static_cast<void*>(*p));
    if (it != allocs_.end()) allocs_.erase(it);
    cudaFree(*p);
    *p = nullptr;
  }
  return dalloc(p, count);
}
#define DA(p, n)                                  \
  do {                                            \
    int rc_ = dalloc(&(p), (n));                  \
    if (rc_ != LINMT_OK) return rc_;              \
  } while (0)

Engine::~Engine() {
  if (stream) { cudaSetDevice(opt.device); cudaStreamSynchronize(stream); }
  for (void* p : allocs_) cudaFree(p);
  for (void* p : trace_allocs_) cudaFree(p);
  if (h_meta_) cudaFreeHost(h_meta_);
  if (ev0_) cudaEventDestroy(ev0_);
  if (ev1_) cudaEventDestroy(ev1_);
  for (auto e : kt_ev_) cudaEventDestroy(e);
  for (auto& v : enc_events_) for (auto e : v) cudaEventDestroy(e);
  if (enc_start_ev_) cudaEventDestroy(enc_start_ev_);
  for (auto st : enc_streams_) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
  if (stream) cudaStreamDestroy(stream);
}

// ---------------------------------------------------------------------------------------
// Host-side packing.  A reference weight "out x in" sits column-major, i.e. [in][out]
// (src/utility_cu.h:37).  Packed gate matrix row 4j+g = gate g of hidden unit j, columns =
// the K-concatenation of the segments, each padded to Hp.
void pack_gate_weights(const float* const* mats, int nseg, int H, int Hp, float* out) {
  const size_t K = (size_t)nseg * Hp;
  std::memset(out, 0, sizeof(float) * 4 * (size_t)Hp * K);
#pragma omp parallel for schedule(static)
  for (int j = 0; j < H; ++j)
    for (int g = 0; g < 4; ++g) {
      float* row = out + ((size_t)4 * j + g) * K;
      for (int s = 0; s < nseg; ++s) {
        const float* m = mats[s * 4 + g];
        float* dst = row + (size_t)s * Hp;
        for (int kx = 0; kx < H; ++kx) dst[kx] = m[(size_t)kx * H + j];
      }
    }
}

namespace {
struct BlobView {
  struct Lstm {
    const float *Whi, *bi, *Whf, *bf, *Whc, *bc, *Who, *bo, *emb, *Mi, *Mf, *Mo, *Mc, *Qi, *Qf, *Qo, *Qc;
  };
  std::vector<Lstm> src, tgt;
  const float *Wa, *Wp, *vp, *bout, *Wc1, *Wc2, *D, *bd;
};
// Matrix order of a model file: src/layer_input_to_hidden.h:1378-1423,
// src/layer_hidden_to_hidden.h:953-979, src/layer_attention.h:1246-1260,
// src/layer_loss.h:1191-1196, sequence src/deep_rnn.h:1878-1969.
BlobView view_blob(const linmt_model_desc& d, const float* p) {
  BlobView v;
  const size_t H = d.hidden, hh = H * H;
  auto take = [&](size_t n) { const float* q = p; p += n; return q; };
  auto lstm = [&](BlobView::Lstm& w, bool first, size_t vocab, bool feed) {
    w.Whi = take(hh); w.bi = take(H); w.Whf = take(hh); w.bf = take(H);
    w.Whc = take(hh); w.bc = take(H); w.Who = take(hh); w.bo = take(H);
    w.emb = first ? take(H * vocab) : nullptr;
    w.Mi = take(hh); w.Mf = take(hh); w.Mo = take(hh); w.Mc = take(hh);
    w.Qi = w.Qf = w.Qo = w.Qc = nullptr;
    if (feed) { w.Qi = take(hh); w.Qf = take(hh); w.Qo = take(hh); w.Qc = take(hh); }
  };
  v.src.resize(d.layers); v.tgt.resize(d.layers);
  for (int l = 0; l < d.layers; ++l) lstm(v.src[l], l == 0, d.vocab_src, false);
  for (int l = 0; l < d.layers; ++l) lstm(v.tgt[l], l == 0, d.vocab_tgt, l == 0 && d.feed_input);
  v.Wa = take(hh); v.Wp = take(hh); v.vp = take(H); v.bout = take(H); v.Wc1 = take(hh); v.Wc2 = take(hh);
  v.D = take((size_t)d.vocab_tgt * H); v.bd = take(d.vocab_tgt);
  return v;
}
}  // namespace

int Engine::pack_model(const float* blob, DevModel& m) {
  const BlobView bv = view_blob(desc, blob);
  if (use_tc_ && fmt_ == 1) {
    // the fp16 pair cannot hold a weight beyond fp16's range (nor a NaN); trained weights are orders of magnitude below it
    const size_t nf = (size_t)linmt_blob_floats(&desc);
    for (size_t i = 0; i < nf; ++i)
      if (!(std::fabs(blob[i]) <= 60000.0f))
        return fail(LINMT_EINVAL, "a weight is not finite or exceeds 60000 in magnitude: use gemm_path tensor3 or simt for this model");
  }
  std::vector<float> host;
  auto upload = [&](float** dst, size_t n) -> int {
    DA(*dst, n);
    cudaError_t e = cudaMemcpy(*dst, host.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(LINMT_ECUDA, std::string("weight upload: ") + cudaGetErrorString(e));
    return LINMT_OK;
  };
  // a dense operand goes to the device either as fp32 (CUDA-core path) or as bf16 planes
  auto store = [&](float** dst, tc::Planes* planes, size_t rows, int ld) -> int {
    if (use_tc_) return to_planes(host, rows, ld, *planes);
    return upload(dst, host.size());
  };
  auto pack_emb = [&](const float* emb, int vocab, float** dst, tc::Planes* planes) -> int {
    host.assign((size_t)vocab * Hp, 0.f);
#pragma omp parallel for schedule(static)
    for (int v = 0; v < vocab; ++v) std::memcpy(&host[(size_t)v * Hp], emb + (size_t)v * H, sizeof(float) * H);
    return store(dst, planes, vocab, Hp);
  };
  auto pack_bias4 = [&](const BlobView::Lstm& w, float** dst) -> int {
    host.assign((size_t)4 * Hp, 0.f);
    const float* bs[4] = {w.bi, w.bf, w.bc, w.bo};
    for (int j = 0; j < H; ++j)
      for (int g = 0; g < 4; ++g) host[(size_t)4 * j + g] = bs[g][j];
    return upload(dst, host.size());
  };
  auto pack_lstm = [&](const BlobView::Lstm& w, bool feed, float** wdst, tc::Planes* planes, float** bdst, int* ldw) -> int {
    const int nseg = feed ? 3 : 2;
    const float* mats[12] = {w.Mi, w.Mf, w.Mc, w.Mo, w.Whi, w.Whf, w.Whc, w.Who, w.Qi, w.Qf, w.Qc, w.Qo};
    host.resize((size_t)4 * Hp * nseg * Hp);
    pack_gate_weights(mats, nseg, H, Hp, host.data());
    *ldw = nseg * Hp;
    int rc = store(wdst, planes, (size_t)4 * Hp, nseg * Hp);
    if (rc) return rc;
    return pack_bias4(w, bdst);
  };
  int rc;
  if ((rc = pack_emb(bv.src[0].emb, desc.vocab_src, &m.emb_src, &m.p_emb_src))) return rc;
  if ((rc = pack_emb(bv.tgt[0].emb, desc.vocab_tgt, &m.emb_tgt, &m.p_emb_tgt))) return rc;
  m.enc_w.resize(L); m.enc_b.resize(L); m.dec_w.resize(L); m.dec_b.resize(L); m.dec_ldw.resize(L);
  m.p_enc_w.resize(L); m.p_dec_w.resize(L);
  for (int l = 0; l < L; ++l) {
    int ld;
    if ((rc = pack_lstm(bv.src[l], false, &m.enc_w[l], &m.p_enc_w[l], &m.enc_b[l], &ld))) return rc;
    if ((rc = pack_lstm(bv.tgt[l], l == 0 && desc.feed_input, &m.dec_w[l], &m.p_dec_w[l], &m.dec_b[l], &m.dec_ldw[l]))) return rc;
  }
  // attention projections: rows < Hp: W_p (out n, in k) = blob[k*H + n];
  // rows Hp + j: (W_a^T h)[j] = sum_i W_a[i,j] h[i], W_a[i,j] = blob[j*H + i]  (src/layer_attention.h:327)
  // rows 2Hp + n (tensor path): W_c2, the h_top half of the attention output product -- it depends on h_top
  // alone, so it is computed with the projections, ahead of the attention kernel, instead of after it
  const int proj_rows = use_tc_ ? 3 * Hp : 2 * Hp;
  host.assign((size_t)proj_rows * Hp, 0.f);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < H; ++n)
    for (int kx = 0; kx < H; ++kx) {
      host[(size_t)n * Hp + kx] = bv.Wp[(size_t)kx * H + n];
      host[(size_t)(Hp + n) * Hp + kx] = bv.Wa[(size_t)n * H + kx];
      if (use_tc_) host[(size_t)(2 * Hp + n) * Hp + kx] = bv.Wc2[(size_t)kx * H + n];
    }
  if ((rc = store(&m.att_proj_w, &m.p_att_proj_w, (size_t)proj_rows, Hp))) return rc;
  // attention output: columns (ctx | h_top) -> W_c1 | W_c2 (src/layer_attention.h:441,448)
  host.assign((size_t)Hp * 2 * Hp, 0.f);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < H; ++n)
    for (int kx = 0; kx < H; ++kx) {
      host[(size_t)n * 2 * Hp + kx] = bv.Wc1[(size_t)kx * H + n];
      host[(size_t)n * 2 * Hp + Hp + kx] = bv.Wc2[(size_t)kx * H + n];
    }
  if ((rc = store(&m.att_out_w, &m.p_att_out_w, (size_t)Hp, 2 * Hp))) return rc;
  host.assign(Hp, 0.f);
  std::memcpy(host.data(), bv.bout, sizeof(float) * H);
  if ((rc = upload(&m.att_bout, host.size()))) return rc;
  host.assign(Hp, 0.f);
  std::memcpy(host.data(), bv.vp, sizeof(float) * H);
  if ((rc = upload(&m.vp, host.size()))) return rc;
  // output matrix D (V x H), element (v,h) = blob[h*V + v]  ->  [Vp][Hp]
  host.assign((size_t)Vp * Hp, 0.f);
#pragma omp parallel for schedule(static)
  for (int v = 0; v < V; ++v)
    for (int kx = 0; kx < H; ++kx) host[(size_t)v * Hp + kx] = bv.D[(size_t)kx * V + v];
  {
    double best = 0.0;
    for (int v = 0; v < V; ++v) {
      double ss = 0.0;
      for (int kx = 0; kx < H; ++kx) { const double w = host[(size_t)v * Hp + kx]; ss += w * w; }
      if (ss > best) best = ss;
    }
    m.voc_wnorm_max = (float)std::sqrt(best);
  }
  if ((rc = store(&m.voc_w, &m.p_voc_w, (size_t)Vp, Hp))) return rc;
  host.assign(Vp, 0.f);
  std::memcpy(host.data(), bv.bd, sizeof(float) * V);
  for (int v = 0; v < V; ++v) m.voc_babs_max = std::max(m.voc_babs_max, std::fabs(host[v]));
  if ((rc = upload(&m.voc_b, host.size()))) return rc;
  return LINMT_OK;
}

int Engine::alloc_state(DevState& s) {
  const size_t rh = (size_t)R * Hp;
  DA(s.x, rh);
  s.h_cur.resize(L); s.c_cur.resize(L); s.h_prev.resize(L); s.c_prev.resize(L);
  for (int l = 0; l < L; ++l) { DA(s.h_cur[l], rh); DA(s.c_cur[l], rh); DA(s.h_prev[l], rh); DA(s.c_prev[l], rh); }
  DA(s.htilde, rh); DA(s.htilde_prev, rh);
  DA(s.proj, 3 * rh); DA(s.ctx, rh);
  DA(s.logits, (size_t)R * Vp);
  if (logits16_) DA(s.logits16, (size_t)R * Vp);
  DA(s.hs, (size_t)B * opt.max_src_len * Hp);
  CK(cudaMemset(s.hs, 0, sizeof(float) * (size_t)B * opt.max_src_len * Hp));   // rows past a sentence's end are never written, but read as GEMM operand rows by the fold
  if (att_fold_) DA(s.hs_wc1, (size_t)B * opt.max_src_len * Hp);
  DA(s.enc_x, (size_t)B * Hp);
  for (int i = 0; i < 2; ++i) {
    s.enc_h[i].resize(L); s.enc_c[i].resize(L);
    for (int l = 0; l < L; ++l) { DA(s.enc_h[i][l], (size_t)B * Hp); DA(s.enc_c[i][l], (size_t)B * Hp); }
  }
  return LINMT_OK;
}

int Engine::init(const linmt_model_desc& d, const float* const* blobs, int nm, size_t blob_floats, const linmt_options& o) {
  desc = d; opt = o; n_models = nm;
  if (d.layers < 1 || d.layers > 5 || d.hidden < 4 || d.vocab_tgt < 4 || d.vocab_src < 1)
    return fail(LINMT_EINVAL, "bad model dimensions (layers 1..5)");
  if (nm < 1) return fail(LINMT_EINVAL, "need at least one model");
  if (nm > 8) return fail(LINMT_ELIMIT, "at most 8 ensemble members");
  if (o.precision != LINMT_PREC_FP32 && o.precision != LINMT_PREC_BF16) return fail(LINMT_EINVAL, "bad precision");
  if (o.gemm_path < LINMT_GEMM_AUTO || o.gemm_path > LINMT_GEMM_TENSOR_V16X) return fail(LINMT_EINVAL, "bad gemm_path");
  if (o.precision == LINMT_PREC_BF16 && o.gemm_path == LINMT_GEMM_SIMT)
    return fail(LINMT_EINVAL, "bf16 precision runs on the tensor-core path only");
  use_tc_ = o.gemm_path != LINMT_GEMM_SIMT;
  { const char* pe = std::getenv("LINMT_XW"); xw_table_ = use_tc_ && !(pe && std::atoi(pe) == 0); }   // LINMT_XW=0: test knob
  { const char* pe = std::getenv("LINMT_PMAX"); pmax_on_ = !(pe && std::atoi(pe) == 0); }
  { const char* pe = std::getenv("LINMT_ATT_MERGE"); att_merge_ = use_tc_ && !(pe && std::atoi(pe) == 0); }
  // (local attention only: over a whole sentence the second window costs the attention kernel more than the GEMM it replaces)
  { const char* pe = std::getenv("LINMT_ATT_FOLD"); att_fold_ = att_merge_ && o.attention_mode == LINMT_ATT_LOCAL_P_GENERAL && !(pe && std::atoi(pe) == 0); }
  { const char* pe = std::getenv("LINMT_TC_PERSIST"); persist_ = !(pe && std::atoi(pe) == 0); }
  { const char* pe = std::getenv("LINMT_TC_PAIR"); pair_ = !(pe && std::atoi(pe) == 0); }
  { const char* pe = std::getenv("LINMT_PDL"); pdl_ = use_tc_ && !(pe && std::atoi(pe) == 0); }   // LINMT_PDL=0: test knob
  // fp32 weights on the tensor cores: the f16 pair by default (3 partial products), bf16 planes on request
  fmt_ = (o.precision == LINMT_PREC_FP32 && (o.gemm_path == LINMT_GEMM_AUTO || o.gemm_path == LINMT_GEMM_TENSOR || o.gemm_path == LINMT_GEMM_TENSOR_V16 ||
          o.gemm_path == LINMT_GEMM_TENSOR_V16X)) ? 1 : 0;
  nt_ = (o.precision == LINMT_PREC_BF16) ? 1 : (o.gemm_path == LINMT_GEMM_TENSOR3 ? 3 : 2);
  // The vocabulary product feeds only the softmax of its own step (nothing recurrent), so two
  // planes (error ~2^-17 per product, ~3e-7 relative on a log-probability) are enough there:
  // measured parity on the 64-sentence reference configuration is unchanged and the GEMM is 1.3x faster.
  nt_vocab_ = (nt_ == 3) ? 2 : nt_;
  // AUTO = TENSOR_V16X: plain fp16 logits (the first plane of each pair) with the candidates recomputed accurately
  // in the softmax kernel; ensembles combine whole distributions and keep the three-product logits
  const bool v16x = o.gemm_path == LINMT_GEMM_TENSOR_V16X || o.gemm_path == LINMT_GEMM_AUTO;
  if (fmt_ == 1 && (o.gemm_path == LINMT_GEMM_TENSOR_V16 || (v16x && nm == 1))) nt_vocab_ = 1;
  refine_ = fmt_ == 1 && v16x && nm == 1;
  { const char* pe = std::getenv("LINMT_LOGITS16"); logits16_ = refine_ && !(pe && std::atoi(pe) == 0); }
  if (linmt_blob_floats(&d) != blob_floats) return fail(LINMT_EINVAL, "weight blob size does not match the model dimensions");
  if (o.beam <= 0) return fail(LINMT_EINVAL, "--beam-size cannot be <= 0");
  if (o.penalty < 0) return fail(LINMT_EINVAL, "--penalty cannot be < 0");
  if (o.nbest < 1 || o.nbest > 32) return fail(LINMT_EINVAL, "nbest must be in 1..32");
  if (o.max_batch < 1 || o.max_src_len < 1 || o.max_steps < 1) return fail(LINMT_EINVAL, "bad capacity options");
  L = d.layers; H = d.hidden; V = d.vocab_tgt;
  k = std::min<int>(o.beam, (int)std::sqrt((double)V));  // src/decoder.h:1549-1551
  if (k > kMaxBeam) return fail(LINMT_ELIMIT, "beam larger than 31 is not supported");
  kk = k + 1;
  Hp = round_up(H, 64);
  Vp = round_up(V, 128);
  B = o.max_batch; R = B * k;
  win = (o.attention_mode == LINMT_ATT_LOCAL_P_GENERAL) ? 2 * o.attention_d + 1 : o.max_src_len;
  rec_win = (nm > 1) ? o.max_src_len : win;   // ensembles keep dense alignment records: the members' windows differ
  Tcap = o.max_steps + 1;
  fin_cap = Tcap * k;
  CK(cudaSetDevice(o.device));
  int cc_major = 0;
  CK(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, o.device));
  if (cc_major != 10) return fail(LINMT_ECUDA, "this library is built for sm_100a (B200) only");
  CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  CK(cudaEventCreate(&ev0_)); CK(cudaEventCreate(&ev1_));
  CK(cudaDeviceGetAttribute(&n_sm_, cudaDevAttrMultiProcessorCount, o.device));
  DA(d_tc_err_, 1);
  CK(cudaMemset(d_tc_err_, 0, sizeof(int)));
  if (use_tc_) {
    DA(d_splitk_ws_, kSplitKWsFloats);
    DA(d_splitk_counters_, kSplitKMaxTiles);
    CK(cudaMemset(d_splitk_counters_, 0, sizeof(int) * kSplitKMaxTiles));
    if (pair_ && !pairs_available()) pair_ = false;   // (a device that cannot co-schedule two such CTAs keeps the one-tile kernels)
  }
  models_.resize(nm); states_.resize(nm); tc_states_.resize(nm);
  for (int i = 0; i < nm; ++i) {
    int rc = pack_model(blobs[i], models_[i]);
    if (rc) return rc;
    // fp16 storage of the logits needs them inside fp16's range with room to spare: |z| <= |w_row| |htilde| + |b| and
    // every component of htilde is below 1 in magnitude
    if (logits16_ && !(models_[i].voc_wnorm_max * std::sqrt((float)H) + models_[i].voc_babs_max < 3.0e4f)) logits16_ = false;
    if ((rc = alloc_state(states_[i]))) return rc;
    if (use_tc_ && (rc = alloc_state_tc(tc_states_[i]))) return rc;
  }
  DA(d_off_, B + 1); DA(d_len_, B); DA(d_steps_, B); DA(d_orig_, B);
  CK(cudaMallocHost(&h_meta_, sizeof(int32_t) * 4 * (B + 1)));
  DA(d_tok_, R); DA(d_parent_, R); DA(d_score_, R);
  DA(d_hist_tok_, (size_t)Tcap * R); DA(d_hist_parent_, (size_t)Tcap * R);
  DA(d_fin_t_, (size_t)B * fin_cap); DA(d_fin_b_, (size_t)B * fin_cap); DA(d_fin_n_, B);
  DA(d_fin_score_, (size_t)B * fin_cap); DA(d_fin_final_, (size_t)B * fin_cap);
  if (nm > 1) DA(d_combined_, (size_t)R * Vp);
  DA(d_cand_idx_, (size_t)R * kk); DA(d_cand_logp_, (size_t)R * kk); DA(d_eos_logp_, R); DA(d_row_stats_, 2 * (size_t)R);
  pmax_ld_ = 4 * ((Vp + 47) / 48) + 4;   // four column blocks per tile, tiles at least 48 wide
  DA(d_pmax_, (size_t)R * pmax_ld_);
  if (o.print_info) {
    DA(d_rec_align_, (size_t)Tcap * R * rec_win); DA(d_rec_lo_, (size_t)Tcap * R); DA(d_rec_vit_, (size_t)Tcap * R);
  }
  if (use_tc_ && xw_table_) { const int rc_xw = build_xw_tables(); if (rc_xw) return rc_xw; }
  CK(cudaDeviceSynchronize());  // every weight upload has landed before the first decode
  return LINMT_OK;
}

// ---------------------------------------------------------------------------------------
// Encoder (NeuralMachineTranslation::ForwardPropSource, src/deep_rnn.h:1572-1721): all
// sentences of the batch advance together, one position per round; a row stops changing
// once its sentence is consumed.  Top-layer states go to hs[b][pos].
int Engine::run_encoder(int n, int Smax) {
  for (int mi = 0; mi < n_models; ++mi) {
    DevModel& m = models_[mi];
    DevState& s = states_[mi];
    for (int l = 0; l < L; ++l) {
      CK(cudaMemsetAsync(s.enc_h[0][l], 0, sizeof(float) * (size_t)B * Hp, stream));
      CK(cudaMemsetAsync(s.enc_c[0][l], 0, sizeof(float) * (size_t)B * Hp, stream));
    }
    for (int pos = 0; pos < Smax; ++pos) {
      const int in = pos & 1, out = in ^ 1;
      enc_embed_kernel<<<n, 256, 0, stream>>>(cur_ids_, d_off_, d_len_, m.emb_src, desc.vocab_src, s.enc_x, Hp, pos);
      LAUNCHED();
      for (int l = 0; l < L; ++l) {
        ASegs a{};
        a.ptr[0] = (l == 0) ? s.enc_x : s.enc_h[out][l - 1]; a.ld[0] = Hp;
        a.ptr[1] = s.enc_h[in][l]; a.ld[1] = Hp;
        a.nseg = 2; a.seg_k = Hp;
        EpiLstm e{};
        e.bias = m.enc_b[l]; e.c_prev = s.enc_c[in][l]; e.h_prev = s.enc_h[in][l];
        e.c_out = s.enc_c[out][l]; e.h_out = s.enc_h[out][l];
        e.h_out2 = (l == L - 1) ? s.hs + (size_t)pos * Hp : nullptr;
        e.h2_row_stride = (long long)opt.max_src_len * Hp;
        e.row_len = d_len_; e.pos = pos; e.ld = Hp;
        CK(gemm_simt(a, m.enc_w[l], 2 * Hp, n, 4 * Hp, 2 * Hp, e, stream));
        LAUNCHED();
      }
    }
  }
  return LINMT_OK;
}


// ---------------------------------------------------------------------------------------
// One decoder forward for the first `rows` rows plus beam selection
// (DecoderModelWrapper::ForwardPropTarget src/decoder.h:1396-1423,
//  NeuralMachineTranslation::ForwardPropTarget src/deep_rnn.h:1754-1836).
int Engine::run_decoder_step(int mi, int t, int rows) {
  DevModel& m = models_[mi];
  DevState& s = states_[mi];
  const int n_act = rows / k;
  // 1. reorder states through the parents, look up the new tokens' embeddings
  {
    PrepArrays pa{};
    int na = 0;
    for (int l = 0; l < L; ++l) {
      pa.src[na] = (t == 0) ? s.enc_h[enc_final_buf_][l] : s.h_cur[l]; pa.dst[na++] = s.h_prev[l];
      pa.src[na] = (t == 0) ? s.enc_c[enc_final_buf_][l] : s.c_cur[l]; pa.dst[na++] = s.c_prev[l];
    }
    if (t > 0 && desc.feed_input) { pa.src[na] = s.htilde; pa.dst[na++] = s.htilde_prev; }
    pa.n_arr = na;
    dim3 grid(rows, na + 1);
    if (int rc = kt(KC_GATHER)) return rc;
    dec_prep_kernel<<<grid, 256, 0, stream>>>(pa, d_parent_, d_tok_, m.emb_tgt, V, s.x, Hp, k, t == 0 ? 1 : 0);
    LAUNCHED();
  }
  // 2. LSTM stack
  for (int l = 0; l < L; ++l) {
    if (int rc = kt(KC_LSTM)) return rc;
    ASegs a{};
    a.seg_k = Hp;
    a.ptr[0] = (l == 0) ? s.x : s.h_cur[l - 1]; a.ld[0] = Hp;
    a.ptr[1] = s.h_prev[l]; a.ld[1] = Hp;
    a.nseg = 2;
    if (l == 0 && desc.feed_input && t > 0) { a.ptr[2] = s.htilde_prev; a.ld[2] = Hp; a.nseg = 3; }  // node_input_to_hidden.h:325
    EpiLstm e{};
    e.bias = m.dec_b[l]; e.c_prev = s.c_prev[l]; e.h_prev = s.h_prev[l];
    e.c_out = s.c_cur[l]; e.h_out = s.h_cur[l]; e.h_out2 = nullptr; e.h2_row_stride = 0;
    e.row_len = nullptr; e.pos = 0; e.ld = Hp;
    CK(gemm_simt(a, m.dec_w[l], m.dec_ldw[l], rows, 4 * Hp, a.nseg * Hp, e, stream));
    LAUNCHED();
    if (kernel_timing) rec_flops_ += 2.0 * rows * 4.0 * H * (double)(a.nseg * H);
  }
  float* htop = s.h_cur[L - 1];
  // 3. attention projections
  const float* u_alt = nullptr;
  if (int rc = kt(KC_PROJ)) return rc;
  if (opt.attention_mode == LINMT_ATT_LOCAL_P_GENERAL) {
    ASegs a{}; a.ptr[0] = htop; a.ld[0] = Hp; a.nseg = 1; a.seg_k = Hp;
    EpiAttnProj e{s.proj, 2 * Hp, Hp};
    CK(gemm_simt(a, m.att_proj_w, Hp, rows, 2 * Hp, Hp, e, stream));
    LAUNCHED();
  } else if (opt.attention_mode == LINMT_ATT_GLOBAL_GENERAL) {
    ASegs a{}; a.ptr[0] = htop; a.ld[0] = Hp; a.nseg = 1; a.seg_k = Hp;
    EpiBias e{nullptr, s.proj + Hp, 2 * Hp};
    CK(gemm_simt(a, m.att_proj_w + (size_t)Hp * Hp, Hp, rows, Hp, Hp, e, stream));
    LAUNCHED();
  } else {
    u_alt = htop;
  }
  // 4. scores, softmax x Gaussian, context
  {
    float* ra = d_rec_align_ ? d_rec_align_ + (size_t)t * R * rec_win : nullptr;
    int32_t* rl = d_rec_lo_ ? d_rec_lo_ + (size_t)t * R : nullptr;
    int32_t* rv = d_rec_vit_ ? d_rec_vit_ + (size_t)t * R : nullptr;
    if (int rc = kt(KC_ATTENTION)) return rc;
    if (int rc = launch_attention(mi, t, rows, u_alt, s.ctx, tc::Planes{}, 0, ra, rl, rv)) return rc;
  }
  // 5. attentional state htilde = tanh(W_c1 ctx + W_c2 h + b)
  {
    if (int rc = kt(KC_ATTOUT)) return rc;
    ASegs a{}; a.ptr[0] = s.ctx; a.ld[0] = Hp; a.ptr[1] = htop; a.ld[1] = Hp; a.nseg = 2; a.seg_k = Hp;
    EpiBiasTanh e{m.att_bout, s.htilde, Hp};
    CK(gemm_simt(a, m.att_out_w, 2 * Hp, rows, Hp, 2 * Hp, e, stream));
    LAUNCHED();
  }
  // 6. logits
  {
    ASegs a{}; a.ptr[0] = s.htilde; a.ld[0] = Hp; a.nseg = 1; a.seg_k = Hp;
    EpiBias e{m.voc_b, s.logits, Vp};
    if (int rc = kt(KC_VOCAB)) return rc;
    CK(gemm_simt(a, m.voc_w, Hp, rows, Vp, Hp, e, stream));
    LAUNCHED();
  }
  return LINMT_OK;
}

// Attention of one decoder forward (both GEMM families).
int Engine::launch_attention(int mi, int t, int rows, const float* u_alt, float* ctx, const tc::Planes& ctx_planes, int nt,
                             float* ra, int32_t* rl, int32_t* rv, bool fold) {
  // the record of member mi: [n][Tm+1][k] at pt + mi * (sentences of this device batch's record) * (Tm+1) * k
  const AttTrace at{trace_dev_.pt ? trace_dev_.pt + (size_t)mi * trace_pt_member_stride_ : nullptr, d_orig_, trace_dev_.Tm + 1, t};
  DevModel& m = models_[mi];
  DevState& s = states_[mi];
  const int ldp = att_merge_ ? 3 * Hp : 2 * Hp;
  const size_t smem = sizeof(float) * (win + 8);
  // fold: the weighted sum runs over W_c1 . hs and the kernel writes htilde (ctx_planes = the htilde panel)
  const AttFold af = fold ? AttFold{s.hs_wc1, s.proj + 2 * Hp, 3 * Hp, m.att_bout} : AttFold{nullptr, nullptr, 0, nullptr};
  CK(tc::launch_k(pdl_, attention_kernel, dim3(rows), dim3(256), smem, stream, (const float*)s.proj, ldp, u_alt, Hp, (const float*)m.vp,
                  (const float*)s.hs, (const int32_t*)d_len_, ctx, H, Hp, k, (int)opt.max_src_len, (int)opt.attention_mode,
                  (int)opt.attention_d, win, ra, rl, rv, ctx_planes, nt, rec_win, ens_member_code(mi), at, af));
  LAUNCHED();
  return LINMT_OK;
}

// Log-softmax statistics + per-beam top-(k+1), then beam selection (both paths).
int Engine::step_tail(int t, int rows) {
  DevState& s = states_[0];
  const int n_act = rows / k;
  {
    TopkOut o{d_cand_idx_, d_cand_logp_, d_eos_logp_, d_row_stats_};
    trace_dev_.logits = (n_models == 1) ? s.logits : d_combined_;
    trace_dev_.ld_logits = Vp;
    trace_dev_.row_stats = d_row_stats_;
    if (n_models == 1) {
      if (int rc = kt(KC_SOFTMAX)) return rc;
      TopkRefine rf{};
      if (refine_) {
        const TcState& ts = tc_states_[0];
        const DevModel& m0 = models_[0];
        rf.a0 = reinterpret_cast<const __half*>(ts.panel_ht.p[0]); rf.a1 = reinterpret_cast<const __half*>(ts.panel_ht.p[1]);
        rf.lda = ts.panel_ht.ld;
        rf.b0 = reinterpret_cast<const __half*>(m0.p_voc_w.p[0]); rf.b1 = reinterpret_cast<const __half*>(m0.p_voc_w.p[1]);
        rf.ldb = m0.p_voc_w.ld;
        rf.bias = m0.voc_b; rf.K = Hp;
        rf.eps_coef = 1.1f * (1.0f / 1024.0f) * m0.voc_wnorm_max;
      }
      if (refine_) trace_dev_.rf = rf;
      CK(launch_softmax_topk(s.logits, Vp, V, kk, rows, o, 1, stream, pdl_, d_pmax_, pmax_ld_, pmax_slots_, refine_ ? &rf : nullptr,
                             logits16_ ? s.logits16 : nullptr));
    } else {
      // EnsembleFactory::EnsemblesModels (src/decoder.h:1910-1931): mean of the members'
      // probabilities, renormalised -- written as log(mean p) so that the log-softmax of the
      // combined row IS the renormalisation; or the plain mean of log-probabilities.
      EnsembleRows er{};
      for (int mi = 0; mi < n_models; ++mi) er.logits[mi] = states_[mi].logits;
      er.n = n_models;
      if (int rc = kt(KC_COMBINE)) return rc;
      CK(tc::launch_k(pdl_, ensemble_combine_kernel, dim3(rows), dim3(256), 0, stream, er, Vp, V, (int)opt.ensemble_mode, d_combined_));
      LAUNCHED();
      if (int rc = kt(KC_SOFTMAX)) return rc;
      CK(launch_softmax_topk(d_combined_, Vp, V, kk, rows, o, opt.ensemble_mode == LINMT_ENS_PROB_MEAN ? 1 : 0, stream, pdl_));
    }
    LAUNCHED();
  }
  {
    BeamState bs{d_tok_, d_score_, d_parent_, d_hist_tok_, d_hist_parent_, d_fin_t_, d_fin_b_, d_fin_score_, d_fin_n_, fin_cap, R};
    const size_t smem = (size_t)k * kk * 24 + 16;
    if (int rc = kt(KC_SELECT)) return rc;
    CK(tc::launch_k(pdl_, beam_select_kernel, dim3(n_act), dim3(256), smem, stream, bs, (const int32_t*)d_cand_idx_, (const float*)d_cand_logp_,
                    (const float*)d_eos_logp_, (const int32_t*)d_steps_, (const int32_t*)d_orig_, t, k, opt.penalty, opt.diversity, trace_dev_));
    LAUNCHED();
    if (int rc = kt(KC_END)) return rc;
  }
  CK(cudaGetLastError());
  stats.decoder_row_steps += rows;
  stats.sentence_steps += n_act;
  return LINMT_OK;
}

// ---------------------------------------------------------------------------------------
// Decode of one device batch (n <= max_batch); every data pointer is a device pointer.
int Engine::decode_core(const int32_t* d_ids, const int32_t* off_host, int n, const int32_t* steps_host, int max_len,
                        int32_t* d_out_tok, int32_t* d_out_len, float* d_out_score, int32_t* d_out_vit, float* d_out_align,
                        const linmt_trace* trace_dev, int trace_Tm) {
  if (n < 1) return LINMT_OK;
  if (n > B) return fail(LINMT_ELIMIT, "batch larger than max_batch");
  // order by step count, longest first: the rows still decoding at any step are a prefix
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return steps_host[a] > steps_host[b]; });
  int32_t* m_off = h_meta_;
  int32_t* m_len = h_meta_ + (B + 1);
  int32_t* m_steps = h_meta_ + 2 * (B + 1);
  int32_t* m_orig = h_meta_ + 3 * (B + 1);
  int Smax = 0, Tm = 0;
  for (int i = 0; i < n; ++i) {
    const int s = order[i];
    const int len = off_host[s + 1] - off_host[s];
    if (len < 1) return fail(LINMT_EINVAL, "empty source sentence");
    if (len > opt.max_src_len) return fail(LINMT_ELIMIT, "source sentence longer than max_src_len");
    if (steps_host[s] < 0 || steps_host[s] > opt.max_steps) return fail(LINMT_ELIMIT, "step count outside 0..max_steps");
    m_off[i] = off_host[s]; m_len[i] = len; m_steps[i] = steps_host[s]; m_orig[i] = s;
    Smax = std::max(Smax, len); Tm = std::max(Tm, steps_host[s]);
  }
  if (max_len < Tm + 2) return fail(LINMT_EINVAL, "max_len smaller than max steps + 2");
  CK(cudaSetDevice(opt.device));
  CK(cudaEventRecord(ev0_, stream));
  CK(cudaMemcpyAsync(d_off_, m_off, sizeof(int32_t) * n, cudaMemcpyHostToDevice, stream));
  CK(cudaMemcpyAsync(d_len_, m_len, sizeof(int32_t) * n, cudaMemcpyHostToDevice, stream));
  CK(cudaMemcpyAsync(d_steps_, m_steps, sizeof(int32_t) * n, cudaMemcpyHostToDevice, stream));
  CK(cudaMemcpyAsync(d_orig_, m_orig, sizeof(int32_t) * n, cudaMemcpyHostToDevice, stream));
  CK(cudaMemsetAsync(d_tok_, 0, sizeof(int32_t) * R, stream));     // START = 0 (src/decoder.h:339-342)
  CK(cudaMemsetAsync(d_parent_, 0, sizeof(int32_t) * R, stream));
  CK(cudaMemsetAsync(d_score_, 0, sizeof(float) * R, stream));
  CK(cudaMemsetAsync(d_fin_n_, 0, sizeof(int32_t) * B, stream));
  cur_ids_ = d_ids;
  trace_dev_ = TraceDev{};
  if (trace_dev) {
    trace_dev_.cand_tok = trace_dev->cand_tok; trace_dev_.cand_logp = trace_dev->cand_logp;
    trace_dev_.surv_tok = trace_dev->surv_tok; trace_dev_.surv_parent = trace_dev->surv_parent;
    trace_dev_.surv_score = trace_dev->surv_score; trace_dev_.final_logp = trace_dev->final_logp;
    trace_dev_.force_tok = trace_dev->force_tok; trace_dev_.force_parent = trace_dev->force_parent;
    trace_dev_.force_score = trace_dev->force_score; trace_dev_.Tm = trace_Tm;
    trace_dev_.gold_logp = trace_dev->gold_logp;
    trace_dev_.pt = trace_dev->pt;
  }
  kt_used_ = 0; rec_flops_ = 0.0;
  int rc = use_tc_ ? run_encoder_tc(n, Smax) : run_encoder(n, Smax);
  if (rc) return rc;
  // the encoder's final states sit in buffer (Smax & 1)
  enc_final_buf_ = Smax & 1;
  const auto host_t0 = std::chrono::steady_clock::now();
  for (int t = 0; t <= Tm; ++t) {
    int n_act = 0;
    while (n_act < n && m_steps[n_act] >= t) ++n_act;
    if (n_act == 0) break;
    for (int mi = 0; mi < n_models; ++mi)
      if ((rc = use_tc_ ? run_decoder_step_tc(mi, t, n_act * k) : run_decoder_step(mi, t, n_act * k))) return rc;
    if ((rc = step_tail(t, n_act * k))) return rc;
  }
  {
    FinalizeArgs a{};
    a.bs = BeamState{d_tok_, d_score_, d_parent_, d_hist_tok_, d_hist_parent_, d_fin_t_, d_fin_b_, d_fin_score_, d_fin_n_, fin_cap, R};
    a.steps = d_steps_; a.src_len = d_len_; a.orig = d_orig_;
    a.rec_align = d_rec_align_; a.rec_lo = d_rec_lo_; a.rec_vit = d_rec_vit_;
    a.fin_final = d_fin_final_; a.win = rec_win; a.k = k; a.nbest = opt.nbest; a.max_len = max_len; a.max_src = opt.max_src_len;
    a.lp_alpha = opt.lp_alpha; a.cp_beta = opt.cp_beta; a.min_ratio = opt.min_ratio;
    a.out_tok = d_out_tok; a.out_len = d_out_len; a.out_score = d_out_score; a.out_vit = d_out_vit; a.out_align = d_out_align;
    const size_t smem = 4 * ((size_t)opt.max_src_len * sizeof(float) + (size_t)max_len * sizeof(int));
    finalize_kernel<<<n, 128, smem, stream>>>(a);
    LAUNCHED();
    CK(cudaGetLastError());
  }
  CK(cudaEventRecord(ev1_, stream));
  stats.last_host_issue_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
  return LINMT_OK;
}

int Engine::finish_timing() {
  CK(cudaStreamSynchronize(stream));
  if (use_tc_) {
    int herr = 0;
    CK(cudaMemcpy(&herr, d_tc_err_, sizeof(int), cudaMemcpyDeviceToHost));
    if (herr) return fail(LINMT_ECUDA, "a tensor-core GEMM gave up waiting on a barrier (results of this call are invalid)");
  }
  CK(cudaEventElapsedTime(&stats.last_decode_ms, ev0_, ev1_));
  for (int c = 0; c < KC_COUNT; ++c) { class_ms[c] = 0.f; class_launches[c] = 0; }
  for (size_t i = 0; i + 1 < kt_used_; ++i) {
    if (kt_cls_[i] == KC_END) continue;
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, kt_ev_[i], kt_ev_[i + 1]));
    class_ms[kt_cls_[i]] += ms;
    ++class_launches[kt_cls_[i]];
  }
  stats.last_gemm_ms = class_ms[KC_VOCAB];
  stats.last_gemm_launches = class_launches[KC_VOCAB];
  stats.last_rec_gemm_ms = class_ms[KC_LSTM];
  stats.last_rec_gemm_launches = class_launches[KC_LSTM];
  stats.last_rec_gemm_flops = rec_flops_;
  return LINMT_OK;
}

int Engine::kt(int cls) {
  if (!kernel_timing) return LINMT_OK;
  if (kt_used_ == kt_ev_.size()) { cudaEvent_t ev; CK(cudaEventCreate(&ev)); kt_ev_.push_back(ev); kt_cls_.push_back(0); }
  kt_cls_[kt_used_] = cls;
  CK(cudaEventRecord(kt_ev_[kt_used_++], stream));
  return LINMT_OK;
}

// Host-pointer front of decode_core: copies ids in, results out, in chunks of max_batch.
int Engine::decode_host(const int32_t* src_ids, const int32_t* src_off, int n, const int32_t* steps, int max_len,
                        int32_t* out_tok, int32_t* out_len, float* out_score, int32_t* out_vit, float* out_align,
                        const linmt_trace* trace) {
  if (n < 0 || !src_ids || !src_off || !steps || !out_tok || !out_len || !out_score) return fail(LINMT_EINVAL, "null argument");
  if (out_align && !opt.print_info) return fail(LINMT_EINVAL, "alignments need print_info = 1");
  CK(cudaSetDevice(opt.device));
  const int nb = opt.nbest;
  int Tm_all = 0;
  for (int i = 0; i < n; ++i) Tm_all = std::max(Tm_all, steps[i]);
  float total_ms = 0.f, gemm_ms = 0.f;
  int gemm_launches = 0;
  for (int c0 = 0; c0 < n; c0 += B) {
    const int cn = std::min(B, n - c0);
    const int32_t base = src_off[c0];
    const size_t n_ids = (size_t)(src_off[c0 + cn] - base);
    // staging buffers grow with the longest input seen; the outgrown buffer is freed (the previous chunk's
    // work on it ended with the synchronisation in finish_timing)
    if (n_ids > d_ids_cap_) {
      if (int rc_ = regrow(&d_ids_, n_ids + 1024)) return rc_;
      d_ids_cap_ = n_ids + 1024;
    }
    const size_t need = (size_t)cn * nb;
    if (need > out_cap_len_ || max_len > out_cap_maxlen_) {
      const size_t ml = std::max<size_t>(max_len, out_cap_maxlen_);
      const size_t cap = std::max<size_t>(need, (size_t)B * nb);
      int rc_;
      if ((rc_ = regrow(&d_out_tok_, cap * ml)) || (rc_ = regrow(&d_out_vit_, cap * ml)) || (rc_ = regrow(&d_out_len_, cap)) ||
          (rc_ = regrow(&d_out_score_, cap)))
        return rc_;
      if (opt.print_info && (rc_ = regrow(&d_out_align_, cap * ml * opt.max_src_len))) return rc_;
      out_cap_len_ = cap; out_cap_maxlen_ = ml;
    }
    CK(cudaMemcpyAsync(d_ids_, src_ids + base, n_ids * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
    std::vector<int32_t> off(cn + 1);
    for (int i = 0; i <= cn; ++i) off[i] = src_off[c0 + i] - base;
    // per-chunk device trace buffers
    linmt_trace td{};
    std::vector<std::pair<void*, std::pair<void*, size_t>>> copy_back;  // (device, (host, bytes))
    if (trace) {
      for (void* p : trace_allocs_) cudaFree(p);
      trace_allocs_.clear();
      const size_t n_c = (size_t)cn * Tm_all * k * kk, n_s = (size_t)cn * Tm_all * k, n_f = (size_t)cn * k;
      auto mk = [&](size_t count, size_t esz, void* host_dst, const void* host_src, void** dev) -> int {
        if (!host_dst && !host_src) { *dev = nullptr; return LINMT_OK; }
        void* q = nullptr;
        if (cudaMalloc(&q, std::max<size_t>(count, 1) * esz) != cudaSuccess) return fail(LINMT_ENOMEM, "trace buffer allocation failed");
        trace_allocs_.push_back(q);
        if (host_src) {
          if (cudaMemcpyAsync(q, host_src, count * esz, cudaMemcpyHostToDevice, stream) != cudaSuccess) return fail(LINMT_ECUDA, "trace upload failed");
        } else {
          if (cudaMemsetAsync(q, 0xff, count * esz, stream) != cudaSuccess) return fail(LINMT_ECUDA, "trace clear failed");
          copy_back.push_back({q, {host_dst, count * esz}});
        }
        *dev = q;
        return LINMT_OK;
      };
      int rc;
      if ((rc = mk(n_c, 4, trace->cand_tok ? trace->cand_tok + (size_t)c0 * Tm_all * k * kk : nullptr, nullptr, (void**)&td.cand_tok))) return rc;
      if ((rc = mk(n_c, 4, trace->cand_logp ? trace->cand_logp + (size_t)c0 * Tm_all * k * kk : nullptr, nullptr, (void**)&td.cand_logp))) return rc;
      if ((rc = mk(n_s, 4, trace->surv_tok ? trace->surv_tok + (size_t)c0 * Tm_all * k : nullptr, nullptr, (void**)&td.surv_tok))) return rc;
      if ((rc = mk(n_s, 4, trace->surv_parent ? trace->surv_parent + (size_t)c0 * Tm_all * k : nullptr, nullptr, (void**)&td.surv_parent))) return rc;
      if ((rc = mk(n_s, 4, trace->surv_score ? trace->surv_score + (size_t)c0 * Tm_all * k : nullptr, nullptr, (void**)&td.surv_score))) return rc;
      if ((rc = mk(n_f, 4, trace->final_logp ? trace->final_logp + (size_t)c0 * k : nullptr, nullptr, (void**)&td.final_logp))) return rc;
      if ((rc = mk(n_s, 4, trace->gold_logp ? trace->gold_logp + (size_t)c0 * Tm_all * k : nullptr, nullptr, (void**)&td.gold_logp))) return rc;
      // p_t: one [cn][Tm+1][k] block per member on the device, copied back member by member into [n_models][n][Tm+1][k]
      const size_t n_pt = (size_t)cn * (Tm_all + 1) * k;
      td.pt = nullptr;
      if (trace->pt) {
        void* q = nullptr;
        if (cudaMalloc(&q, std::max<size_t>(n_pt * n_models, 1) * 4) != cudaSuccess) return fail(LINMT_ENOMEM, "trace buffer allocation failed");
        trace_allocs_.push_back(q);
        if (cudaMemsetAsync(q, 0xff, n_pt * n_models * 4, stream) != cudaSuccess) return fail(LINMT_ECUDA, "trace clear failed");
        td.pt = static_cast<float*>(q);
        trace_pt_member_stride_ = n_pt;
        for (int mi = 0; mi < n_models; ++mi)
          copy_back.push_back({td.pt + (size_t)mi * n_pt,
                               {trace->pt + ((size_t)mi * n + c0) * (Tm_all + 1) * k, n_pt * 4}});
      }
      if ((rc = mk(n_s, 4, nullptr, trace->force_tok ? trace->force_tok + (size_t)c0 * Tm_all * k : nullptr, (void**)&td.force_tok))) return rc;
      if ((rc = mk(n_s, 4, nullptr, trace->force_parent ? trace->force_parent + (size_t)c0 * Tm_all * k : nullptr, (void**)&td.force_parent))) return rc;
      if ((rc = mk(n_s, 4, nullptr, trace->force_score ? trace->force_score + (size_t)c0 * Tm_all * k : nullptr, (void**)&td.force_score))) return rc;
    }
    int rc = decode_core(d_ids_, off.data(), cn, steps + c0, max_len, d_out_tok_, d_out_len_, d_out_score_,
                         out_vit ? d_out_vit_ : nullptr, out_align ? d_out_align_ : nullptr, trace ? &td : nullptr, Tm_all);
    if (rc) return rc;
    CK(cudaMemcpyAsync(out_tok + (size_t)c0 * nb * max_len, d_out_tok_, need * max_len * 4, cudaMemcpyDeviceToHost, stream));
    CK(cudaMemcpyAsync(out_len + (size_t)c0 * nb, d_out_len_, need * 4, cudaMemcpyDeviceToHost, stream));
    CK(cudaMemcpyAsync(out_score + (size_t)c0 * nb, d_out_score_, need * 4, cudaMemcpyDeviceToHost, stream));
    if (out_vit) CK(cudaMemcpyAsync(out_vit + (size_t)c0 * nb * max_len, d_out_vit_, need * max_len * 4, cudaMemcpyDeviceToHost, stream));
    if (out_align)
      CK(cudaMemcpyAsync(out_align + (size_t)c0 * nb * max_len * opt.max_src_len, d_out_align_,
                         need * max_len * opt.max_src_len * 4, cudaMemcpyDeviceToHost, stream));
    for (auto& cb : copy_back) CK(cudaMemcpyAsync(cb.second.first, cb.first, cb.second.second, cudaMemcpyDeviceToHost, stream));
    if ((rc = finish_timing())) return rc;
    total_ms += stats.last_decode_ms; gemm_ms += stats.last_gemm_ms; gemm_launches += stats.last_gemm_launches;
  }
  stats.last_decode_ms = total_ms; stats.last_gemm_ms = gemm_ms; stats.last_gemm_launches = gemm_launches;
  return LINMT_OK;
}

int run_on_engines(linmt_engine* h, const std::vector<int>& order, const std::function<int(Engine&, int)>& job) {
  const int ne = h->n_engines();
  if (ne == 1 || order.size() <= 1) {
    for (int item : order)
      if (int rc = job(h->eng, item)) return rc;
    return LINMT_OK;
  }
  std::atomic<size_t> next{0};
  std::atomic<int> first_rc{LINMT_OK};
  std::mutex err_mutex;
  std::string err_text;
  auto worker = [&](int ei) {
    Engine& g = h->engine(ei);
    while (first_rc.load() == LINMT_OK) {
      const size_t i = next.fetch_add(1);
      if (i >= order.size()) break;
      const int rc = job(g, order[i]);
      if (rc != LINMT_OK) {
        std::lock_guard<std::mutex> lock(err_mutex);
        if (first_rc.load() == LINMT_OK) { first_rc.store(rc); err_text = g.err; }
      }
    }
  };
  std::vector<std::thread> threads;
  for (int ei = 1; ei < ne; ++ei) threads.emplace_back(worker, ei);
  worker(0);
  for (auto& t : threads) t.join();
  if (first_rc.load() != LINMT_OK) h->eng.err = err_text;
  return first_rc.load();
}

}  // namespace linmt

// =========================================================================================
// C ABI (numeric part; the sentence front-end lives in frontend.cpp)
// =========================================================================================
using linmt::Engine;


static std::string g_create_error;

extern "C" {

void linmt_default_options(linmt_options* o) {
  std::memset(o, 0, sizeof(*o));
  o->beam = 12; o->nbest = 1; o->attention_mode = LINMT_ATT_LOCAL_P_GENERAL; o->attention_d = 10;
  o->print_info = 0; o->precision = LINMT_PREC_FP32; o->ensemble_mode = LINMT_ENS_PROB_MEAN; o->gemm_path = LINMT_GEMM_AUTO;
  o->max_batch = 64; o->max_src_len = 100; o->max_steps = 200; o->device = 0;
  o->penalty = 0.f; o->diversity = 0.f; o->lp_alpha = 0.65f; o->cp_beta = 0.20f; o->min_ratio = 0.5f; o->max_ratio = 1.5f;
}

size_t linmt_blob_floats(const linmt_model_desc* d) {
  const size_t H = d->hidden, hh = H * H, L = d->layers;
  size_t n = 0;
  n += 8 * hh + 4 * H + H * (size_t)d->vocab_src;
  n += (L - 1) * (8 * hh + 4 * H);
  n += 8 * hh + 4 * H + H * (size_t)d->vocab_tgt + (d->feed_input ? 4 * hh : 0);
  n += (L - 1) * (8 * hh + 4 * H);
  n += 4 * hh + 2 * H;
  n += (size_t)d->vocab_tgt * H + d->vocab_tgt;
  return n;
}

int linmt_create_from_weights_on(const linmt_model_desc* desc, const float* const* blobs, int32_t n_models, size_t blob_floats,
                                 const linmt_options* opt, const int32_t* devices, int32_t n_devices, linmt_engine** out) {
  if (!desc || !blobs || !opt || !out || (n_devices > 0 && !devices)) { g_create_error = "null argument"; return LINMT_EINVAL; }
  *out = nullptr;
  if (n_devices > 64) { g_create_error = "at most 64 devices"; return LINMT_ELIMIT; }
  for (int i = 0; i < n_devices; ++i)
    for (int j = 0; j < i; ++j)
      if (devices[i] == devices[j]) { g_create_error = "a device is listed twice"; return LINMT_EINVAL; }
  linmt_engine* e = new (std::nothrow) linmt_engine();
  if (!e) { g_create_error = "out of host memory"; return LINMT_ENOMEM; }
  const int nd = n_devices > 0 ? n_devices : 1;
  for (int i = 0; i < nd; ++i) {
    linmt_options o = *opt;
    if (n_devices > 0) o.device = devices[i];
    Engine* g = &e->eng;
    if (i > 0) { e->replicas.emplace_back(new (std::nothrow) Engine()); g = e->replicas.back().get(); }
    int rc = g ? g->init(*desc, blobs, n_models, blob_floats, o) : LINMT_ENOMEM;
    if (rc != LINMT_OK) {
      g_create_error = g ? g->err : "out of host memory";
      delete e;
      return rc;
    }
  }
  *out = e;
  return LINMT_OK;
}

int linmt_create_from_weights(const linmt_model_desc* desc, const float* const* blobs, int32_t n_models, size_t blob_floats,
                              const linmt_options* opt, linmt_engine** out) {
  return linmt_create_from_weights_on(desc, blobs, n_models, blob_floats, opt, nullptr, 0, out);
}

int32_t linmt_device_count(const linmt_engine* e) { return e ? e->n_engines() : 0; }

void linmt_destroy(linmt_engine* e) { delete e; }

const char* linmt_last_error(const linmt_engine* e) { return e ? e->eng.err.c_str() : g_create_error.c_str(); }

int32_t linmt_beam(const linmt_engine* e) { return e ? e->eng.k : 0; }

int linmt_decode_batch(linmt_engine* e, const int32_t* src_ids, const int32_t* src_off, int32_t n, const int32_t* steps,
                       int32_t max_len, int32_t* out_tok, int32_t* out_len, float* out_score, int32_t* out_vit,
                       float* out_align, const linmt_trace* trace) {
  if (!e) return LINMT_EINVAL;
  Engine& g0 = e->eng;
  const int B = g0.B;
  if (e->n_engines() == 1 || trace || n <= B || !src_ids || !src_off || !steps || !out_tok || !out_len || !out_score)
    return g0.decode_host(src_ids, src_off, n, steps, max_len, out_tok, out_len, out_score, out_vit, out_align, trace);
  // several devices: the job is cut into device batches of consecutive sentences; each device's host thread
  // takes the next batch when it is free, the batches with the most decoder forwards first
  const int nchunks = (n + B - 1) / B;
  std::vector<long long> cost(nchunks, 0);
  for (int c = 0; c < nchunks; ++c) {
    int tm = 0;
    const int cn = std::min(B, n - c * B);
    for (int i = 0; i < cn; ++i) tm = std::max(tm, steps[c * B + i]);
    cost[c] = (long long)(tm + 1) * cn;
  }
  std::vector<int> order(nchunks);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  const size_t nb = (size_t)g0.opt.nbest, ml = (size_t)max_len, ms = (size_t)g0.opt.max_src_len;
  std::vector<float> ms_per_engine(e->n_engines(), 0.f);
  std::mutex stat_mutex;
  int rc = linmt::run_on_engines(e, order, [&](Engine& g, int c) -> int {
    const size_t c0 = (size_t)c * B;
    const int cn = std::min(B, n - (int)c0);
    int r = g.decode_host(src_ids, src_off + c0, cn, steps + c0, max_len, out_tok + c0 * nb * ml, out_len + c0 * nb,
                          out_score + c0 * nb, out_vit ? out_vit + c0 * nb * ml : nullptr,
                          out_align ? out_align + c0 * nb * ml * ms : nullptr, nullptr);
    if (r == LINMT_OK) {
      std::lock_guard<std::mutex> lock(stat_mutex);
      for (int i = 0; i < e->n_engines(); ++i)
        if (&e->engine(i) == &g) ms_per_engine[i] += g.stats.last_decode_ms;
    }
    return r;
  });
  if (rc != LINMT_OK) return rc;
  // device time of the call = the busiest device's; the counters of the replicas are folded into the handle's
  g0.stats.last_decode_ms = *std::max_element(ms_per_engine.begin(), ms_per_engine.end());
  return LINMT_OK;
}

int linmt_decode_batch_device(linmt_engine* e, const int32_t* d_src_ids, const int32_t* src_off_host, int32_t n,
                              const int32_t* steps_host, int32_t max_len, int32_t* d_out_tok, int32_t* d_out_len,
                              float* d_out_score) {
  if (!e) return LINMT_EINVAL;
  int rc = e->eng.decode_core(d_src_ids, src_off_host, n, steps_host, max_len, d_out_tok, d_out_len, d_out_score, nullptr,
                              nullptr, nullptr, 0);
  if (rc) return rc;
  return e->eng.finish_timing();
}

int linmt_score_batch(linmt_engine* e, const int32_t* src_ids, const int32_t* src_off, const int32_t* tgt_ids,
                      const int32_t* tgt_off, int32_t n, float* out_logprob, float* out_token_logp, int32_t max_tgt) {
  if (!e || !src_ids || !src_off || !tgt_ids || !tgt_off || !out_logprob || n < 0) return LINMT_EINVAL;
  Engine& g = e->eng;
  if (g.n_models > 1 && g.opt.ensemble_mode != LINMT_ENS_PROB_MEAN) { g.err = "scoring supports single models and prob_mean ensembles"; return LINMT_EINVAL; }
  const int k = g.k;
  int Tm = 0;
  std::vector<int32_t> steps(n);
  for (int i = 0; i < n; ++i) {
    steps[i] = tgt_off[i + 1] - tgt_off[i];
    if (steps[i] < 1 || steps[i] > g.opt.max_steps) { g.err = "target length outside 1..max_steps"; return LINMT_ELIMIT; }
    Tm = std::max(Tm, steps[i]);
  }
  if (out_token_logp && max_tgt < Tm) { g.err = "max_tgt smaller than the longest target"; return LINMT_EINVAL; }
  // every beam slot is forced to the given token: slot b continues slot b
  std::vector<int32_t> ftok((size_t)n * Tm * k, 2), fpar((size_t)n * Tm * k, 0);
  std::vector<float> fscore((size_t)n * Tm * k, 0.f), gold((size_t)n * Tm * k, 0.f), fin((size_t)n * k, 0.f);
  for (int i = 0; i < n; ++i)
    for (int t = 0; t < steps[i]; ++t)
      for (int b = 0; b < k; ++b) {
        const size_t off = ((size_t)i * Tm + t) * k + b;
        ftok[off] = tgt_ids[tgt_off[i] + t];
        fpar[off] = b;
      }
  linmt_trace tr{};
  tr.force_tok = ftok.data(); tr.force_parent = fpar.data(); tr.force_score = fscore.data();
  tr.gold_logp = gold.data(); tr.final_logp = fin.data();
  const int max_len = Tm + 2, nb = g.opt.nbest;
  std::vector<int32_t> tok((size_t)n * nb * max_len), len((size_t)n * nb);
  std::vector<float> score((size_t)n * nb);
  int rc = g.decode_host(src_ids, src_off, n, steps.data(), max_len, tok.data(), len.data(), score.data(), nullptr, nullptr, &tr);
  if (rc != LINMT_OK) return rc;
  for (int i = 0; i < n; ++i) {
    float sum = 0.f;
    for (int t = 0; t < steps[i]; ++t) {
      const float lp = gold[((size_t)i * Tm + t) * k];
      sum += lp;
      if (out_token_logp) out_token_logp[(size_t)i * (max_tgt + 1) + t] = lp;
    }
    const float le = fin[(size_t)i * k];
    sum += le;
    if (out_token_logp) {
      out_token_logp[(size_t)i * (max_tgt + 1) + steps[i]] = le;
      for (int t = steps[i] + 1; t <= max_tgt; ++t) out_token_logp[(size_t)i * (max_tgt + 1) + t] = 0.f;
    }
    out_logprob[i] = sum;
  }
  return LINMT_OK;
}

int linmt_get_stats(const linmt_engine* e, linmt_stats* out) {
  if (!e || !out) return LINMT_EINVAL;
  *out = e->eng.stats;
  for (const auto& r : e->replicas) {   // launches and forwards of every device
    out->kernel_launches += r->stats.kernel_launches;
    out->pair_launches += r->stats.pair_launches;
    out->decoder_row_steps += r->stats.decoder_row_steps;
    out->sentence_steps += r->stats.sentence_steps;
  }
  return LINMT_OK;
}

int linmt_kernel_times(const linmt_engine* e, float* ms, int32_t* launches, int32_t n) {
  if (!e || !ms || !launches || n < linmt::KC_COUNT) return LINMT_EINVAL;
  for (int c = 0; c < linmt::KC_COUNT; ++c) { ms[c] = e->eng.class_ms[c]; launches[c] = e->eng.class_launches[c]; }
  return LINMT_OK;
}

int linmt_set_kernel_timing(linmt_engine* e, int32_t on) {
  if (!e) return LINMT_EINVAL;
  e->eng.kernel_timing = on != 0;
  return LINMT_OK;
}

}  // extern "C"

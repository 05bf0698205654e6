// engine_tc.cu -- the tensor-core path of the engine: operands as bf16 planes, every GEMM a
// tcgen05/TMEM kernel fed by TMA, LSTM cell / tanh / bias fused into the epilogues.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "engine.h"
#include "gemm_tc.cuh"
#include "gemm_tc_pair.cuh"
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

int Engine::alloc_planes(tc::Planes& p, size_t rows, int ld) {
  p = tc::Planes{};
  p.ld = ld;
  p.fmt = fmt_;
  for (int t = 0; t < nt_; ++t) {
    void* q = nullptr;
    const size_t bytes = rows * (size_t)ld * sizeof(__nv_bfloat16);
    if (cudaMalloc(&q, bytes ? bytes : 2) != cudaSuccess) return fail(LINMT_ENOMEM, "cudaMalloc failed (operand planes)");
    allocs_.push_back(q);
    if (cudaMemset(q, 0, bytes) != cudaSuccess) return fail(LINMT_ECUDA, "cudaMemset failed (operand planes)");
    p.p[t] = static_cast<__nv_bfloat16*>(q);
  }
  return LINMT_OK;
}

// fp32 host matrix -> device -> bf16 planes (the split runs on the GPU).
int Engine::to_planes(const std::vector<float>& host, size_t rows, int ld, tc::Planes& dst) {
  int rc = alloc_planes(dst, rows, ld);
  if (rc) return rc;
  float* tmp = nullptr;
  const size_t n = rows * (size_t)ld;
  if (host.size() < n) return fail(LINMT_EINVAL, "internal: packed matrix smaller than its planes");
  if (cudaMalloc(&tmp, n * sizeof(float)) != cudaSuccess) return fail(LINMT_ENOMEM, "cudaMalloc failed (weight staging)");
  // stream-ordered copy: the split kernel must not start before the last byte has landed
  cudaError_t e = cudaMemcpyAsync(tmp, host.data(), n * sizeof(float), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) {
    tc::split_planes_kernel<<<2048, 256, 0, stream>>>(tmp, dst, nt_, n);
    LAUNCHED();
    e = cudaStreamSynchronize(stream);
  }
  cudaFree(tmp);
  if (e != cudaSuccess) return fail(LINMT_ECUDA, std::string("weight split: ") + cudaGetErrorString(e));
  return LINMT_OK;
}

int Engine::alloc_state_tc(TcState& s) {
  int rc;
  if ((rc = alloc_planes(s.panel1, R, 3 * Hp))) return rc;
  s.panel.resize(L);
  for (int l = 1; l < L; ++l)
    if ((rc = alloc_planes(s.panel[l], R, 2 * Hp))) return rc;
  if ((rc = alloc_planes(s.panel_top, R, 2 * Hp))) return rc;
  if ((rc = alloc_planes(s.panel_ht, R, Hp))) return rc;
  if (att_fold_ && (rc = alloc_planes(s.hs_planes, (size_t)B * opt.max_src_len, Hp))) return rc;
  for (int i = 0; i < 2; ++i) {
    s.encp[i].resize(L);
    for (int l = 0; l < L; ++l)
      if ((rc = alloc_planes(s.encp[i][l], B, 2 * Hp))) return rc;
  }
  return LINMT_OK;
}

// Tensor maps are built once per (buffer view, shape) and reused by every launch.
const CUtensorMap* Engine::a_maps(const tc::Planes& p, int col0, int rows_cap, int K, int bk) {
  auto key = std::make_tuple((const void*)(p.p[0] + col0), rows_cap, K, p.ld, (int)tc::BM + 1000 * bk);
  auto it = tmap_cache_.find(key);
  if (it == tmap_cache_.end()) {
    std::array<CUtensorMap, 3> m{};
    for (int t = 0; t < nt_; ++t)
      if (!tc::make_tmap(&m[t], p.p[t] + col0, rows_cap, K, p.ld, tc::BM, bk)) return nullptr;
    it = tmap_cache_.emplace(key, m).first;
  }
  return it->second.data();
}
const CUtensorMap* Engine::b_maps(const tc::Planes& p, int rows, int K, int bn, int bk) {
  auto key = std::make_tuple((const void*)p.p[0], rows, K, p.ld, bn + 1000 * bk);
  auto it = tmap_cache_.find(key);
  if (it == tmap_cache_.end()) {
    std::array<CUtensorMap, 3> m{};
    for (int t = 0; t < nt_; ++t)
      if (!tc::make_tmap(&m[t], p.p[t], rows, K, p.ld, bn, bk)) return nullptr;
    it = tmap_cache_.emplace(key, m).first;
  }
  return it->second.data();
}

// C[M][N] = A[:, a_col0 : a_col0+K] . W[N][K]^T with the tile width chosen for this shape.
template <class Epi>
int Engine::tc_gemm(const tc::Planes& A, int a_col0, int a_rows_cap, const tc::Planes& W, int M, int N, int K, const Epi& e_in, int nt, int drain) {
  Epi e = e_in;
  if (nt <= 0 || nt > nt_) nt = nt_;
  int bn = 0, splits = 1;
  // a layer's slice of the split-K workspace: whole 256-byte units, so that every slice starts aligned for the
  // 16-byte partial-tile stores whatever the number of layers sharing it
  const size_t ws_floats = (kSplitKWsFloats / ws_parts_) & ~(size_t)63;
  const int max_tiles = kSplitKMaxTiles / ws_parts_;
  // The encoder runs its L layers as a wavefront on L streams: a GEMM sized for the whole machine would only
  // queue behind its neighbours, so there each one is shaped for its share of the SMs and they run side by side.
  const int sm_budget = ws_parts_ > 1 ? (n_sm_ / ws_parts_ > 0 ? n_sm_ / ws_parts_ : 1) : n_sm_;
  tc::pick_shape(M, N, K, nt, sm_budget, ws_floats, max_tiles, &bn, &splits, fmt_);
  // one plane (bf16 precision): 64-deep stages with 128-byte rows halve the per-k-block overheads
  // (measured 1.5x on the gate GEMMs); with split operands only 32-deep stages leave room for a ring
  // the f16 pair: 64-deep stages as well, except for a weight matrix far larger than L2 under
  // the widest tiles, where only two such stages fit and four 32-deep ones hide DRAM latency better
  // (vocabulary GEMM: 143 us against 149 us)
  int bk = (nt == 1) ? 64 : 32;
  if (fmt_ == 1 && nt == 2 && K % 64 == 0) bk = (bn >= 240 && (size_t)N * K * 4 > ((size_t)96 << 20)) ? 32 : 64;
  // CTA pairs (gemm_tc_pair.cuh) where the one-tile shape has room for two stages only: an even number of row
  // tiles (an odd one is rounded up, which must still fit one wave), split operands, 64-deep stages, K not split
  const int mt = (M + tc::BM - 1) / tc::BM;
  // The many-wave one-plane logits GEMM has a persistent pair form as well: worth it for an even number of row tiles
  // (measured at N = 30016, K = 1024: 56.2 against 61.7 us at 768 rows, 24.5 against 27.7 at 192; an odd number of
  // row tiles wastes half a pair and loses), with 208-wide tiles.
  const bool one_plane_logits = nt == 1 && Epi::kHasPmax;   // the fp32-output GEMMs: vocabulary projection
  bool ppair = false;
  if (pair_ && persist_ && one_plane_logits && splits == 1 && bk == 64 && mt % 2 == 0 && ws_parts_ == 1 &&
      (long)mt * ((N + bn - 1) / bn) > n_sm_ && (long)(mt / 2) * ((N + 207) / 208) > n_sm_ / 2) {
    ppair = true;
    bn = 208;
  }
  const long ntile_cols = (N + bn - 1) / bn;
  const bool pair = ppair || (pair_ && fmt_ == 1 && nt == 2 && bk == 64 && splits == 1 && mt >= 2 && bn % 16 == 0 &&
                    tc::make_shape(bn, nt, bk, fmt_).stages < 3 && (long)((mt + 1) & ~1) * ntile_cols <= n_sm_ && ws_parts_ == 1);
  const CUtensorMap* am = a_maps(A, a_col0, a_rows_cap, K, bk);
  const CUtensorMap* bm = b_maps(W, N, K, pair ? bn / 2 : bn, bk);
  if (!am || !bm) return fail(LINMT_ECUDA, "cuTensorMapEncodeTiled failed");
  tc::TmapSet tm;
  std::memcpy(tm.a, am, sizeof(tm.a));
  std::memcpy(tm.b, bm, sizeof(tm.b));
  tc::Shape sh = pair ? tc::make_shape_pair(bn, nt, bk, fmt_) : tc::make_shape(bn, nt, bk, fmt_);
  sh.splits = splits;
  if (drain > 0) sh.drain = drain;
  sh.pdl = (pdl_ && pdl_gemm_) ? 1 : 0;
  if constexpr (Epi::kHasPmax) {
    // block maxima for the softmax: four column blocks per tile; not from the split-K fix-up path
    if (e.pmax) {
      const int slots = 4 * ((N + bn - 1) / bn);
      if (splits > 1 || slots > e.pmax_ld) { e.pmax = nullptr; pmax_slots_ = 0; }
      else pmax_slots_ = slots;
    }
  }
  // many waves of tiles whose leading product is one chain: one persistent CTA per SM
  const long tiles = (long)((M + tc::BM - 1) / tc::BM) * ((N + bn - 1) / bn);
  if (ppair) {
    const int pdl = sh.pdl;
    sh = tc::make_shape_persist_pair(bn, nt, bk, fmt_);
    sh.pdl = pdl;
    if (fmt_ == 1) CK((tc::launch_gemm_tc_persist_pair<1, 64, 1, Epi>(tm, M, N, K, sh, e, d_tc_err_, stream, n_sm_)));
    else CK((tc::launch_gemm_tc_persist_pair<1, 64, 0, Epi>(tm, M, N, K, sh, e, d_tc_err_, stream, n_sm_)));
    LAUNCHED();
    ++stats.pair_launches;
    return LINMT_OK;
  }
  if (persist_ && splits == 1 && tiles > n_sm_ && ((nt == 2 && drain >= K / 32) || one_plane_logits)) {
    if (nt == 1) {
      const int pdl = sh.pdl;
      sh = tc::make_shape_persist(bn, nt, bk, fmt_);   // a ring of one stage less, staging areas of its own
      sh.pdl = pdl;
    }
    CK(tc::launch_gemm_tc_persist(tm, M, N, K, sh, e, d_tc_err_, stream, n_sm_));
    LAUNCHED();
    return LINMT_OK;
  }
  if (pair) {
    CK((tc::launch_gemm_tc_pair<2, 64, 1, Epi>(tm, M, N, K, sh, e, d_tc_err_, stream, nullptr, nullptr)));
    LAUNCHED();
    ++stats.pair_launches;
    return LINMT_OK;
  }
  CK(tc::launch_gemm_tc(tm, M, N, K, sh, e, d_tc_err_, stream, d_splitk_ws_ + (size_t)ws_part_ * ws_floats,
                        d_splitk_counters_ + ws_part_ * max_tiles));
  LAUNCHED();
  return LINMT_OK;
}

bool Engine::pairs_available() { return tc::max_resident_pairs<2, 64, 1, tc::TcEpiLstm>() > 0; }

static tc::Planes no_planes() { return tc::Planes{}; }

// Input-term table of the first decoder layer: dec_xw[v][:] = W_x . embedding(v) for every target word, computed
// once with the same tensor GEMM (W_x = the first Hp of the K columns of the layer's weight planes).
int Engine::build_xw_tables() {
  for (int mi = 0; mi < n_models; ++mi) {
    DevModel& m = models_[mi];
    void* q = nullptr;
    const size_t bytes = (size_t)desc.vocab_tgt * 4 * Hp * sizeof(float);
    if (cudaMalloc(&q, bytes) != cudaSuccess) return fail(LINMT_ENOMEM, "cudaMalloc failed (input-term table)");
    allocs_.push_back(q);
    m.dec_xw = static_cast<float*>(q);
    tc::TcEpiF32 e{nullptr, m.dec_xw, 4 * Hp, 0};
    pdl_gemm_ = false;
    int rc = tc_gemm(m.p_emb_tgt, 0, desc.vocab_tgt, m.p_dec_w[0], desc.vocab_tgt, 4 * Hp, Hp, e);
    if (rc) return rc;
  }
  CK(cudaStreamSynchronize(stream));
  int herr = 0;
  CK(cudaMemcpy(&herr, d_tc_err_, sizeof(int), cudaMemcpyDeviceToHost));
  if (herr) return fail(LINMT_ECUDA, "a tensor-core GEMM gave up waiting on a barrier while building the input-term table");
  return LINMT_OK;
}

// Encoder, tensor-core path (see Engine::run_encoder for the reference procedure).  Panel of
// layer l at position p: encp[p&1][l] = (input from below | h_prev).  The epilogue writes h to
// the next position's h_prev slot and to the next layer's input slot of this position.
//
// (layer l, position p) depends on (l-1, p) and (l, p-1) only, and each launch fills about half
// the SMs (64 rows = one row tile), so the layers run as a wavefront: one stream per layer,
// events for the cross-layer edges.  Besides the true dependencies, (l, p) waits for (l+1, p-2),
// the last reader of the double-buffered input slot it overwrites.
int Engine::run_encoder_tc(int n, int Smax) {
  constexpr int kRing = 4;
  if (enc_streams_.empty()) {
    enc_streams_.resize(L);
    enc_events_.assign(L, std::vector<cudaEvent_t>(kRing));
    for (int l = 0; l < L; ++l) {
      CK(cudaStreamCreateWithFlags(&enc_streams_[l], cudaStreamNonBlocking));
      for (int r = 0; r < kRing; ++r) CK(cudaEventCreateWithFlags(&enc_events_[l][r], cudaEventDisableTiming));
    }
    CK(cudaEventCreateWithFlags(&enc_start_ev_, cudaEventDisableTiming));
  }
  cudaStream_t main_stream = stream;
  pdl_gemm_ = false;
  for (int mi = 0; mi < n_models; ++mi) {
    DevModel& m = models_[mi];
    DevState& s = states_[mi];
    TcState& ts = tc_states_[mi];
    for (int l = 0; l < L; ++l) {
      CK(cudaMemsetAsync(s.enc_c[0][l], 0, sizeof(float) * (size_t)B * Hp, main_stream));
      for (int t = 0; t < nt_; ++t)  // h_prev = 0 at the first position
        CK(cudaMemset2DAsync(ts.encp[0][l].p[t] + Hp, (size_t)2 * Hp * 2, 0, (size_t)Hp * 2, B, main_stream));
    }
    CK(cudaEventRecord(enc_start_ev_, main_stream));
    for (int l = 0; l < L; ++l) CK(cudaStreamWaitEvent(enc_streams_[l], enc_start_ev_, 0));
    int rc = LINMT_OK;
    for (int pos = 0; pos < Smax && rc == LINMT_OK; ++pos) {
      const int in = pos & 1, out = in ^ 1;
      for (int l = 0; l < L && rc == LINMT_OK; ++l) {
        cudaStream_t sl = enc_streams_[l];
        if (l > 0) CK(cudaStreamWaitEvent(sl, enc_events_[l - 1][pos % kRing], 0));
        if (l + 1 < L && pos >= 2) CK(cudaStreamWaitEvent(sl, enc_events_[l + 1][(pos - 2) % kRing], 0));
        if (l == 0) {
          dim3 grid(n, nt_);
          enc_embed_planes_kernel<<<grid, 128, 0, sl>>>(cur_ids_, d_off_, d_len_, m.p_emb_src, desc.vocab_src, ts.encp[in][0], Hp, pos);
          LAUNCHED();
        }
        tc::TcEpiLstm e{};
        e.bias = m.enc_b[l]; e.c_prev = s.enc_c[in][l]; e.ldc = Hp; e.c_out = s.enc_c[out][l];
        e.h_out1 = ts.encp[out][l]; e.h1_col0 = Hp;
        if (l + 1 < L) { e.h_out2 = ts.encp[in][l + 1]; e.h2_col0 = 0; } else { e.h_out2 = no_planes(); e.h2_col0 = 0; }
        e.h_prev = ts.encp[in][l]; e.hp_col0 = Hp;
        e.h_f32 = (l == L - 1) ? s.hs + (size_t)pos * Hp : nullptr;
        e.hf_row_stride = (long long)opt.max_src_len * Hp;
        e.row_len = d_len_; e.pos = pos; e.nt = nt_;
        stream = sl;  // tc_gemm launches on the member stream, with this layer's slice of the split-K workspace
        ws_part_ = l; ws_parts_ = L;
        rc = tc_gemm(ts.encp[in][l], 0, B, m.p_enc_w[l], n, 4 * Hp, 2 * Hp, e);
        stream = main_stream; ws_part_ = 0; ws_parts_ = 1;
        if (rc == LINMT_OK) CK(cudaEventRecord(enc_events_[l][pos % kRing], sl));
      }
    }
    // the decoder (main stream) starts after the last launch of every layer
    for (int l = 0; l < L; ++l)
      if (Smax > 0) CK(cudaStreamWaitEvent(main_stream, enc_events_[l][(Smax - 1) % kRing], 0));
    if (rc != LINMT_OK) return rc;
    if (att_fold_) {
      // W_c1 applied to every encoder state of the batch, once: the decoder's attention then sums these rows and
      // needs no output GEMM of its own (see AttFold in step_kernels.cuh).  Rows past a sentence's length hold
      // whatever an earlier batch left there; nothing reads their products.
      const size_t rows_all = (size_t)n * opt.max_src_len;
      tc::split_planes_kernel<<<1024, 256, 0, main_stream>>>(s.hs, ts.hs_planes, nt_, rows_all * Hp);
      LAUNCHED();
      tc::TcEpiF32 e{nullptr, s.hs_wc1, Hp, 0};
      if ((rc = tc_gemm(ts.hs_planes, 0, B * (int)opt.max_src_len, m.p_att_out_w, (int)rows_all, Hp, Hp, e))) return rc;
    }
  }
  return LINMT_OK;
}

// One decoder forward, tensor-core path (see Engine::run_decoder_step).
int Engine::run_decoder_step_tc(int mi, int t, int rows) {
  DevModel& m = models_[mi];
  DevState& s = states_[mi];
  TcState& ts = tc_states_[mi];
  const bool feed = desc.feed_input && t > 0;
  pdl_gemm_ = true;
  // where h_cur of layer l lives after its GEMM: the input slot of the consumer panel
  auto hcur_planes = [&](int l) -> const tc::Planes& { return (l + 1 < L) ? ts.panel[l + 1] : ts.panel_top; };
  auto hcur_col0 = [&](int l) { return (l + 1 < L) ? 0 : Hp; };
  auto hprev_planes = [&](int l) -> const tc::Planes& { return l == 0 ? ts.panel1 : ts.panel[l]; };
  // 1. gather states through the parents into the h_prev slots, look up embeddings
  {
    GatherJobs jobs{};
    int nj = 0;
    auto add = [&](const void* src, long long sstride, void* dst, long long dstride, int bytes, int kind) {
      jobs.j[nj++] = GatherJob{static_cast<const unsigned char*>(src), sstride, static_cast<unsigned char*>(dst), dstride, bytes, kind};
    };
    const int fb = enc_final_buf_;
    for (int l = 0; l < L; ++l) {
      for (int p = 0; p < nt_; ++p) {
        const __nv_bfloat16* src;
        long long sst;
        if (t == 0) { src = ts.encp[fb][l].p[p] + Hp; sst = (long long)ts.encp[fb][l].ld * 2; }
        else { src = hcur_planes(l).p[p] + hcur_col0(l); sst = (long long)hcur_planes(l).ld * 2; }
        add(src, sst, hprev_planes(l).p[p] + Hp, (long long)hprev_planes(l).ld * 2, Hp * 2, 0);
      }
      // the cell state is copied only at the first step (from the encoder); afterwards the LSTM epilogue
      // reads it through the parent index and the two buffers swap roles every step
      if (t == 0) add(s.enc_c[fb][l], (long long)Hp * 4, s.c_prev[l], (long long)Hp * 4, Hp * 4, 0);
    }
    if (feed)
      for (int p = 0; p < nt_; ++p)
        add(ts.panel_ht.p[p], (long long)ts.panel_ht.ld * 2, ts.panel1.p[p] + 2 * Hp, (long long)ts.panel1.ld * 2, Hp * 2, 0);
    if (!m.dec_xw)   // with the input-term table the embedding never enters the GEMM
      for (int p = 0; p < nt_; ++p)
        add(m.p_emb_tgt.p[p], (long long)m.p_emb_tgt.ld * 2, ts.panel1.p[p], (long long)ts.panel1.ld * 2, Hp * 2, 1);
    jobs.n = nj;
    dim3 grid(rows, (nj + kGatherJobsPerBlock - 1) / kGatherJobsPerBlock);
    if (int rc = kt(KC_GATHER)) return rc;
    CK(tc::launch_k(pdl_, row_gather_kernel, grid, dim3(128), 0, stream, jobs, (const int32_t*)d_parent_, (const int32_t*)d_tok_, V, k, t == 0 ? 1 : 0));
    LAUNCHED();
  }
  // 2. LSTM stack
  for (int l = 0; l < L; ++l) {
    if (int rc = kt(KC_LSTM)) return rc;
    tc::TcEpiLstm e{};
    e.bias = m.dec_b[l]; e.ldc = Hp;
    if (t == 0) { e.c_prev = s.c_prev[l]; e.c_out = s.c_cur[l]; }
    else {
      e.c_prev = (t & 1) ? s.c_cur[l] : s.c_prev[l];
      e.c_out = (t & 1) ? s.c_prev[l] : s.c_cur[l];
      e.c_parent = d_parent_; e.c_k = k;
    }
    e.h_out1 = hcur_planes(l); e.h1_col0 = hcur_col0(l);
    e.h_out2 = no_planes(); e.h2_col0 = 0;
    e.h_prev = no_planes(); e.hp_col0 = 0;
    e.h_f32 = (l == L - 1 && opt.attention_mode == LINMT_ATT_GLOBAL_DOT) ? s.h_cur[l] : nullptr;
    e.hf_row_stride = Hp;
    e.row_len = nullptr; e.pos = 0; e.nt = nt_;
    int K = (l == 0 && feed) ? 3 * Hp : 2 * Hp;
    int rc;
    if (l == 0 && m.dec_xw) {
      // K columns (h_prev | htilde_prev) only: the x columns of panel and weights are skipped, their term comes from the table
      tc::Planes wrest = m.p_dec_w[0];
      for (int p = 0; p < 3; ++p) if (wrest.p[p]) wrest.p[p] += Hp;
      e.xw = m.dec_xw; e.x_tok = d_tok_; e.x_ld = 4 * Hp; e.x_vocab = V; e.x_unk = kUnk;
      K -= Hp;
      rc = tc_gemm(hprev_planes(0), Hp, R, wrest, rows, 4 * Hp, K, e);
    } else {
      rc = tc_gemm(hprev_planes(l), 0, R, m.p_dec_w[l], rows, 4 * Hp, K, e);
    }
    if (rc) return rc;
    if (kernel_timing) rec_flops_ += 2.0 * rows * 4.0 * H * (double)((K / Hp) * H);
  }
  // 3. attention projections: tanh(W_p h) | W_a^T h
  if (int rc = kt(KC_PROJ)) return rc;
  const float* u_alt = (opt.attention_mode == LINMT_ATT_GLOBAL_DOT) ? s.h_cur[L - 1] : nullptr;
  if (att_merge_) {
    // ... | W_c2 h: the half of the attention output's pre-activation that needs h_top only (global dot
    // attention uses no projection, so only those rows run)
    const int n0 = (opt.attention_mode == LINMT_ATT_GLOBAL_DOT) ? 2 * Hp : 0;
    tc::Planes w = m.p_att_proj_w;
    for (int p = 0; p < 3; ++p) if (w.p[p]) w.p[p] += (size_t)n0 * w.ld;
    tc::TcEpiF32 e{nullptr, s.proj + n0, 3 * Hp, n0 ? 0 : Hp};
    int rc = tc_gemm(ts.panel_top, Hp, R, w, rows, 3 * Hp - n0, Hp, e);
    if (rc) return rc;
  } else if (opt.attention_mode != LINMT_ATT_GLOBAL_DOT) {
    tc::TcEpiF32 e{nullptr, s.proj, 2 * Hp, Hp};
    int rc = tc_gemm(ts.panel_top, Hp, R, m.p_att_proj_w, rows, 2 * Hp, Hp, e);
    if (rc) return rc;
  }
  // 4. scores, softmax x Gaussian, context (written into the attention-output panel)
  {
    float* ra = d_rec_align_ ? d_rec_align_ + (size_t)t * R * rec_win : nullptr;
    int32_t* rl = d_rec_lo_ ? d_rec_lo_ + (size_t)t * R : nullptr;
    int32_t* rv = d_rec_vit_ ? d_rec_vit_ + (size_t)t * R : nullptr;
    if (int rc = kt(KC_ATTENTION)) return rc;
    if (int rc = launch_attention(mi, t, rows, u_alt, nullptr, att_fold_ ? ts.panel_ht : ts.panel_top, nt_, ra, rl, rv, att_fold_)) return rc;
  }
  // 5. htilde = tanh(W_c1 ctx + W_c2 h + b) (with the fold the attention kernel has written it already)
  if (!att_fold_) {
    tc::TcEpiBiasTanh e{m.att_bout, ts.panel_ht, 0, nt_};
    if (int rc0 = kt(KC_ATTOUT)) return rc0;
    int rc;
    if (att_merge_) {
      // W_c1 ctx over the first Hp of the K columns; W_c2 h comes in as a precomputed row
      e.add = s.proj + 2 * Hp; e.ld_add = 3 * Hp;
      rc = tc_gemm(ts.panel_top, 0, R, m.p_att_out_w, rows, Hp, Hp, e);
    } else {
      rc = tc_gemm(ts.panel_top, 0, R, m.p_att_out_w, rows, Hp, 2 * Hp, e);
    }
    if (rc) return rc;
  }
  // 6. logits
  {
    tc::TcEpiF32 e{m.voc_b, s.logits, Vp, 0};
    if (logits16_) e.out16 = s.logits16;   // the softmax of this step is their only reader
    pmax_slots_ = 0;
    if (n_models == 1 && pmax_on_) { e.pmax = d_pmax_; e.pmax_ld = pmax_ld_; e.n_valid = V; }
    if (int rc = kt(KC_VOCAB)) return rc;
    // Logits feed only the softmax of their own step: the tensor core's truncation bias over one
    // K = Hp chain (~32 ulp of the accumulator, 2e-7 relative on a log-probability) does not
    // accumulate over steps as it does through the recurrent products, so this GEMM runs its
    // leading product as one chain (no intermediate drains: 5 % faster).
    int rc = tc_gemm(ts.panel_ht, 0, R, m.p_voc_w, rows, Vp, Hp, e, nt_vocab_, Hp / 32);
    if (rc) return rc;
  }
  return LINMT_OK;
}

}  // namespace linmt

// engine.h -- the decoding engine behind the C ABI (host side, C++).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/linmt_decoder.h"
#include "step_kernels.cuh"
#include "gemm_tc.cuh"
#include <array>
#include <functional>
#include <map>
#include <memory>
#include <tuple>

namespace linmt {

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Packed weights of one ensemble member in device memory.  Every dense operand is stored
// K-major ("[out][in]", in padded to Hp) so both GEMM operands are K-contiguous.
struct DevModel {
  float* emb_src = nullptr;              // [Vs][Hp]
  float* emb_tgt = nullptr;              // [V][Hp]
  std::vector<float*> enc_w, enc_b;      // [4Hp][2Hp], [4Hp]   gate-interleaved rows 4j+g
  std::vector<float*> dec_w, dec_b;      // layer 0: [4Hp][3Hp] (x | h' | htilde'), others [4Hp][2Hp]
  std::vector<int> dec_ldw;
  float* att_proj_w = nullptr;           // [2Hp][Hp]: rows < Hp = W_p, rows >= Hp = W_a^T (tensor path: [3Hp][Hp], rows >= 2Hp = W_c2)
  float* att_out_w = nullptr;            // [Hp][2Hp]: (ctx | h_top)
  float* att_bout = nullptr;             // [Hp]
  float* vp = nullptr;                   // [Hp]
  float* voc_w = nullptr;                // [Vp][Hp]
  float* voc_b = nullptr;                // [Vp]
  float* dec_xw = nullptr;               // [V][4Hp] W_x . embedding(v) of the first decoder layer (tensor path, optional)
  float voc_wnorm_max = 0.f;             // largest 2-norm of a vocabulary weight row
  float voc_babs_max = 0.f;              // largest magnitude of a vocabulary bias
  // the same operands as bf16 planes for the tensor-core path (fp32 copies are then not kept)
  tc::Planes p_emb_src{}, p_emb_tgt{}, p_att_proj_w{}, p_att_out_w{}, p_voc_w{};
  std::vector<tc::Planes> p_enc_w, p_dec_w;
};

// Activation panels of the tensor-core path: every GEMM reads ONE K-contiguous panel, so the
// producers write straight into the column range of the panel that consumes them.
struct TcState {
  tc::Planes panel1{};               // [R][3Hp]  x | h_prev(layer 0) | htilde_prev
  std::vector<tc::Planes> panel;     // l = 1..L-1: [R][2Hp]  h_cur(l-1) | h_prev(l)
  tc::Planes panel_top{};            // [R][2Hp]  ctx | h_cur(L-1)
  tc::Planes panel_ht{};             // [R][Hp]   htilde
  tc::Planes hs_planes{};            // [B * max_src][Hp]  the encoder's top states as operand planes (attention fold)
  std::vector<tc::Planes> encp[2];   // [L] x [B][2Hp]  below | h_prev, double buffered over positions
};

struct DevState {
  float* x = nullptr;                        // [R][Hp]
  std::vector<float*> h_cur, c_cur, h_prev, c_prev;  // [L] x [R][Hp]
  float *htilde = nullptr, *htilde_prev = nullptr;   // [R][Hp]
  float *proj = nullptr, *ctx = nullptr;             // [R][2Hp or 3Hp], [R][Hp]
  float* logits = nullptr;                           // [R][Vp]
  __half* logits16 = nullptr;                        // [R][Vp]  the same in fp16 (one-product logits whose candidates are recomputed)
  float* hs = nullptr;                               // [B][max_src][Hp]
  float* hs_wc1 = nullptr;                           // [B][max_src][Hp]  W_c1 . hs (tensor path with the attention fold)
  float* enc_x = nullptr;                            // [B][Hp]
  std::vector<float*> enc_h[2], enc_c[2];            // [L] x [B][Hp], double buffered
};

// Kernel classes of a decoder step, in launch order (linmt_kernel_times reports one entry per class).
enum KernelClass { KC_GATHER = 0, KC_LSTM, KC_PROJ, KC_ATTENTION, KC_ATTOUT, KC_VOCAB, KC_COMBINE, KC_SOFTMAX, KC_SELECT, KC_COUNT, KC_END = KC_COUNT };

class Engine {
 public:
  float class_ms[KC_COUNT] = {};      // device time per kernel class in the last timed decode
  int class_launches[KC_COUNT] = {};
  Engine() = default;
  ~Engine();
  int init(const linmt_model_desc& d, const float* const* blobs, int n_models, size_t blob_floats, const linmt_options& o);
  int decode_core(const int32_t* d_ids, const int32_t* off_host, int n, const int32_t* steps_host, int max_len,
                  int32_t* d_out_tok, int32_t* d_out_len, float* d_out_score, int32_t* d_out_vit, float* d_out_align,
                  const linmt_trace* trace_dev, int trace_Tm);
  int finish_timing();
  int decode_host(const int32_t* src_ids, const int32_t* src_off, int n, const int32_t* steps, int max_len,
                  int32_t* out_tok, int32_t* out_len, float* out_score, int32_t* out_vit, float* out_align,
                  const linmt_trace* trace);

  std::string err;
  linmt_model_desc desc{};
  linmt_options opt{};
  int k = 0, kk = 0, H = 0, Hp = 0, V = 0, Vp = 0, L = 0, B = 0, R = 0, win = 0, rec_win = 0, Tcap = 0, fin_cap = 0;
  int n_models = 0;
  cudaStream_t stream = nullptr;
  linmt_stats stats{};
  bool kernel_timing = false;

  // sentence front-end (filled by the config-file constructor)
  std::vector<std::string> tgt_words;
  std::vector<std::pair<std::string, int>> src_words_sorted;
  int longest_sentence = 0;
  int print_align_scores = 0;
  int src_unk_id = 0;   // id unknown source words read: the source map's "UNK" entry, 0 when it has none
  std::string result_buf;

 private:
  int fail(int code, const std::string& msg) { err = msg; return code; }
  // role of member mi in the alignment record of a step: 0 = single model, 1 / 2 / 3 = first / middle / last member
  int ens_member_code(int mi) const { return n_models == 1 ? 0 : (mi == 0 ? 1 : (mi == n_models - 1 ? 3 : 2)); }
  int pack_model(const float* blob, DevModel& m);
  int alloc_state(DevState& s);
  int run_encoder(int n, int Smax);
  int run_decoder_step(int mi, int t, int rows);
  int run_encoder_tc(int n, int Smax);
  int run_decoder_step_tc(int mi, int t, int rows);
  int step_tail(int t, int rows);
  bool pairs_available();   // clusters of two GEMM CTAs can be scheduled on the current device (engine_tc.cu)
  int launch_attention(int mi, int t, int rows, const float* u_alt, float* ctx, const tc::Planes& ctx_planes, int nt,
                       float* rec_align, int32_t* rec_lo, int32_t* rec_vit, bool fold = false);
  int alloc_state_tc(TcState& s);
  int build_xw_tables();   // dec_xw of every model (tensor path, xw_table_)
  int alloc_planes(tc::Planes& p, size_t rows, int ld);
  int to_planes(const std::vector<float>& host, size_t rows, int ld, tc::Planes& dst);
  const CUtensorMap* a_maps(const tc::Planes& p, int col0, int rows_cap, int K, int bk);
  const CUtensorMap* b_maps(const tc::Planes& p, int rows, int K, int bn, int bk);
  template <class Epi>
  int tc_gemm(const tc::Planes& A, int a_col0, int a_rows_cap, const tc::Planes& W, int M, int N, int K, const Epi& e, int nt = 0, int drain = 0);

  bool use_tc_ = false;
  // encoder wavefront: one stream per layer, a small ring of events per layer
  std::vector<cudaStream_t> enc_streams_;
  std::vector<std::vector<cudaEvent_t>> enc_events_;
  cudaEvent_t enc_start_ev_ = nullptr;
  int nt_ = 3;
  bool pdl_ = false;  // decoder-step kernels launched with programmatic stream serialization (tensor path)
  bool xw_table_ = false;  // first decoder layer: embedding term from a per-vocabulary table instead of the GEMM
  bool refine_ = false;    // one-product vocabulary GEMM + accurate recomputation of the candidates in the softmax kernel
  bool logits16_ = false;  // one-product logits stored as fp16 (only with the accurate recomputation of the candidates; LINMT_LOGITS16=0: test knob)
  bool att_fold_ = false;  // tensor path: W_c1 applied to the encoder states once per batch, attention writes htilde (LINMT_ATT_FOLD=0: test knob)
  bool att_merge_ = false; // tensor path: W_c2 . h_top computed with the attention projections (LINMT_ATT_MERGE=0: test knob)
  bool pmax_on_ = true;    // vocabulary GEMM hands block maxima to the softmax (LINMT_PMAX=0: test knob)
  bool pair_ = true;       // CTA pairs for the GEMM shapes that are down to two stages (LINMT_TC_PAIR=0: test knob)
  bool persist_ = true;    // persistent kernel for the many-wave vocabulary GEMM (LINMT_TC_PERSIST=0: test knob)
  bool pdl_gemm_ = false;  // true while the decoder step issues its GEMMs (the encoder's wavefront does not take part)
  int fmt_ = 0;       // plane format of every operand: 0 = bf16 planes, 1 = f16 pair
  int nt_vocab_ = 0;  // planes used by the vocabulary GEMM (0 = nt_)
  int n_sm_ = 148;
  int* d_tc_err_ = nullptr;
  float* d_splitk_ws_ = nullptr;      // split-K partial tiles
  int* d_splitk_counters_ = nullptr;  // one arrival counter per output tile
  static constexpr size_t kSplitKWsFloats = (size_t)16 << 20;  // 64 MiB
  int ws_part_ = 0, ws_parts_ = 1;    // slice of the workspace a launch may use (concurrent encoder layers get one each)
  static constexpr int kSplitKMaxTiles = 4096;
  std::vector<TcState> tc_states_;
  std::map<std::tuple<const void*, int, int, int, int>, std::array<CUtensorMap, 3>> tmap_cache_;

  const int32_t* cur_ids_ = nullptr;
  TraceDev trace_dev_{};
  size_t trace_pt_member_stride_ = 0;   // floats between two members' p_t records in the device trace buffer
  int enc_final_buf_ = 0;
  size_t out_cap_maxlen_ = 0;
  std::vector<DevModel> models_;
  std::vector<DevState> states_;
  std::vector<void*> allocs_;
  template <class T> int dalloc(T** p, size_t count);
  template <class T> int regrow(T** p, size_t count);

  // batch metadata (device) and pinned staging
  int32_t *d_off_ = nullptr, *d_len_ = nullptr, *d_steps_ = nullptr, *d_orig_ = nullptr;
  int32_t* h_meta_ = nullptr;  // pinned [4][B+1]
  // beam state
  int32_t *d_tok_ = nullptr, *d_parent_ = nullptr, *d_hist_tok_ = nullptr, *d_hist_parent_ = nullptr;
  float* d_score_ = nullptr;
  int32_t *d_fin_t_ = nullptr, *d_fin_b_ = nullptr, *d_fin_n_ = nullptr;
  float *d_fin_score_ = nullptr, *d_fin_final_ = nullptr;
  float* d_combined_ = nullptr;  // [R][Vp] ensemble-combined log-values (n_models > 1)
  int32_t* d_cand_idx_ = nullptr;
  float *d_cand_logp_ = nullptr, *d_eos_logp_ = nullptr, *d_row_stats_ = nullptr;
  float* d_pmax_ = nullptr;   // [R][pmax_ld_] block maxima of the logits, by-product of the vocabulary GEMM
  int pmax_ld_ = 0;
  int pmax_slots_ = 0;        // slots the last vocabulary GEMM filled (0 = none: the softmax finds its own maxima)
  // alignment records (print_info)
  float* d_rec_align_ = nullptr;
  int32_t *d_rec_lo_ = nullptr, *d_rec_vit_ = nullptr;
  // host staging for decode_host
  int32_t* d_ids_ = nullptr;
  size_t d_ids_cap_ = 0;
  int32_t *d_out_tok_ = nullptr, *d_out_len_ = nullptr, *d_out_vit_ = nullptr;
  float *d_out_score_ = nullptr, *d_out_align_ = nullptr;
  size_t out_cap_len_ = 0;
  // trace buffers (device), sized on demand
  std::vector<void*> trace_allocs_;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
  // kernel timing (off by default): an event before every kernel of the decoder steps, tagged with the kernel's
  // class; the time to the next event is booked to that class.  The events end the overlap of consecutive
  // kernels, so a timed decode is a measurement pass, not the number to report as throughput.
  std::vector<cudaEvent_t> kt_ev_;
  std::vector<int> kt_cls_;
  size_t kt_used_ = 0;
  double rec_flops_ = 0.0;
  int kt(int cls);
};

// host-side weight packing
void pack_gate_weights(const float* const* mats, int nseg, int H, int Hp, float* out /*[4Hp][nseg*Hp]*/);

}  // namespace linmt

// The opaque handle of the C ABI: the engine on the first device and, for a handle created on several
// devices, one replica of the same models per further device.  Sentences are independent, so a job is
// dealt to the devices in device batches, one host thread per device, with no traffic between them.
struct linmt_engine {
  linmt::Engine eng;
  std::vector<std::unique_ptr<linmt::Engine>> replicas;
  int n_engines() const { return 1 + (int)replicas.size(); }
  linmt::Engine& engine(int i) { return i == 0 ? eng : *replicas[i - 1]; }
};

namespace linmt {
// Runs job(engine, item) for item = order[0], order[1], ... on the engines of a handle, one host thread per
// engine, each taking the next item when it is free.  Returns the first error; engine 0's `err` names it.
int run_on_engines(linmt_engine* h, const std::vector<int>& order, const std::function<int(Engine&, int)>& job);
}  // namespace linmt

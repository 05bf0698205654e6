/* linmt_decoder.h -- C ABI of the B200 beam-search decoding engine.
 *
 * The library replaces LiNMT's sentence-decoding path.  Every entry point takes plain
 * pointers and sizes; nothing here depends on a tensor library.  Unless a function says
 * otherwise, pointers are HOST pointers and the call copies to and from the GPU itself.
 *
 * Citations are into the reference project's tree (src/...).
 */
#ifndef LINMT_DECODER_H_
#define LINMT_DECODER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------
 * 1. The reference's own exported symbols (src/decoder_sentence.h:94-97, definitions
 *    src/decoder_sentence.cu:847-873).  Same names, same signatures, same ownership rule:
 *    the returned string belongs to the library and stays valid until the next call.
 *    `msg` is the path of a decoding-sentence config file (param="--key" value="..." lines,
 *    src/decoder_sentence.cu:267-318).  Like the reference, init prints and exits the
 *    process on a fatal configuration error; do_job never exits and returns "" on error.
 * ------------------------------------------------------------------------------------ */
void python_decoder_init(char* msg);
char* python_decoder_do_job(char* sentence);

/* UNK post-processing, the pair the reference's wrapper and server call right after
 * python_decoder_do_job (src/postprocess_unks.h:89-92, definitions src/postprocess_unks.cc:716-752;
 * callers server/LiNMT-python-wrapper.py:24-33, server/LiNMT-server.py:52-57).  Host string code.
 * `msg` = config file with --phrase-table ("src ||| tgt ||| x" lines), --stopword and --end-punct
 * (tab-separated "tag<TAB>word" lines) and optional --rm-oov-mode; init exits on a missing file as
 * the reference does.  do_job takes the source line (optionally "words |||| {generalizations}") and
 * the decoder's "words |||| score |||| alignments |||| unk alignments |||| a/a/a ..." line and
 * returns the final words; the string belongs to the library until the next call. */
void python_unk_init(char* msg);
char* python_unk_do_job(char* src_sentence, char* translation);
/* The same on a handle, returning the whole line with its "||||" fields
 * (PostProcessUnks::Init / Process, src/postprocess_unks.cc:14-30). */
typedef struct linmt_unk linmt_unk;
int linmt_unk_create(const char* config_path, linmt_unk** out);
int linmt_unk_process(const linmt_unk* h, const char* source, const char* translation, char* out, int32_t out_cap);
void linmt_unk_destroy(linmt_unk* h);

/* ------------------------------------------------------------------------------------
 * 2. Handle-based API at the reference's numeric boundary
 *    (EnsembleFactory<T>::InitDecoderSentence, src/decoder.h:1526-1575, and
 *    EnsembleFactory<T>::DecodeSentence, src/decoder.h:1780-1840), extended from one
 *    sentence per call to a batch of independent sentences.
 * ------------------------------------------------------------------------------------ */
typedef struct linmt_engine linmt_engine;

enum { LINMT_OK = 0, LINMT_EINVAL = 1, LINMT_ECUDA = 2, LINMT_EIO = 3, LINMT_ENOMEM = 4, LINMT_ELIMIT = 5 };

enum { LINMT_ATT_LOCAL_P_GENERAL = 0, LINMT_ATT_GLOBAL_GENERAL = 1, LINMT_ATT_GLOBAL_DOT = 2 };
enum { LINMT_ENS_PROB_MEAN = 0, LINMT_ENS_LOGPROB_MEAN = 1 };
enum { LINMT_PREC_FP32 = 0, LINMT_PREC_BF16 = 1 };
/* GEMM kernel family.  SIMT = fp32 CUDA-core kernels (fp32 FMA arithmetic).  TENSOR = tcgen05
 * tensor-core kernels; with fp32 precision every operand is held as an fp16 pair x ~ a0 + 2^-11 a1
 * (22 mantissa bits, three partial products per product, fp32-class accuracy; operands must be
 * below 65504 in magnitude).  TENSOR3 = three bf16 planes (six partial products, same accuracy,
 * no range limit), TENSOR2 = two bf16 planes (error ~2^-17 per product).  TENSOR_V16 = TENSOR for the
 * recurrent and attention products, but the vocabulary projection in plain fp16 (one product instead of three:
 * logits carry ~2^-12 relative noise, 1e-5 on a log-probability; near-ties in the beam may resolve differently;
 * ~15 % faster).  TENSOR_V16X = TENSOR_V16 plus a refinement in the softmax kernel: every logit that can still
 * be among the k+1 best of its row given the error bound of the fp16 product (and EOS) is recomputed from both
 * planes, so candidates and their log-probabilities are fp32-class again; only the normaliser sums fp16 logits.
 * AUTO = TENSOR_V16X for a single model (measured: the same parity as TENSOR, 13 % faster), TENSOR for ensembles. */
enum { LINMT_GEMM_AUTO = 0, LINMT_GEMM_SIMT = 1, LINMT_GEMM_TENSOR = 2, LINMT_GEMM_TENSOR2 = 3, LINMT_GEMM_TENSOR3 = 4, LINMT_GEMM_TENSOR_V16 = 5, LINMT_GEMM_TENSOR_V16X = 6 };

/* Model dimensions: first five of the nine integers on line 1 of a model file
 * (src/decoder.h:1202-1210). */
typedef struct linmt_model_desc {
  int32_t layers;      /* L  */
  int32_t hidden;      /* H = LSTM size = embedding size */
  int32_t vocab_tgt;   /* V  */
  int32_t vocab_src;   /* Vs */
  int32_t feed_input;  /* 1 = previous attentional state feeds layer 1 */
} linmt_model_desc;

/* Decoding options; defaults are the reference's (src/global_configuration.h:228-235). */
typedef struct linmt_options {
  int32_t beam;            /* 12; clamped to floor(sqrt(V)) (src/decoder.h:1549-1551)      */
  int32_t nbest;           /* 1                                                            */
  int32_t attention_mode;  /* LINMT_ATT_*                                                  */
  int32_t attention_d;     /* local attention half width D, 10 (src/global_configuration.h:45) */
  int32_t print_info;      /* 1 = track viterbi and dense alignments (--print-decoding-info) */
  int32_t precision;       /* LINMT_PREC_*                                                 */
  int32_t ensemble_mode;   /* LINMT_ENS_*                                                  */
  int32_t gemm_path;       /* LINMT_GEMM_*: which hand-written GEMM kernel family to use   */
  int32_t max_batch;       /* most sentences per device batch (64)                         */
  int32_t max_src_len;     /* longest source sentence accepted (100)                       */
  int32_t max_steps;       /* most beam expansions per sentence (200)                      */
  int32_t device;          /* CUDA device ordinal                                          */
  float penalty;           /* 0    */
  float diversity;         /* 0    */
  float lp_alpha;          /* 0.65 */
  float cp_beta;           /* 0.20 */
  float min_ratio;         /* 0.5: keep hypotheses with len/S > min_ratio (src/decoder.h:762-765) */
  float max_ratio;         /* 1.5: only used by the sentence API to derive the step count
                              min((int)(max_ratio*S), longest-2) (src/decoder.h:1806)      */
} linmt_options;

/* Fills `opt` with the defaults above. */
void linmt_default_options(linmt_options* opt);

/* Number of floats in one weight blob of the given shape. */
size_t linmt_blob_floats(const linmt_model_desc* desc);

/* Creates an engine from in-memory weights.  `blobs[m]` is ensemble member m: the matrices
 * of a model file in LoadWeights order (src/deep_rnn.h:1878-1969), each rows x cols
 * column-major as the reference holds them on the device (src/deep_rnn_kernel.h:1543-1560).
 * Replaces DecoderModelWrapper::InitDecoderSentence + LoadWeights
 * (src/decoder.h:1040-1107, src/deep_rnn.h:1878-1969). */
int linmt_create_from_weights(const linmt_model_desc* desc, const float* const* blobs, int32_t n_models,
                              size_t blob_floats, const linmt_options* opt, linmt_engine** out);

/* The same engine on several GPUs of one box: devices[0..n_devices) each get a replica of the model(s)
 * (opt->device is then ignored), and linmt_decode_batch / linmt_decode_file deal device batches of
 * sentences to them, one host thread per device inside the library; nothing crosses between the GPUs
 * and results come back in the caller's order.  Sentences are independent in the reference too
 * (EnsembleFactory::DecodeSentence keeps no state between calls, src/decoder.h:1780-1840); its own use
 * of several GPUs is one DecoderModelWrapper per GPU index (src/decoder.h:1676-1684, config key
 * --multi-gpu, src/decoder_sentence.cu:183-198), which this replaces.  n_devices = 0 means opt->device. */
int linmt_create_from_weights_on(const linmt_model_desc* desc, const float* const* blobs, int32_t n_models,
                                 size_t blob_floats, const linmt_options* opt, const int32_t* devices,
                                 int32_t n_devices, linmt_engine** out);
/* Number of devices a handle decodes on. */
int32_t linmt_device_count(const linmt_engine* e);

/* Creates an engine from a decoding-sentence config file, reading the model file(s) named
 * by --nmt-model in the reference's text format.  Replaces DecoderSentence::Init
 * (src/decoder_sentence.cu:14-37). */
int linmt_create(const char* config_path, linmt_engine** out);

void linmt_destroy(linmt_engine* e);

/* Text of the last error on this handle (or of the last failed create when e == NULL).
 * A decode that returns LINMT_ECUDA with "gave up waiting on a barrier" leaves the handle unusable:
 * every wait inside the GEMM kernels is bounded (about a second) and a wait that ran out means the
 * device state of this handle can no longer be trusted, so every later decode on it fails the same
 * way.  Destroy the handle and create a new one. */
const char* linmt_last_error(const linmt_engine* e);
/* Text of the last error of linmt_create / linmt_read_model_file (config and model-file problems). */
const char* linmt_front_error(void);

/* Effective beam after clamping. */
int32_t linmt_beam(const linmt_engine* e);

/* Optional per-step records of a decode, and optional forcing of the beam.
 * All pointers are host pointers and may be NULL.  Tm = max steps[i], k = effective beam.
 *   cand_tok, cand_logp   [n][Tm][k][k+1]  per-beam top-(k+1) tokens and log-probabilities
 *   surv_tok, surv_parent, surv_score [n][Tm][k]  survivors chosen at each step
 *   final_logp            [n][k]  log p(EOS) at the extra forward
 *   force_tok, force_parent, force_score [n][Tm][k]  if set, the beam continues from these
 *                         survivors instead of its own (the records still show its own). */
typedef struct linmt_trace {
  int32_t* cand_tok;
  float* cand_logp;
  int32_t* surv_tok;
  int32_t* surv_parent;
  float* surv_score;
  float* final_logp;
  const int32_t* force_tok;
  const int32_t* force_parent;
  const float* force_score;
  float* gold_logp;   /* [n][Tm][k]: log p of the forced token of each slot (needs force_*), may be NULL */
  float* pt;          /* [n_models][n][Tm+1][k]: attention centre p_t of every forward of every ensemble member (local
                         attention), may be NULL.  Entries of forwards that did not run hold the bit pattern 0xffffffff. */
} linmt_trace;

/* Decodes n independent sentences.  Replaces EnsembleFactory<T>::DecodeSentence
 * (src/decoder.h:1780-1840) and Decoder<T>::ObtainOneBestHypothesis (src/decoder.h:703-859)
 * up to, not including, the formatting of the output string.
 *   src_ids, src_off  sentence i = src_ids[src_off[i] .. src_off[i+1]) in natural order
 *                     (the engine reverses it as src/decoder_sentence.cu:68 does)
 *   steps             T_i beam expansions for sentence i; one more forward appends EOS
 *   max_len           row length of the outputs, >= max T_i + 2
 *   out_tok   [n][nbest][max_len]  hypothesis including START(0) and EOS(1)
 *   out_len   [n][nbest]           its length, 0 = fewer than nbest hypotheses passed the filter
 *   out_score [n][nbest]
 *   out_vit   [n][nbest][max_len]  viterbi alignment per position, may be NULL
 *   out_align [n][nbest][max_len][max_src_len]  dense alignments, may be NULL (print_info only)
 * Sentences are processed in device batches of at most max_batch. */
int linmt_decode_batch(linmt_engine* e, const int32_t* src_ids, const int32_t* src_off, int32_t n,
                       const int32_t* steps, int32_t max_len, int32_t* out_tok, int32_t* out_len,
                       float* out_score, int32_t* out_vit, float* out_align, const linmt_trace* trace);

/* Same decode with every buffer already in device memory (no host copies inside): the
 * sentences must fit one device batch (n <= max_batch), `steps` is still a host array
 * because it sizes the launches.  Outputs stay on the device. */
int linmt_decode_batch_device(linmt_engine* e, const int32_t* d_src_ids, const int32_t* src_off_host,
                              int32_t n, const int32_t* steps_host, int32_t max_len, int32_t* d_out_tok,
                              int32_t* d_out_len, float* d_out_score);

/* Counters since creation: kernels launched by this library, decoder forwards (row-steps)
 * and device time of the last decode call in milliseconds (CUDA events). */
typedef struct linmt_stats {
  int64_t kernel_launches;
  int64_t decoder_row_steps;
  int64_t sentence_steps;
  float last_decode_ms;
  float last_gemm_ms;     /* time inside the dominant (vocabulary) GEMM launches, if timing is on */
  int32_t last_gemm_launches;
  int32_t last_rec_gemm_launches; /* decoder LSTM-stack GEMM launches of the last call, if timing is on */
  float last_rec_gemm_ms;         /* time inside them */
  float last_host_issue_ms;       /* host time spent issuing the decoder steps of the last device batch */
  double last_rec_gemm_flops;     /* their algorithmic flops: 2 * rows * 4H * K per launch */
  int64_t pair_launches;          /* GEMM launches, of kernel_launches, that ran on CTA pairs (tcgen05 cta_group::2) */
} linmt_stats;
int linmt_get_stats(const linmt_engine* e, linmt_stats* out);
/* 1 = put a CUDA event before every kernel of the decoder steps (for roofline measurements).  The events
 * end the overlap of consecutive kernels, so a timed decode is a measurement pass: slower than an untimed one. */
int linmt_set_kernel_timing(linmt_engine* e, int32_t on);
/* Device time and launch count per kernel class of the last timed device batch (first device of the handle).
 * Classes in launch order: 0 state gather, 1 LSTM gate GEMMs, 2 attention projections GEMM, 3 attention,
 * 4 attention output GEMM (no launches on the tensor-core path: that layer is applied to the encoder states once per
 * batch and finished inside the attention kernel), 5 vocabulary GEMM, 6 ensemble combine, 7 softmax / top-k, 8 beam selection.
 * `ms` and `launches` hold n >= 9 entries. */
int linmt_kernel_times(const linmt_engine* e, float* ms, int32_t* launches, int32_t n);

/* Sentence API on a handle: DecoderSentence::Process (src/decoder_sentence.cu:40-49).
 * Needs an engine created from a config file (vocabularies).  Returns a library-owned
 * string valid until the next call on the same handle. */
const char* linmt_translate(linmt_engine* e, const char* sentence);

/* Force-decoding / scoring: log-probability of given target sentences under the model
 * (the reference's --force-decoding path, src/deep_rnn.h:1490-1568, src/dispatcher.cu:699-752).
 *   tgt_ids, tgt_off  target token ids per sentence WITHOUT START / EOS
 *   out_logprob [n]   sum over the m_i tokens and the closing EOS of log p(token | source, prefix)
 *   out_token_logp    optional [n][max_tgt + 1]: the per-token terms (EOS last), zero padded
 * Every sentence needs 1 <= m_i <= max_steps. */
int linmt_score_batch(linmt_engine* e, const int32_t* src_ids, const int32_t* src_off, const int32_t* tgt_ids,
                      const int32_t* tgt_off, int32_t n, float* out_logprob, float* out_token_logp, int32_t max_tgt);

/* Reads a model file in the reference's text format (header, vocabularies, matrices; the format
 * written by DumpBestModel, src/deep_rnn.h:1972-2146, and read by LoadWeights, :1878-1969) without
 * creating an engine: fills `desc` and, if `blob` is given, the weights in the blob layout of
 * linmt_create_from_weights (`blob_cap` floats available).  use_cache = 1 reads / writes the raw
 * copy "<path>.linmtcache" that makes later loads of the same unchanged text file fast.  No GPU call. */
int linmt_read_model_file(const char* path, linmt_model_desc* desc, float* blob, uint64_t blob_cap, int32_t use_cache);

/* File-mode decoding: one source sentence per line of `in_path`; writes the n-best
 * translations of every sentence to `out_path` in input order.  Replaces
 * EnsembleFactory::DecodeFile (src/decoder.h:1702-1776), Decoder::OutputKBestHypotheses
 * (src/decoder.h:529-699) and InputFilePreprocess::UnintFile
 * (src/input_file_preprocess.cc:1485-1572).  Needs an engine created from a config file; sentences
 * are decoded in length-sorted batches of --batch-size. */
int linmt_decode_file(linmt_engine* e, const char* in_path, const char* out_path);

/* ------------------------------------------------------------------------------------
 * 3. Single-kernel entry points (host pointers) used by the parity tests.
 * ------------------------------------------------------------------------------------ */
/* Y[R][N] = X[R][K] . W[K][N] with W stored like a reference weight ([in][out]);
 * stands in for one cublasSgemm call of the reference (src/utility_cu.h:153-157).
 * gemm_path: LINMT_GEMM_SIMT or LINMT_GEMM_TENSOR; precision: LINMT_PREC_*. */
int linmt_k_gemm(const float* X, const float* W, float* Y, int32_t R, int32_t K, int32_t N, int32_t gemm_path,
                 int32_t precision, int32_t device);
/* Per-row log-softmax statistics and top-kk of logits[R][V]: replaces the softmax kernel
 * (src/deep_rnn_kernel.h:352-429) plus the per-beam top-(k+1) scan of
 * src/decoder.h:401-410.  idx/logp are [R][kk], eos_logp [R]. */
int linmt_k_softmax_topk(const float* logits, int32_t R, int32_t V, int32_t kk, int32_t* idx, float* logp,
                         float* eos_logp, int32_t device);

/* Y[R][N] = X[R][K] . Wt[N][K]^T on the tensor-core kernel (three bf16 planes, fp32-class
 * result) WITHOUT allocating: for hosts that cannot call cudaMalloc once they are running --
 * processes that gave the whole GPU to their own memory pool at start-up, or that share the
 * device and must not trigger the device-wide stall an allocation can cause.  It has no
 * counterpart in the reference.
 *   d_x, d_wt, d_y  DEVICE pointers, fp32, row-major; K a multiple of 32, N a multiple of 16.
 *   Limits: R <= 256, K <= 1024, N <= 1024 (LINMT_ELIMIT beyond): the kernel's working memory
 *   (the bf16 planes of both operands, 7.5 MiB) is a fixed array inside the library that every
 *   GPU loading the library holds until exit.
 * The first call on a device looks that array's address up (cudaGetSymbolAddress); make it
 * before any stream capture.  Work is issued on the default stream and the call returns when
 * the result is in d_y.  All calls share the one array and it keeps the last call's contents:
 * two calls that overlap on the GPU (from two threads, say) race -- serialise them. */
int linmt_gemm_f32_noalloc(const float* d_x, const float* d_wt, float* d_y, int32_t R, int32_t K, int32_t N,
                           int32_t device);

#ifdef __cplusplus
}
#endif
#endif /* LINMT_DECODER_H_ */

// frontend.cu -- the sentence-level front of the library: decoding config files, model
// files (vocabularies + weights), word <-> id mapping, output formatting, and the two
// symbols the reference exports for its Python wrapper and server.
//
// Mirrors DecoderSentence (src/decoder_sentence.cu:14-388) and the output format of
// Decoder<T>::ObtainOneBestHypothesis (src/decoder.h:777-856) without Boost.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>
#include <sys/stat.h>

#include "engine.h"


namespace linmt {

// ---- config file: param="--key" value="..." lines, '#' comments -------------------------
// (DecoderSentence::ReadConfigFile, src/decoder_sentence.cu:267-318)
bool read_config_file(const std::string& path, std::map<std::string, std::string>& kv, std::string& err) {
  std::ifstream in(path.c_str());
  if (!in) { err = "Config File " + path + " does not exist"; return false; }
  std::string line;
  while (std::getline(in, line)) {
    while (!line.empty() && (line.back() == '\r' || line.back() == '\n' || line.back() == ' ' || line.back() == '\t')) line.pop_back();
    size_t b = 0;
    while (b < line.size() && (line[b] == ' ' || line[b] == '\t')) ++b;
    line = line.substr(b);
    if (line.empty() || line[0] == '#') continue;
    const size_t pp = line.find("param=\""), vp = line.find("value=\"");
    if (pp == std::string::npos || vp == std::string::npos) continue;
    const size_t pe = line.find('"', pp + 7), ve = line.find('"', vp + 7);
    if (pe == std::string::npos || ve == std::string::npos) continue;
    kv[line.substr(pp + 7, pe - pp - 7)] = line.substr(vp + 7, ve - vp - 7);
  }
  return true;
}

static std::vector<std::string> split_ws(const std::string& s) {
  std::vector<std::string> out;
  std::istringstream iss(s);
  std::string w;
  while (iss >> w) out.push_back(w);
  return out;
}

struct SentenceConfig {
  linmt_options opt;
  std::vector<std::string> model_names;
  int longest_sentence;  // user value + 4 (src/decoder_sentence.cu:126)
  int print_align_scores;
  int model_cache;       // 1 = keep / use a binary copy of the weights next to a text model
  std::vector<int32_t> devices;   // --devices: GPUs that each hold a replica and share the sentences (empty: opt.device)
};

// DecoderSentence::GeneralSettings, src/decoder_sentence.cu:110-264.  Like the reference,
// --decoding-ratio is parsed as two INTEGERS (atoi/stoi, :224-225) and --penalty is not
// read in sentence mode.  Keys beyond the reference's: --precision, --attention-type,
// --ensemble-mode, --batch-size, --device, --devices, --max-src-len, --gemm-path.  --devices "0 1 ..." puts a
// replica of the model(s) on every listed GPU and deals the sentences of a file (or of a batch call) to them.
// The reference's --multi-gpu (one GPU index per ensemble member, src/decoder_sentence.cu:183-198) is read
// as the same list without repeats: here every member lives on every listed GPU.
bool sentence_settings(const std::map<std::string, std::string>& kv, SentenceConfig& c, std::string& err) {
  linmt_default_options(&c.opt);
  auto get = [&](const char* key) -> const std::string* {
    auto it = kv.find(key);
    return it == kv.end() ? nullptr : &it->second;
  };
  int longest = 100;  // src/global_configuration.h:298
  if (auto v = get("--longest-sent")) longest = std::atoi(v->c_str());
  c.longest_sentence = longest + 4;
  if (auto v = get("--beam-size")) c.opt.beam = std::atoi(v->c_str());
  if (auto v = get("--attention-width")) c.opt.attention_d = std::atoi(v->c_str());
  if (auto v = get("--print-decoding-info")) c.opt.print_info = std::atoi(v->c_str()) ? 1 : 0;
  c.print_align_scores = 0;
  if (auto v = get("--print-align-scores")) c.print_align_scores = std::atoi(v->c_str());
  if (auto v = get("--nmt-model")) c.model_names = split_ws(*v);
  else { err = "you must assign --nmt-model in config file!"; return false; }
  if (c.model_names.empty()) { err = "you must assign --nmt-model in config file!"; return false; }
  c.model_cache = 1;
  if (auto v = get("--model-cache")) c.model_cache = std::atoi(v->c_str()) ? 1 : 0;
  if (auto v = get("--nbest")) c.opt.nbest = std::atoi(v->c_str());
  if (c.opt.beam <= 0) { err = "--beam-size cannot be <= 0!"; return false; }
  if (auto v = get("--decoding-ratio")) {
    std::vector<std::string> r = split_ws(*v);
    if (r.size() != 2) { err = "only two inputs for --decoding-ratio"; return false; }
    c.opt.min_ratio = (float)std::atoi(r[0].c_str());
    c.opt.max_ratio = (float)std::atoi(r[1].c_str());
    if (c.opt.min_ratio >= c.opt.max_ratio) { err = "min decoding ratio must be less than max decoding ratio!"; return false; }
  }
  if (auto v = get("--lp-alpha")) c.opt.lp_alpha = (float)std::atof(v->c_str());
  if (auto v = get("--cp-beta")) c.opt.cp_beta = (float)std::atof(v->c_str());
  if (auto v = get("--diversity")) c.opt.diversity = (float)std::atof(v->c_str());
  if (auto v = get("--precision")) {
    if (*v == "fp32") c.opt.precision = LINMT_PREC_FP32;
    else if (*v == "bf16") c.opt.precision = LINMT_PREC_BF16;
    else { err = "--precision must be fp32 or bf16"; return false; }
  }
  if (auto v = get("--attention-type")) {
    if (*v == "local_p_general") c.opt.attention_mode = LINMT_ATT_LOCAL_P_GENERAL;
    else if (*v == "global_general") c.opt.attention_mode = LINMT_ATT_GLOBAL_GENERAL;
    else if (*v == "global_dot") c.opt.attention_mode = LINMT_ATT_GLOBAL_DOT;
    else { err = "--attention-type must be local_p_general, global_general or global_dot"; return false; }
  }
  if (auto v = get("--ensemble-mode")) {
    if (*v == "prob_mean") c.opt.ensemble_mode = LINMT_ENS_PROB_MEAN;
    else if (*v == "logprob_mean") c.opt.ensemble_mode = LINMT_ENS_LOGPROB_MEAN;
    else { err = "--ensemble-mode must be prob_mean or logprob_mean"; return false; }
  }
  if (auto v = get("--gemm-path")) {
    if (*v == "auto") c.opt.gemm_path = LINMT_GEMM_AUTO;
    else if (*v == "simt") c.opt.gemm_path = LINMT_GEMM_SIMT;
    else if (*v == "tensor") c.opt.gemm_path = LINMT_GEMM_TENSOR;
    else if (*v == "tensor2") c.opt.gemm_path = LINMT_GEMM_TENSOR2;
    else if (*v == "tensor3") c.opt.gemm_path = LINMT_GEMM_TENSOR3;
    else if (*v == "tensor_v16") c.opt.gemm_path = LINMT_GEMM_TENSOR_V16;
    else if (*v == "tensor_v16x") c.opt.gemm_path = LINMT_GEMM_TENSOR_V16X;
    else { err = "--gemm-path must be auto, simt, tensor, tensor2, tensor3, tensor_v16 or tensor_v16x"; return false; }
  }
  if (auto v = get("--batch-size")) c.opt.max_batch = std::atoi(v->c_str());
  if (auto v = get("--device")) c.opt.device = std::atoi(v->c_str());
  for (const char* key : {"--devices", "--multi-gpu"})
    if (auto v = get(key)) {
      c.devices.clear();
      for (const std::string& w : split_ws(*v)) {
        const int32_t d = std::atoi(w.c_str());
        if (std::find(c.devices.begin(), c.devices.end(), d) == c.devices.end()) c.devices.push_back(d);
      }
      break;
    }
  if (auto v = get("--max-src-len")) c.opt.max_src_len = std::atoi(v->c_str());
  // the sentence API decodes one sentence per call unless told otherwise
  if (!get("--batch-size")) c.opt.max_batch = 1;
  c.opt.max_steps = std::max(1, c.longest_sentence - 2);
  if (!get("--max-src-len")) c.opt.max_src_len = std::max(1, c.longest_sentence);
  return true;
}

// ---- model file -------------------------------------------------------------------------
// Line 1: nine integers (src/decoder.h:1202-1210); "===" line; source map "id word";
// "===" line; target map; "===" line (src/decoder_sentence.cu:321-388); then the matrices
// in LoadWeights order, `rows` text lines of `cols` values and one blank line each, value
// (i,j) at column-major offset j*rows+i (src/deep_rnn_kernel.h:1543-1560).  A binary body
// ("BINARY <count>" line followed by raw little-endian floats in the same order and layout)
// is accepted as a faster form of the same file.
//
// Parsing the text body of a full-size model (~2 GB of decimal text for 4 x 1000, 30k / 30k)
// takes tens of seconds, so after a successful parse the weights are also written, raw, to
// "<model>.linmtcache" (header: magic, the nine integers, size and mtime of the text file, float
// count), and later loads of the same unchanged text file read that instead.  The cache is only
// ever a copy: a text file with another size or mtime, or other dimensions, invalidates it; an
// unwritable directory just means no cache.
struct ModelFile {
  linmt_model_desc desc{};
  int header[9]{};
  std::vector<std::pair<std::string, int>> src_words;
  std::vector<std::string> tgt_words;
  std::vector<float> blob;
};

static bool is_sep(const std::string& s) { return s.size() > 3 && s[0] == '=' && s[1] == '=' && s[2] == '='; }

static const char kCacheMagic[8] = {'L', 'I', 'N', 'M', 'T', 'B', 'I', '1'};
struct CacheHeader {
  char magic[8];
  int32_t header[9];
  int32_t pad;
  uint64_t text_size;
  int64_t text_mtime;
  uint64_t n_floats;
};
static bool stat_text(const std::string& path, uint64_t& size, int64_t& mtime) {
  struct stat st;
  if (stat(path.c_str(), &st) != 0) return false;
  size = (uint64_t)st.st_size; mtime = (int64_t)st.st_mtime;
  return true;
}
static bool cache_read(const std::string& path, const int32_t* header9, std::vector<float>& blob) {
  uint64_t size; int64_t mtime;
  if (!stat_text(path, size, mtime)) return false;
  FILE* c = std::fopen((path + ".linmtcache").c_str(), "rb");
  if (!c) return false;
  CacheHeader h;
  bool ok = std::fread(&h, sizeof h, 1, c) == 1 && std::memcmp(h.magic, kCacheMagic, 8) == 0 &&
            std::memcmp(h.header, header9, sizeof h.header) == 0 && h.text_size == size && h.text_mtime == mtime &&
            h.n_floats == blob.size();
  if (ok) ok = std::fread(blob.data(), sizeof(float), blob.size(), c) == blob.size();
  std::fclose(c);
  return ok;
}
static void cache_write(const std::string& path, const int32_t* header9, const std::vector<float>& blob) {
  CacheHeader h{};
  std::memcpy(h.magic, kCacheMagic, 8);
  std::memcpy(h.header, header9, sizeof h.header);
  if (!stat_text(path, h.text_size, h.text_mtime)) return;
  h.n_floats = blob.size();
  const std::string tmp = path + ".linmtcache.tmp", fin = path + ".linmtcache";
  FILE* c = std::fopen(tmp.c_str(), "wb");
  if (!c) return;
  const bool ok = std::fwrite(&h, sizeof h, 1, c) == 1 && std::fwrite(blob.data(), sizeof(float), blob.size(), c) == blob.size();
  if (std::fclose(c) != 0 || !ok || std::rename(tmp.c_str(), fin.c_str()) != 0) std::remove(tmp.c_str());
}

bool read_model_file(const std::string& path, ModelFile& mf, bool want_weights, std::string& err, bool use_cache = false) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) { err = "can not open " + path + " file!"; return false; }
  std::vector<char> buf(1 << 22);
  auto getline = [&](std::string& out) -> bool {
    out.clear();
    bool any = false;
    while (std::fgets(buf.data(), (int)buf.size(), f)) {
      any = true;
      const size_t n = std::strlen(buf.data());
      out.append(buf.data(), n);
      if (n && buf[n - 1] == '\n') { out.pop_back(); break; }
    }
    if (!out.empty() && out.back() == '\r') out.pop_back();
    return any;
  };
  std::string line;
  if (!getline(line)) { std::fclose(f); err = "empty model file"; return false; }
  {
    std::vector<std::string> h = split_ws(line);
    if (h.size() < 6) { std::fclose(f); err = "bad model header"; return false; }
    for (size_t i = 0; i < 9; ++i) mf.header[i] = i < h.size() ? std::atoi(h[i].c_str()) : 0;
    mf.desc.layers = mf.header[0]; mf.desc.hidden = mf.header[1]; mf.desc.vocab_tgt = mf.header[2];
    mf.desc.vocab_src = mf.header[3]; mf.desc.feed_input = mf.header[5];
    if (!mf.header[4]) { std::fclose(f); err = "model has no attention layer; only attention models are supported"; return false; }
    if (mf.header[6] || mf.header[7] || mf.header[8]) { std::fclose(f); err = "multi-source / char-cnn models are not supported"; return false; }
  }
  getline(line);  // the first separator
  while (getline(line)) {
    if (is_sep(line)) break;
    std::istringstream iss(line);
    std::string idx, word;
    iss >> idx >> word;
    if (!idx.empty()) mf.src_words.push_back({word, std::atoi(idx.c_str())});
  }
  mf.tgt_words.assign(mf.desc.vocab_tgt, "");
  while (getline(line)) {
    if (is_sep(line)) break;
    std::istringstream iss(line);
    std::string idx, word;
    iss >> idx >> word;
    if (idx.empty()) continue;
    const int i = std::atoi(idx.c_str());
    if (i >= 0 && i < mf.desc.vocab_tgt) mf.tgt_words[i] = word;
  }
  if (!want_weights) { std::fclose(f); return true; }
  const size_t n = linmt_blob_floats(&mf.desc);
  mf.blob.resize(n);
  const long body = std::ftell(f);
  if (getline(line) && line.compare(0, 6, "BINARY") == 0) {
    const size_t cnt = (size_t)std::strtoull(line.c_str() + 6, nullptr, 10);
    if (cnt != n) { std::fclose(f); err = "binary model body has the wrong size"; return false; }
    const size_t got = std::fread(mf.blob.data(), sizeof(float), n, f);
    std::fclose(f);
    if (got != n) { err = "truncated model file"; return false; }
    return true;
  }
  std::fseek(f, body, SEEK_SET);
  int32_t header9[9];
  for (int i = 0; i < 9; ++i) header9[i] = mf.header[i];
  if (use_cache && cache_read(path, header9, mf.blob)) { std::fclose(f); return true; }
  // text matrices
  const int H = mf.desc.hidden, L = mf.desc.layers;
  std::vector<std::pair<int, int>> shapes;
  auto lstm = [&](bool first, int vocab, bool feed) {
    for (int g = 0; g < 4; ++g) { shapes.push_back({H, H}); shapes.push_back({H, 1}); }
    if (first) shapes.push_back({H, vocab});
    for (int g = 0; g < 4; ++g) shapes.push_back({H, H});
    if (feed) for (int g = 0; g < 4; ++g) shapes.push_back({H, H});
  };
  for (int l = 0; l < L; ++l) lstm(l == 0, mf.desc.vocab_src, false);
  for (int l = 0; l < L; ++l) lstm(l == 0, mf.desc.vocab_tgt, l == 0 && mf.desc.feed_input);
  shapes.push_back({H, H}); shapes.push_back({H, H}); shapes.push_back({H, 1}); shapes.push_back({H, 1});
  shapes.push_back({H, H}); shapes.push_back({H, H});
  shapes.push_back({mf.desc.vocab_tgt, H}); shapes.push_back({mf.desc.vocab_tgt, 1});
  float* dst = mf.blob.data();
  for (auto& sh : shapes) {
    const int rows = sh.first, cols = sh.second;
    for (int i = 0; i < rows; ++i) {
      if (!getline(line)) { std::fclose(f); err = "truncated model file"; return false; }
      const char* p = line.c_str();
      char* end = nullptr;
      for (int j = 0; j < cols; ++j) {
        const double v = std::strtod(p, &end);
        if (end == p) { std::fclose(f); err = "bad number in model file"; return false; }
        dst[(size_t)j * rows + i] = (float)v;
        p = end;
      }
    }
    getline(line);  // blank line after each matrix
    dst += (size_t)rows * cols;
  }
  std::fclose(f);
  if (use_cache) cache_write(path, header9, mf.blob);
  return true;
}

// ---- formatting -------------------------------------------------------------------------
static std::string float_to_string(float v) {  // std::stringstream << float, src/utility_cc.cc:291-295
  std::stringstream oss;
  oss << v;
  return oss.str();
}

// Text of Decoder<T>::ObtainOneBestHypothesis's result (src/decoder.h:777-856) followed by
// DecoderSentence::UnintSentence (src/decoder_sentence.cu:72-107).
std::string format_result(const Engine& e, int S, int nbest, int max_len, const int32_t* tok, const int32_t* len,
                          const float* score, const int32_t* vit, const float* align, int max_src, bool fixed3 = false) {
  // file mode prints every float with three decimals (the stream is set to fixed, precision 3,
  // src/decoder.h:267); sentence mode with the stream's default six significant digits
  auto fmt = [&](float v) {
    if (!fixed3) return float_to_string(v);
    char b[64];
    std::snprintf(b, sizeof b, "%.3f", v);
    return std::string(b);
  };
  std::string ids_out;
  for (int q = 0; q < nbest; ++q) {
    const int n = len[q];
    if (n == 0) continue;
    const int32_t* t = tok + (size_t)q * max_len;
    const int32_t* v = vit + (size_t)q * max_len;
    bool first = true;
    for (int j = 1; j < n - 1; ++j) {
      if (!first) ids_out += " ";
      ids_out += std::to_string(t[j]);
      first = false;
    }
    if (e.opt.print_info) {
      ids_out += " |||| " + fmt(score[q]);
      ids_out += " ||||";
      int cnt = 0;
      for (int j = 1; j < n - 1; ++j) { ++cnt; ids_out += " " + std::to_string(v[j + 1]); }
      if (cnt == 0) ids_out += " ";
      ids_out += " ||||";
      int unk = 0;
      for (int j = 1; j < n - 1; ++j)
        if (t[j] == 2) { ++unk; ids_out += " " + std::to_string(v[j + 1]); }
      if (unk == 0) ids_out += " -1";
      if (e.print_align_scores && align) {
        ids_out += " ||||";
        int c2 = 0;
        for (int j = 1; j < n - 1; ++j) {
          ++c2;
          ids_out += " ";
          for (int s = 0; s < S; ++s) {
            if (s) ids_out += "/";
            ids_out += fmt(align[((size_t)q * max_len + (j + 1)) * max_src + s]);
          }
        }
        if (c2 == 0) ids_out += " ";
      }
    }
  }
  // ids -> words, keep everything from the first "||||" on
  std::istringstream iss(ids_out);
  std::vector<int> ids;
  std::string other, w;
  bool other_flag = false;
  while (iss >> w) {
    if (other_flag) other += " " + w;
    else if (w != "||||") ids.push_back(std::atoi(w.c_str()));
    else { other_flag = true; other += " " + w; }
  }
  if (other.size() >= 4 && other.compare(other.size() - 4, 4, "||||") == 0) other += " ";
  std::string out;
  for (size_t i = 0; i < ids.size(); ++i) {
    if (ids[i] >= 0 && ids[i] < (int)e.tgt_words.size()) out += e.tgt_words[ids[i]];
    if (i + 1 != ids.size()) out += " ";
  }
  out += other;
  return out;
}

}  // namespace linmt

static std::string g_front_error;

extern "C" {

int linmt_create(const char* config_path, linmt_engine** out) {
  using namespace linmt;
  if (!config_path || !out) { g_front_error = "null argument"; return LINMT_EINVAL; }
  *out = nullptr;
  std::map<std::string, std::string> kv;
  std::string err;
  if (!read_config_file(config_path, kv, err)) { g_front_error = err; return LINMT_EIO; }
  SentenceConfig sc;
  if (!sentence_settings(kv, sc, err)) { g_front_error = err; return LINMT_EINVAL; }
  std::vector<ModelFile> mfs(sc.model_names.size());
  for (size_t i = 0; i < mfs.size(); ++i) {
    if (!read_model_file(sc.model_names[i], mfs[i], true, err, sc.model_cache != 0)) { g_front_error = err; return LINMT_EIO; }
    if (i && std::memcmp(&mfs[i].desc, &mfs[0].desc, sizeof(linmt_model_desc)) != 0) {
      g_front_error = "ensemble members must have the same dimensions";
      return LINMT_EINVAL;
    }
  }
  std::vector<const float*> blobs;
  for (auto& m : mfs) blobs.push_back(m.blob.data());
  linmt_engine* e = nullptr;
  int rc = linmt_create_from_weights_on(&mfs[0].desc, blobs.data(), (int)blobs.size(), mfs[0].blob.size(), &sc.opt,
                                        sc.devices.data(), (int32_t)sc.devices.size(), &e);
  if (rc != LINMT_OK) { g_front_error = linmt_last_error(nullptr); return rc; }
  e->eng.tgt_words = mfs[0].tgt_words;
  e->eng.src_words_sorted = mfs[0].src_words;
  std::sort(e->eng.src_words_sorted.begin(), e->eng.src_words_sorted.end());
  // Unknown words read the id of the source map's "UNK" entry; looking that key up in the reference's map
  // inserts id 0 when the model has no such word (src/decoder_sentence.cu:61-62).
  e->eng.src_unk_id = 0;
  {
    auto it = std::lower_bound(e->eng.src_words_sorted.begin(), e->eng.src_words_sorted.end(), std::make_pair(std::string("UNK"), INT32_MIN));
    if (it != e->eng.src_words_sorted.end() && it->first == "UNK") e->eng.src_unk_id = it->second;
  }
  e->eng.longest_sentence = sc.longest_sentence;
  e->eng.print_align_scores = sc.print_align_scores;
  *out = e;
  return LINMT_OK;
}

const char* linmt_front_error(void) { return g_front_error.c_str(); }

int linmt_read_model_file(const char* path, linmt_model_desc* desc, float* blob, uint64_t blob_cap, int32_t use_cache) {
  if (!path || !desc) return LINMT_EINVAL;
  linmt::ModelFile mf;
  std::string err;
  if (!linmt::read_model_file(path, mf, blob != nullptr, err, use_cache != 0)) { g_front_error = err; return LINMT_EIO; }
  *desc = mf.desc;
  if (blob) {
    if (blob_cap < mf.blob.size()) { g_front_error = "blob buffer too small"; return LINMT_ELIMIT; }
    std::memcpy(blob, mf.blob.data(), mf.blob.size() * sizeof(float));
  }
  return LINMT_OK;
}

// DecoderSentence::Process (src/decoder_sentence.cu:40-49).
const char* linmt_translate(linmt_engine* h, const char* sentence) {
  using namespace linmt;
  if (!h) return "";
  Engine& e = h->eng;
  e.result_buf.clear();
  if (!sentence || !*sentence) return e.result_buf.c_str();
  std::string in(sentence);
  const size_t cut = in.find(" |||| ");
  if (cut != std::string::npos) in = in.substr(0, cut);
  std::vector<int32_t> ids;
  {
    std::istringstream iss(in);
    std::string w;
    while (iss >> w) {
      auto it = std::lower_bound(e.src_words_sorted.begin(), e.src_words_sorted.end(), std::make_pair(w, INT32_MIN));
      if (it != e.src_words_sorted.end() && it->first == w) ids.push_back(it->second);
      else ids.push_back(e.src_unk_id);  // src/decoder_sentence.cu:61-62
    }
  }
  if (ids.empty()) return e.result_buf.c_str();
  const int S = (int)ids.size();
  if (S > e.opt.max_src_len) { e.err = "sentence longer than --longest-sent"; return e.result_buf.c_str(); }
  int32_t off[2] = {0, S};
  int32_t steps = std::min((int)(e.opt.max_ratio * S), e.longest_sentence - 2);  // src/decoder.h:1806
  if (steps < 0) steps = 0;
  const int max_len = steps + 2;
  const int nb = e.opt.nbest;
  std::vector<int32_t> tok((size_t)nb * max_len), len(nb), vit((size_t)nb * max_len, -1);
  std::vector<float> score(nb), align;
  const bool want_align = e.opt.print_info && e.print_align_scores;
  if (want_align) align.resize((size_t)nb * max_len * e.opt.max_src_len);
  int rc = e.decode_host(ids.data(), off, 1, &steps, max_len, tok.data(), len.data(), score.data(), vit.data(),
                         want_align ? align.data() : nullptr, nullptr);
  if (rc != LINMT_OK) return e.result_buf.c_str();
  e.result_buf = format_result(e, S, nb, max_len, tok.data(), len.data(), score.data(), vit.data(),
                               want_align ? align.data() : nullptr, e.opt.max_src_len);
  return e.result_buf.c_str();
}

// File-mode decoding on top of the batch API: EnsembleFactory::DecodeFile (src/decoder.h:1702-1776)
// with Decoder::OutputKBestHypotheses (src/decoder.h:529-699) and InputFilePreprocess::UnintFile
// (src/input_file_preprocess.cc:1485-1572).  One source sentence per input line; per sentence the
// n-best hypotheses one per line (words, then " |||| score |||| alignments |||| unk-alignments"
// when print-decoding-info is on; scores with three decimals as the reference's file stream prints
// them, src/decoder.h:267), followed by a line of sixteen '=' when nbest != 1.  Sentences are
// decoded in length-sorted batches of --batch-size and written back in input order; a sentence
// longer than --longest-sent yields an empty line (the reference's file preprocessing drops it,
// src/input_file_preprocess.cc:1430-1438).
int linmt_decode_file(linmt_engine* h, const char* in_path, const char* out_path) {
  using namespace linmt;
  if (!h || !in_path || !out_path) return LINMT_EINVAL;
  Engine& e = h->eng;
  std::ifstream in(in_path);
  if (!in) { e.err = std::string("can not open ") + in_path; return LINMT_EIO; }
  std::vector<std::vector<int32_t>> sents;
  std::string line;
  while (std::getline(in, line)) {
    const size_t cut = line.find(" |||| ");
    if (cut != std::string::npos) line = line.substr(0, cut);
    std::vector<int32_t> ids;
    std::istringstream iss(line);
    std::string w;
    while (iss >> w) {
      auto it = std::lower_bound(e.src_words_sorted.begin(), e.src_words_sorted.end(), std::make_pair(w, INT32_MIN));
      ids.push_back((it != e.src_words_sorted.end() && it->first == w) ? it->second : e.src_unk_id);
    }
    if ((int)ids.size() > e.opt.max_src_len) ids.clear();
    sents.push_back(std::move(ids));
  }
  const int n_all = (int)sents.size();
  std::vector<int> order;
  for (int i = 0; i < n_all; ++i) if (!sents[i].empty()) order.push_back(i);
  auto steps_of = [&](int i) {
    int st = std::min((int)(e.opt.max_ratio * (int)sents[i].size()), e.longest_sentence - 2);  // src/decoder.h:1806
    return st < 0 ? 0 : st;
  };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return steps_of(a) > steps_of(b); });
  std::vector<std::string> results(n_all);
  const int nb = e.opt.nbest, B = e.opt.max_batch;
  const bool info = e.opt.print_info != 0;
  const bool want_align = info && e.print_align_scores;
  // one job per device batch; with several devices each device's host thread takes the next batch when it is
  // free (the batches are in descending step count, so the long ones go first)
  std::vector<int> batch_ids;
  for (size_t b0 = 0; b0 < order.size(); b0 += B) batch_ids.push_back((int)(b0 / B));
  const int rc_all = run_on_engines(h, batch_ids, [&](Engine& g, int bi) -> int {
    const size_t b0 = (size_t)bi * B;
    const int n = (int)std::min<size_t>(B, order.size() - b0);
    std::vector<int32_t> ids, off(1, 0), steps;
    int Tm = 0;
    for (int i = 0; i < n; ++i) {
      const auto& sv = sents[order[b0 + i]];
      ids.insert(ids.end(), sv.begin(), sv.end());
      off.push_back((int32_t)ids.size());
      steps.push_back(steps_of(order[b0 + i]));
      Tm = std::max(Tm, steps.back());
    }
    const int max_len = Tm + 2;
    std::vector<int32_t> tok((size_t)n * nb * max_len), len((size_t)n * nb), vit((size_t)n * nb * max_len, -1);
    std::vector<float> score((size_t)n * nb), align;
    if (want_align) align.resize((size_t)n * nb * max_len * e.opt.max_src_len);
    int rc = g.decode_host(ids.data(), off.data(), n, steps.data(), max_len, tok.data(), len.data(), score.data(), vit.data(),
                           want_align ? align.data() : nullptr, nullptr);
    if (rc != LINMT_OK) return rc;
    for (int i = 0; i < n; ++i) {
      const int S = off[i + 1] - off[i];
      std::string out;
      for (int q = 0; q < nb; ++q) {
        const size_t ob = (size_t)i * nb + q;
        if (len[ob] == 0) continue;
        // one hypothesis through the sentence formatter, floats with three decimals
        int32_t one_len = len[ob];
        std::string hyp = format_result(e, S, 1, max_len, &tok[ob * max_len], &one_len, &score[ob], &vit[ob * max_len],
                                        want_align ? &align[ob * max_len * e.opt.max_src_len] : nullptr, e.opt.max_src_len, true);
        out += hyp + "\n";
      }
      if (nb != 1) out += "================\n";
      results[order[b0 + i]] = out;
    }
    return LINMT_OK;
  });
  if (rc_all != LINMT_OK) return rc_all;
  std::ofstream outf(out_path);
  if (!outf) { e.err = std::string("can not open ") + out_path; return LINMT_EIO; }
  for (int i = 0; i < n_all; ++i) {
    if (results[i].empty()) outf << (nb != 1 ? "\n================\n" : "\n");
    else outf << results[i];
  }
  return LINMT_OK;
}

// ---- the reference's exported pair (src/decoder_sentence.cu:844-873) ---------------------
static linmt_engine* g_singleton = nullptr;
static char* g_result = nullptr;
static std::mutex g_mutex;

void python_decoder_init(char* msg) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_singleton) { linmt_destroy(g_singleton); g_singleton = nullptr; }
  int rc = linmt_create(msg, &g_singleton);
  if (rc != LINMT_OK) {
    std::fprintf(stderr, "   Error: %s\n", g_front_error.c_str());
    std::exit(EXIT_FAILURE);
  }
}

char* python_decoder_do_job(char* sentence) {
  std::lock_guard<std::mutex> lock(g_mutex);
  delete[] g_result;
  g_result = nullptr;
  std::string out;
  if (g_singleton && sentence && *sentence) out = linmt_translate(g_singleton, sentence);
  g_result = new char[out.size() + 1];
  std::memcpy(g_result, out.c_str(), out.size() + 1);
  return g_result;
}

}  // extern "C"

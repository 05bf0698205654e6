// unk_post.cpp -- UNK post-processing of a decoded line: what LiNMT's Python wrapper and TCP
// server call right after python_decoder_do_job (server/LiNMT-server.py:52-57).  Host string
// code, no GPU.  Behaviour follows PostProcessUnks (src/postprocess_unks.cc): every "<UNK>" of
// the translation is replaced through its viterbi alignment by a dictionary entry / a
// generalization of the source line / the source word in angle brackets, generalization labels
// ($number, $time, ...) are filled from the source line's list, then repeated words, repeated
// bigrams and repeated end punctuation are collapsed.
//
// Organisation here: one table of labels (label -> slot of the generalization store) instead of
// the reference's twenty parallel maps and if-chains; text helpers with the reference's exact
// splitting rules (utility_cc.cc:132-230).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <fstream>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include "../../include/linmt_decoder.h"

namespace linmt {
namespace unk {

typedef std::vector<std::string> Words;

// pieces between single-character separators, empty pieces dropped (BasicMethod::Split)
static Words split_char(const std::string& s, char c) {
  Words out;
  size_t start = 0;
  while (start <= s.size()) {
    size_t end = s.find(c, start);
    if (end == std::string::npos) end = s.size();
    if (end > start) out.push_back(s.substr(start, end - start));
    start = end + 1;
  }
  return out;
}

// pieces between string separators: a separator at the very start is skipped, empty pieces in the
// middle are kept, nothing follows a trailing separator (BasicMethod::SplitWithString)
static Words split_str(const std::string& s, const std::string& sep) {
  Words out;
  size_t start = 0;
  while (start < s.size()) {
    const size_t idx = s.find(sep, start);
    if (idx == 0) { start += sep.size(); continue; }
    if (idx == std::string::npos) { out.push_back(s.substr(start)); break; }
    out.push_back(s.substr(start, idx - start));
    start = idx + sep.size();
  }
  return out;
}

static void strip_newlines(std::string& s) {
  s.erase(std::remove_if(s.begin(), s.end(), [](char ch) { return ch == '\r' || ch == '\n'; }), s.end());
}
static void strip_leading_spaces(std::string& s) {
  size_t p = 0;
  while (p < s.size() && s[p] == ' ') ++p;
  s.erase(0, p);
}
static void strip_trailing_spaces(std::string& s) {
  while (!s.empty() && s.back() == ' ') s.pop_back();
}
static bool is_nmt_label(const std::string& w) { return w.size() > 5 && w.compare(0, 5, "$NMT_") == 0; }

// label of a generalization entry / of a target word -> slot of the store
static const std::unordered_map<std::string, std::string>& label_slots() {
  static const std::unordered_map<std::string, std::string> t = [] {
    std::unordered_map<std::string, std::string> m = {
        {"$number", "number"}, {"$time", "time"},     {"$date", "date"},        {"$day", "day"},        {"$psn", "person"},
        {"$loc", "location"},  {"$location", "location"}, {"$org", "organization"}, {"$literal", "literal"}};
    for (int i = 1; i <= 10; ++i) m["$userdict" + std::to_string(i)] = "userdict" + std::to_string(i);
    return m;
  }();
  return t;
}
// source words the search for a content word passes over (FindUnStopword: neither $day nor $location)
static bool unstop_skips(const std::string& w) {
  static const std::unordered_set<std::string> t = [] {
    std::unordered_set<std::string> s = {"$number", "$time", "$date", "$psn", "$loc", "$org", "$literal"};
    for (int i = 1; i <= 10; ++i) s.insert("$userdict" + std::to_string(i));
    return s;
  }();
  return t.count(w) != 0;
}

// source positions by descending alignment score, later position first among equals (the
// reference walks a multimap<float,int> backwards); false when the score list does not match
static bool ranked_positions(const std::string& scores, size_t n_src, std::vector<int>& order) {
  const Words f = split_char(scores, '/');
  if (f.size() != n_src) return false;
  std::vector<std::pair<float, int>> keyed;
  for (size_t i = 0; i < f.size(); ++i) keyed.emplace_back((float)atof(f[i].c_str()), (int)i);
  std::stable_sort(keyed.begin(), keyed.end(), [](const std::pair<float, int>& a, const std::pair<float, int>& b) {
    return a.first > b.first || (a.first == b.first && a.second > b.second);
  });
  order.clear();
  for (auto& kv : keyed) order.push_back(kv.second);
  return true;
}

class Processor {
 public:
  std::unordered_map<std::string, std::string> dict;
  std::unordered_set<std::string> stopwords, end_puncts;
  bool emit_oov = true;   // "--rm-oov-mode" 1 turns the "<source word>" output off
  std::string error;

  bool init(const std::string& config_path) {
    std::unordered_map<std::string, std::string> kv;
    if (!read_config(config_path, kv)) return false;
    if (kv.count("--rm-oov-mode")) emit_oov = !(std::atoi(kv["--rm-oov-mode"].c_str()) != 0);
    return load_dict(kv["--phrase-table"]) && load_second_column(kv["--stopword"], "", stopwords) &&
           load_second_column(kv["--end-punct"], "ENDPUNCT", end_puncts);
  }

  std::string process(std::string source, std::string translation) const {
    strip_newlines(translation);
    strip_newlines(source);
    const Words src_parts = split_str(source, " |||| ");
    source = src_parts.empty() ? std::string() : src_parts[0];
    std::unordered_map<std::string, std::unordered_map<int, std::string>> store;   // slot -> position -> text
    if (src_parts.size() == 2) {
      const std::string& g = src_parts[1];
      if (g.size() >= 3 && g.front() == '{' && g.back() == '}') {
        for (const std::string& entry : split_str(g.substr(1, g.size() - 2), "}{")) {
          const Words f = split_str(entry, " ||| ");
          if (f.size() != 5) continue;
          if (f[3] == "$dict") store["dict"][std::atoi(f[0].c_str())] = f[2];
          else {
            auto it = label_slots().find(f[3]);
            if (it != label_slots().end()) store[it->second][std::atoi(f[0].c_str())] = f[2];
          }
        }
      }
    }
    const Words fields = split_str(translation, " |||| ");
    if (fields.size() < 5) return translation;
    const Words src = split_char(source, ' ');
    Words tgt = split_char(fields[0], ' ');
    if (!tgt.empty() && tgt.back() == "." && !src.empty() && src.back() == ",") tgt.back() = ",";
    const Words score_fields = split_char(fields[4], ' ');
    std::vector<int> align;
    {
      std::istringstream in(fields[2]);
      int v;
      while (in >> v) align.push_back(v);
    }
    if (tgt.size() != align.size()) return translation;

    std::string out;
    auto& gdict = store["dict"];
    auto scores_of = [&](size_t i) { return i < score_fields.size() ? score_fields[i] : std::string(); };
    auto content_word = [&](size_t i) {   // best-aligned source position that is neither stopword nor label
      std::vector<int> order;
      if (!ranked_positions(scores_of(i), src.size(), order)) return -1;
      for (int p : order)
        if (!stopwords.count(src[p]) && !unstop_skips(src[p])) return p;
      return -1;
    };
    auto emit_from = [&](int pos, bool marked) {
      if (pos == -1) { out += " ."; return; }
      if (pos < 0 || (size_t)pos >= src.size()) return;
      const std::string& w = src[pos];
      if (is_nmt_label(w)) {
        auto it = gdict.find(pos);
        if (it != gdict.end()) out += " " + it->second;
      } else if (dict.count(w)) {
        out += marked ? " <UNK-" + dict.at(w) + ">" : " " + dict.at(w);
      } else if (emit_oov) {
        out += " <" + w + ">";
      }
    };

    for (size_t i = 0; i < tgt.size(); ++i) {
      const std::string& w = tgt[i];
      const int a = align[i];
      auto lab = label_slots().find(w);
      if (w == "<UNK>") {
        if (a < 0 || (size_t)a >= src.size()) continue;
        const std::string& sw = src[a];
        if (is_nmt_label(sw)) {
          auto it = gdict.find(a);
          if (it != gdict.end()) out += " " + it->second;
        } else if (stopwords.count(sw)) {
          emit_from(content_word(i), true);
        } else if (dict.count(sw)) {
          if (!label_slots().count(sw)) out += " <UNK-" + dict.at(sw) + ">";
          else emit_from(content_word(i), false);
        } else if (emit_oov) {
          out += " <" + sw + ">";
        }
      } else if (lab != label_slots().end()) {
        auto& slot = store[lab->second];
        auto it = slot.find(a);
        if (it == slot.end()) {
          std::vector<int> order;
          if (ranked_positions(scores_of(i), src.size(), order))
            for (int p : order) {
              it = slot.find(p);
              if (it != slot.end()) break;
            }
        }
        if (it != slot.end()) { out += " " + it->second; slot.erase(it); }
        else if (emit_oov) out += " <" + w + ">";
      } else {
        out += " " + w;
      }
    }
    strip_leading_spaces(out);
    out = join(drop_repeated_words(split_char(out, ' ')));
    out = drop_repeated_bigrams(split_char(out, ' '), out);
    out = drop_repeated_end_puncts(split_char(out, ' '));
    if (out.find("<UNK-") != std::string::npos) out = unmark(out);
    strip_leading_spaces(out);
    for (size_t i = 1; i < fields.size(); ++i) out += " |||| " + fields[i];
    return out;
  }

 private:
  static std::string join(const Words& w) {
    std::string s;
    for (size_t i = 0; i < w.size(); ++i) { if (i) s += " "; s += w[i]; }
    return s;
  }
  static Words drop_repeated_words(const Words& w) {
    Words kept;
    for (const std::string& x : w)
      if (kept.empty() || kept.back() != x) kept.push_back(x);
    return kept;
  }
  // The reference's scan (postprocess_unks.cc:541-562), kept step for step: it compares the bigram
  // ending at i with the last bigram it emitted and skips two words on a match.
  static std::string drop_repeated_bigrams(const Words& w, const std::string& unchanged) {
    const size_t n = w.size();
    if (n < 4) return unchanged;
    std::string out = w[0] + " " + w[1];
    std::string last = out;
    size_t i = 3;
    for (; i < n; ++i) {
      const std::string cur = w[i - 1] + " " + w[i];
      if (cur != last) { out += " " + w[i - 1]; last = w[i - 2] + " " + w[i - 1]; }
      else ++i;
    }
    if (n + 1 != i) out += " " + w[n - 1];
    return out;
  }
  std::string drop_repeated_end_puncts(const Words& w) const {
    std::string out;
    bool last_end = false;
    for (size_t i = 0; i < w.size(); ++i) {
      const bool is_end = end_puncts.count(w[i]) != 0;
      if (is_end && last_end) continue;
      last_end = is_end;
      if (i) out += " ";
      out += w[i];
    }
    return out;
  }
  // "<UNK-text>" markers become their text (BPE joints removed first); a following word that is
  // part of the text is dropped
  static std::string unmark(std::string s) {
    for (size_t p = 0; (p = s.find("@@ ", p)) != std::string::npos;) s.erase(p, 3);
    const Words w = split_char(s, ' ');
    std::string out;
    for (size_t i = 0; i < w.size(); ++i) {
      const std::string& x = w[i];
      if (x.size() >= 6 && x.compare(0, 5, "<UNK-") == 0 && x.back() == '>') {
        const std::string sub = x.substr(5, x.size() - 6);
        out += " " + sub;
        if (i + 1 < w.size() && sub.find(w[i + 1]) != std::string::npos) ++i;
      } else {
        out += " " + x;
      }
    }
    return out;
  }

  bool read_config(const std::string& path, std::unordered_map<std::string, std::string>& kv) {
    std::ifstream in(path.c_str());
    if (!in) { error = "config file " + path + " does not exist"; return false; }
    std::string line;
    while (std::getline(in, line)) {
      strip_newlines(line);
      strip_leading_spaces(line);
      strip_trailing_spaces(line);
      if (line.empty() || line[0] == '#') continue;
      std::string key, value;
      if (!quoted_after(line, "param=\"", key) || !quoted_after(line, "value=\"", value)) continue;
      kv[key] = value;
    }
    return true;
  }
  static bool quoted_after(const std::string& line, const char* tag, std::string& out) {
    size_t p = line.find(tag);
    if (p == std::string::npos) return false;
    p += std::strlen(tag);
    const size_t q = line.find('"', p);
    if (q == std::string::npos) return false;
    out = line.substr(p, q - p);
    return true;
  }
  bool load_dict(const std::string& path) {
    std::ifstream in(path.c_str());
    if (!in) { error = "can not open " + path; return false; }
    std::string line;
    while (std::getline(in, line)) {
      strip_newlines(line);
      const Words f = split_str(line, " ||| ");
      if (f.size() >= 2) dict[f[0]] = f[1];   // "source ||| target ||| anything"
    }
    return true;
  }
  // tab-separated "tag<TAB>word" lines; with a tag given only lines carrying it count
  bool load_second_column(const std::string& path, const std::string& tag, std::unordered_set<std::string>& out) {
    std::ifstream in(path.c_str());
    if (!in) { error = "can not open " + path; return false; }
    std::string line;
    while (std::getline(in, line)) {
      strip_newlines(line);
      const Words f = split_char(line, '\t');
      if (f.size() >= 2 && (tag.empty() || f[0] == tag)) out.insert(f[1]);
    }
    return true;
  }
};

}  // namespace unk
}  // namespace linmt

namespace {
std::mutex g_unk_mutex;
linmt::unk::Processor* g_unk = nullptr;
std::string g_unk_result;
}  // namespace

extern "C" {

void python_unk_init(char* msg) {
  std::lock_guard<std::mutex> lock(g_unk_mutex);
  auto* p = new linmt::unk::Processor();
  if (!p->init(msg ? msg : "")) {
    // the reference logs and exits on a missing configuration or resource file
    std::fprintf(stderr, "   ERROR: %s, exit!\n", p->error.c_str());
    std::exit(EXIT_FAILURE);
  }
  delete g_unk;
  g_unk = p;
}

char* python_unk_do_job(char* src_sentence, char* translation) {
  std::lock_guard<std::mutex> lock(g_unk_mutex);
  g_unk_result.clear();
  if (g_unk && src_sentence && translation && *src_sentence && *translation) {
    const linmt::unk::Words f = linmt::unk::split_str(g_unk->process(src_sentence, translation), " |||| ");
    if (f.size() > 1) g_unk_result = f[0];
  }
  return const_cast<char*>(g_unk_result.c_str());   // library-owned, valid until the next call
}

int linmt_unk_create(const char* config_path, linmt_unk** out) {
  if (!config_path || !out) return LINMT_EINVAL;
  auto* p = new linmt::unk::Processor();
  if (!p->init(config_path)) {
    delete p;
    return LINMT_EIO;
  }
  *out = reinterpret_cast<linmt_unk*>(p);
  return LINMT_OK;
}

int linmt_unk_process(const linmt_unk* h, const char* source, const char* translation, char* out, int32_t out_cap) {
  if (!h || !source || !translation || !out || out_cap < 1) return LINMT_EINVAL;
  const std::string r = reinterpret_cast<const linmt::unk::Processor*>(h)->process(source, translation);
  if ((size_t)out_cap <= r.size()) return LINMT_ELIMIT;
  std::memcpy(out, r.c_str(), r.size() + 1);
  return LINMT_OK;
}

void linmt_unk_destroy(linmt_unk* h) { delete reinterpret_cast<linmt::unk::Processor*>(h); }

}  // extern "C"

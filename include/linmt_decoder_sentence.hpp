// linmt_decoder_sentence.hpp -- the reference's DecoderSentence class for C++ callers, over the C ABI.
//
// The reference's own C++ caller is Dispatcher::DecodingSentence (src/dispatcher.cu:439-476):
//
//     DecoderSentence decoder_sentence;
//     decoder_sentence.Init(config_file);
//     while (std::getline(in, line)) { std::string out; decoder_sentence.Process(line, out); ... }
//
// This header gives that code the same class -- same method names, argument types and return values as
// src/decoder_sentence.h:36-41 -- so it compiles unchanged against liblinmt_decoder.so.  Header-only; link
// with -llinmt_decoder.  Differences from the reference class, all of them in what happens on failure:
// the reference prints and calls exit() from inside Init (src/decoder_sentence.cu:270-273, 173-176);
// here Init returns false and LastError() names the problem, and Process returns false (with an empty
// output) when the decode fails.  ProcessFile is the file form of the same loop, decoded in batches
// (EnsembleFactory::DecodeFile, src/decoder.h:1702-1776).
#ifndef LINMT_DECODER_SENTENCE_HPP_
#define LINMT_DECODER_SENTENCE_HPP_

#include <string>

#include "linmt_decoder.h"

class DecoderSentence {
 public:
  DecoderSentence() = default;
  DecoderSentence(const DecoderSentence&) = delete;
  DecoderSentence& operator=(const DecoderSentence&) = delete;
  ~DecoderSentence() {
    if (handle_) linmt_destroy(handle_);
  }

  // Reads the decoding-sentence config file, the model file(s) it names and their vocabularies, and puts the
  // model(s) on the GPU(s) (DecoderSentence::Init, src/decoder_sentence.cu:14-37).
  bool Init(std::string& config) {
    if (handle_) { linmt_destroy(handle_); handle_ = nullptr; }
    const int rc = linmt_create(config.c_str(), &handle_);
    if (rc != LINMT_OK) {
      error_ = linmt_front_error();
      handle_ = nullptr;
      return false;
    }
    error_.clear();
    return true;
  }

  // One whitespace-tokenised source sentence in, the translation (and, with --print-decoding-info, its
  // " |||| score |||| alignments |||| unk alignments" fields) out (DecoderSentence::Process,
  // src/decoder_sentence.cu:40-49).
  bool Process(const std::string& input_sentence, std::string& output_sentence) {
    output_sentence.clear();
    if (!handle_) { error_ = "Init was not called"; return false; }
    const char* out = linmt_translate(handle_, input_sentence.c_str());
    output_sentence = out ? out : "";
    if (output_sentence.empty() && !input_sentence.empty()) {
      const char* e = linmt_last_error(handle_);
      if (e && *e) { error_ = e; return false; }
    }
    return true;
  }

  // One sentence per line of in_path, n-best lists to out_path, decoded in length-sorted device batches
  // (and, with --devices, on several GPUs).
  bool ProcessFile(const std::string& in_path, const std::string& out_path) {
    if (!handle_) { error_ = "Init was not called"; return false; }
    const int rc = linmt_decode_file(handle_, in_path.c_str(), out_path.c_str());
    if (rc != LINMT_OK) { error_ = linmt_last_error(handle_); return false; }
    return true;
  }

  const std::string& LastError() const { return error_; }

 private:
  linmt_engine* handle_ = nullptr;
  std::string error_;
};

#endif  // LINMT_DECODER_SENTENCE_HPP_

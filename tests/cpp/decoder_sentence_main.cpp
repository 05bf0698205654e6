// The loop of the reference's Dispatcher::DecodingSentence (src/dispatcher.cu:439-476) written against
// include/linmt_decoder_sentence.hpp: config file, input file, output file; "[n] translation" lines.
// Exit code 2 = Init failed (the message goes to stderr), 3 = a file could not be opened, 4 = Process failed.
#include <fstream>
#include <iostream>
#include <string>

#include "linmt_decoder_sentence.hpp"

int main(int argc, char** argv) {
  if (argc != 4) { std::cerr << "usage: decoder_sentence_main config input output\n"; return 1; }
  std::string config = argv[1];
  DecoderSentence decoder_sentence;
  if (!decoder_sentence.Init(config)) { std::cerr << "Init failed: " << decoder_sentence.LastError() << "\n"; return 2; }
  std::ifstream in_file(argv[2]);
  std::ofstream out_file(argv[3]);
  if (!in_file || !out_file) return 3;
  int number_of_sentences = 0;
  std::string input_sentence;
  while (std::getline(in_file, input_sentence)) {
    ++number_of_sentences;
    std::string output_sentence;
    if (!decoder_sentence.Process(input_sentence, output_sentence)) return 4;
    out_file << "[" << number_of_sentences << "] " << output_sentence << "\n";
  }
  return 0;
}

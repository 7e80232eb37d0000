// Byte-level BPE tokenizer for the native front end: vocabulary, merges and special tokens from GGUF metadata
// (tokenizer.ggml.tokens / merges / token_type) or from a Hugging Face tokenizer.json, GPT-2 style byte-to-unicode mapping and pre-tokenisation.
// Role of the reference's cpp_engine/src/tokenizer.cpp and tools/minimax_gguf_tokenizer.
//
// Pre-tokenisation follows the GPT-2 pattern
//   's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
// with ASCII character classes; every byte >= 0x80 counts as a letter, so text in non-Latin scripts is grouped
// like letters (identical to the pattern for alphabetic scripts, an approximation for symbols and emoji).
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "gguf_reader.hpp"

namespace pk {

class BpeTokenizer {
 public:
  // tokens in the byte-level unicode alphabet; merges as "left right"; special = ids matched verbatim in the input
  BpeTokenizer(std::vector<std::string> tokens, const std::vector<std::string>& merges, const std::vector<int>& special);
  static BpeTokenizer from_gguf(const GgufFile& file);
  // A Hugging Face tokenizer directory (or the tokenizer.json file itself): model.vocab, model.merges (strings "a b" or
  // pairs ["a", "b"]) and added_tokens of a byte-level BPE tokenizer (reference: cpp_engine/include/tokenizer.hpp:14-40).
  static BpeTokenizer from_hf_dir(const std::string& dir_or_file);

  std::vector<int> encode(const std::string& text, bool parse_special = true) const;
  std::string decode(const std::vector<int>& ids, bool skip_special = false) const;
  int vocab_size() const { return (int)tokens_.size(); }
  int token_id(const std::string& piece) const;   // -1 when absent

  // exposed for tests
  static std::vector<std::string> pre_tokenize(const std::string& text);

 private:
  void bpe(const std::string& word, std::vector<int>& out) const;
  std::vector<std::string> tokens_;
  std::unordered_map<std::string, int> vocab_;
  std::unordered_map<std::string, int> rank_;      // "left\x01right" -> merge rank
  std::vector<std::pair<std::string, int>> special_;   // sorted by length, longest first
  std::vector<bool> is_special_;
  std::string byte_to_piece_[256];
  std::unordered_map<uint32_t, uint8_t> cp_to_byte_;
};

}  // namespace pk

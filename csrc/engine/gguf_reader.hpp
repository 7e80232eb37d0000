// GGUF v3 container reader for the native side: header, metadata key/values (all scalar types,
// strings, arrays), tensor table, alignment, and a read-only mmap of the tensor data.
// Plays the role of the reference's cpp_engine/src/gguf_reader.cpp (header/KV/tensor table/mmap).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "json.hpp"

namespace pk {

struct GgufTensor {
  std::string name;
  std::vector<uint64_t> dims;   // GGUF order: innermost dimension first
  uint32_t type = 0;
  uint64_t offset = 0;          // relative to the start of the data section
  uint64_t nbytes = 0;
  uint64_t elements() const;
};

const char* ggml_type_name(uint32_t type);
// {weights per block, bytes per block}; {0, 0} for an unknown type
std::pair<uint32_t, uint32_t> ggml_type_block(uint32_t type);

class GgufFile {
 public:
  explicit GgufFile(const std::string& path);
  ~GgufFile();
  GgufFile(const GgufFile&) = delete;
  GgufFile& operator=(const GgufFile&) = delete;

  uint32_t version() const { return version_; }
  uint64_t alignment() const { return alignment_; }
  // Metadata as a JSON object (arrays become JSON arrays; 64-bit integers stay exact).
  const Json& metadata() const { return meta_; }
  std::string architecture() const { return meta_.get_string("general.architecture", ""); }
  const std::vector<GgufTensor>& tensors() const { return tensors_; }
  const GgufTensor* find(const std::string& name) const;
  const uint8_t* data(const GgufTensor& t) const { return base_ + data_offset_ + t.offset; }
  uint64_t file_size() const { return size_; }

 private:
  void parse(const std::string& path);
  void release();
  std::string path_;
  int fd_ = -1;
  const uint8_t* base_ = nullptr;
  uint64_t size_ = 0, data_offset_ = 0, alignment_ = 32;
  uint32_t version_ = 0;
  Json meta_ = Json::object();
  std::vector<GgufTensor> tensors_;
  std::map<std::string, size_t> index_;
};

}  // namespace pk

// Memory-mapped Safetensors checkpoints: single file or `model.safetensors.index.json`
// plus shards. Counterpart of cpp_engine/src/safetensors_reader.cpp and
// safetensors_model.cpp in the reference.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace pk {

enum class StDtype { F32, F16, BF16, F8_E4M3, F8_E5M2, I8, U8, I32, I64, F8_E8M0, Unknown };

const char* st_dtype_name(StDtype d);
size_t st_dtype_size(StDtype d);

struct StTensor {
  std::string name;
  StDtype dtype = StDtype::Unknown;
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;  // inside the mapping
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

class MappedFile {
 public:
  explicit MappedFile(const std::string& path);
  ~MappedFile();
  MappedFile(const MappedFile&) = delete;
  MappedFile& operator=(const MappedFile&) = delete;
  const uint8_t* data() const { return data_; }
  size_t size() const { return size_; }
  const std::string& path() const { return path_; }

 private:
  std::string path_;
  int fd_ = -1;
  const uint8_t* data_ = nullptr;
  size_t size_ = 0;
};

class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string& path);
  const std::map<std::string, StTensor>& tensors() const { return tensors_; }
  const std::map<std::string, std::string>& metadata() const { return metadata_; }

 private:
  std::unique_ptr<MappedFile> file_;
  std::map<std::string, StTensor> tensors_;
  std::map<std::string, std::string> metadata_;
};

// A checkpoint directory (index + shards, or every *.safetensors file in it) or one file.
class SafetensorsModel {
 public:
  explicit SafetensorsModel(const std::string& path);
  bool has(const std::string& name) const { return lookup_.count(name) != 0; }
  const StTensor& get(const std::string& name) const;
  const StTensor* find(const std::string& name) const;
  std::vector<std::string> names() const;
  size_t num_files() const { return files_.size(); }

 private:
  std::vector<std::unique_ptr<SafetensorsFile>> files_;
  std::map<std::string, const StTensor*> lookup_;
};

}  // namespace pk

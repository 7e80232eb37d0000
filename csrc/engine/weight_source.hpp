// One lookup interface over the two checkpoint containers of DeepSeek-V4: a Safetensors directory (tensors under the
// model's own names, one tensor per routed expert) and a deepseek4 GGUF file (llama.cpp-style names, the experts of a
// layer packed into one 3-d tensor). Callers ask by the model's names; the GGUF source translates and cuts expert
// slices. Views borrow from the file mappings and stay valid as long as the source lives.
// Counterpart of the reference's cpp_engine/include/weight_source.hpp:16-115.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "dsv4_config.hpp"
#include "gguf_reader.hpp"
#include "safetensors.hpp"

namespace pk {

struct TensorView {
  std::string name;          // the model's name that was asked for
  std::string stored_name;   // the name inside the container
  std::string dtype;         // Safetensors dtype name or ggml type name
  std::vector<int64_t> shape;  // outermost dimension first
  const uint8_t* data = nullptr;
  uint64_t nbytes = 0;
  bool found = false;
};

class WeightSource {
 public:
  enum class Format { Safetensors, Gguf };
  virtual ~WeightSource() = default;
  virtual Format format() const = 0;
  virtual bool has(const std::string& name) const = 0;
  // found == false on a miss
  virtual TensorView get(const std::string& name) const = 0;
  TensorView require(const std::string& name) const;
  // Routed expert matrix `part` (w1 = gate, w2 = down, w3 = up) of expert `e` in layer `layer`: the expert's own tensor
  // (Safetensors) or its slice of the packed tensor (GGUF; rows stay quantised blocks).
  virtual TensorView expert(int layer, int e, const std::string& part) const = 0;
  virtual std::vector<std::string> names() const = 0;   // the model's names this source can serve
};

class SafetensorsSource : public WeightSource {
 public:
  explicit SafetensorsSource(const std::string& path);
  Format format() const override { return Format::Safetensors; }
  bool has(const std::string& name) const override { return model_.has(name); }
  TensorView get(const std::string& name) const override;
  TensorView expert(int layer, int e, const std::string& part) const override;
  std::vector<std::string> names() const override { return model_.names(); }
  const SafetensorsModel& model() const { return model_; }

 private:
  SafetensorsModel model_;
};

class GgufSource : public WeightSource {
 public:
  explicit GgufSource(const std::string& path);
  Format format() const override { return Format::Gguf; }
  bool has(const std::string& name) const override;
  TensorView get(const std::string& name) const override;
  TensorView expert(int layer, int e, const std::string& part) const override;
  std::vector<std::string> names() const override;
  const GgufFile& file() const { return file_; }
  const Dsv4Config& config() const { return cfg_; }
  // The container's name for one of the model's names ("" when the model has no such tensor in GGUF form).
  static std::string stored_name_for(const std::string& name);

 private:
  TensorView view_of(const GgufTensor& t, const std::string& asked) const;
  GgufFile file_;
  Dsv4Config cfg_;
};

bool is_gguf_path(const std::string& path);
std::unique_ptr<WeightSource> open_weight_source(const std::string& path);

}  // namespace pk

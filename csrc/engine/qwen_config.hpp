// Configuration of the hybrid Gated-DeltaNet / GQA decoder (Qwen3.x "next" family) parsed
// from a Hugging Face config.json (flat or nested under text_config). Same keys as the
// reference's QwenConfig::from_hf_config (cpp_engine/include/qwen_config.hpp:42-74).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace pk {

class Json;

struct QwenConfig {
  int64_t vocab_size = 0;
  int64_t hidden_size = 0;
  int64_t intermediate_size = 0;
  int num_layers = 0;
  std::vector<int> layer_is_full;  // 1 = full GQA attention, 0 = Gated DeltaNet
  // full attention
  int num_heads = 0;
  int num_kv_heads = 0;
  int head_dim = 128;
  bool attn_output_gate = true;
  double rope_theta = 1.0e6;
  double partial_rotary_factor = 0.25;
  // linear attention
  int linear_key_heads = 0;
  int linear_value_heads = 0;
  int linear_key_head_dim = 128;
  int linear_value_head_dim = 128;
  int linear_conv_kernel = 4;
  double rms_norm_eps = 1.0e-6;
  int64_t max_position_embeddings = 262144;
  int mtp_num_hidden_layers = 0;

  int rotary_dim() const { return (int)(head_dim * partial_rotary_factor) & ~1; }
  int num_full_layers() const;
  int num_linear_layers() const;
  void validate(int tp_world) const;  // throws std::runtime_error

  static QwenConfig from_json(const Json& root);
  static QwenConfig from_file(const std::string& path);
  // The 64-layer, hidden 5120 benchmark shape (3 DeltaNet layers then 1 GQA layer, repeated).
  static QwenConfig benchmark_27b();
  std::string to_json() const;
};

}  // namespace pk

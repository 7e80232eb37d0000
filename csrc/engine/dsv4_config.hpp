// DeepSeek-V4 model configuration on the native side: parsed from a checkpoint's config.json (the field names of the
// published model) or from the metadata of a deepseek4 GGUF. Counterpart of the reference's
// cpp_engine/src/model_config.cpp; the Python twin is pocketllm_b200/models/deepseek_v4.py (DSV4Config).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "json.hpp"

namespace pk {

class GgufFile;

struct Dsv4Config {
  int64_t vocab_size = 129280, dim = 4096, moe_inter_dim = 2048;
  int n_layers = 43, n_hash_layers = 3, n_mtp_layers = 1, n_heads = 64;
  int n_routed_experts = 256, n_shared_experts = 1, n_activated_experts = 6;
  std::string score_func = "sqrtsoftplus";
  double route_scale = 1.5, swiglu_limit = 10.0;
  int q_lora_rank = 1024, head_dim = 512, rope_head_dim = 64;
  double norm_eps = 1e-6;
  int o_groups = 8, o_lora_rank = 1024, window_size = 128;
  std::vector<int> compress_ratios;   // one per layer (and per MTP block); 0 = window only, 4 = overlap + indexer, 128 = plain
  double compress_rope_theta = 160000.0, rope_theta = 10000.0, rope_factor = 16.0;
  int64_t original_seq_len = 65536, max_seq_len = 1048576;
  int beta_fast = 32, beta_slow = 1;
  int index_n_heads = 64, index_head_dim = 128, index_topk = 512;
  int hc_mult = 4, hc_sinkhorn_iters = 20;
  double hc_eps = 1e-6;

  static Dsv4Config from_json(const Json& j);
  static Dsv4Config from_file(const std::string& config_json_path);
  // deepseek4 GGUF: the embedded full config when present, else the counts the file carries over the defaults.
  static Dsv4Config from_gguf(const GgufFile& f);
  Json to_json() const;
  int ratio(int layer) const { return layer < (int)compress_ratios.size() ? compress_ratios[layer] : 0; }
  // Throws std::runtime_error naming the first inconsistent field; tp_world must divide heads, groups and experts.
  void validate(int tp_world = 1) const;
};

}  // namespace pk

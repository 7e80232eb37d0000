#include "qwen_config.hpp"

#include <fstream>
#include <sstream>
#include <stdexcept>

#include "json.hpp"

namespace pk {

int QwenConfig::num_full_layers() const {
  int n = 0;
  for (int v : layer_is_full) n += v;
  return n;
}
int QwenConfig::num_linear_layers() const { return num_layers - num_full_layers(); }

void QwenConfig::validate(int tp_world) const {
  auto req = [](bool ok, const char* what) {
    if (!ok) throw std::runtime_error(std::string("qwen config: ") + what);
  };
  req(vocab_size > 0 && hidden_size > 0 && intermediate_size > 0 && num_layers > 0, "missing sizes");
  req((int)layer_is_full.size() == num_layers, "layer_types length differs from num_hidden_layers");
  req(head_dim == 128, "head_dim must be 128");
  req(linear_key_head_dim == 128 && linear_value_head_dim == 128, "linear head dims must be 128");
  req(linear_conv_kernel == 4, "linear_conv_kernel_dim must be 4");
  req(num_heads % num_kv_heads == 0, "num_attention_heads must be a multiple of num_key_value_heads");
  req(linear_value_heads % linear_key_heads == 0, "value heads must be a multiple of key heads");
  req(linear_value_heads / linear_key_heads <= 2, "at most two value heads per key head");
  req(tp_world >= 1, "tp_world");
  req(num_heads % tp_world == 0 && num_kv_heads % tp_world == 0, "attention heads must divide by tp_world");
  req(linear_key_heads % tp_world == 0 && linear_value_heads % tp_world == 0, "linear heads must divide by tp_world");
  req(intermediate_size % (128 * tp_world) == 0, "intermediate_size shard must be a multiple of 128");
  req(hidden_size % 128 == 0, "hidden_size must be a multiple of 128");
  req(vocab_size % tp_world == 0, "vocab_size must divide by tp_world");
}

QwenConfig QwenConfig::from_json(const Json& root) {
  const Json* nested = root.find("text_config");
  const Json& t = (nested && nested->is_object()) ? *nested : root;
  QwenConfig c;
  c.vocab_size = t.get_int("vocab_size", 0);
  c.hidden_size = t.get_int("hidden_size", 0);
  c.intermediate_size = t.get_int("intermediate_size", 0);
  c.num_layers = (int)t.get_int("num_hidden_layers", 0);
  c.max_position_embeddings = t.get_int("max_position_embeddings", 262144);
  c.mtp_num_hidden_layers = (int)t.get_int("mtp_num_hidden_layers", 0);
  c.rms_norm_eps = t.get_double("rms_norm_eps", 1e-6);
  c.partial_rotary_factor = t.get_double("partial_rotary_factor", 1.0);
  c.rope_theta = t.get_double("rope_theta", 1e6);
  if (const Json* rp = t.find("rope_parameters"); rp && rp->is_object()) {
    c.rope_theta = rp->get_double("rope_theta", c.rope_theta);
    c.partial_rotary_factor = rp->get_double("partial_rotary_factor", c.partial_rotary_factor);
  }
  c.linear_key_heads = (int)t.get_int("linear_num_key_heads", 0);
  c.linear_value_heads = (int)t.get_int("linear_num_value_heads", 0);
  c.linear_key_head_dim = (int)t.get_int("linear_key_head_dim", 128);
  c.linear_value_head_dim = (int)t.get_int("linear_value_head_dim", 128);
  c.linear_conv_kernel = (int)t.get_int("linear_conv_kernel_dim", 4);
  c.num_heads = (int)t.get_int("num_attention_heads", 0);
  c.num_kv_heads = (int)t.get_int("num_key_value_heads", 0);
  c.head_dim = (int)t.get_int("head_dim", c.num_heads ? c.hidden_size / c.num_heads : 128);
  c.attn_output_gate = t.get_bool("attn_output_gate", true);
  if (const Json* lt = t.find("layer_types"); lt && lt->is_array()) {
    for (const auto& v : lt->items()) {
      const std::string& s = v.as_string();
      if (s == "full_attention") c.layer_is_full.push_back(1);
      else if (s == "linear_attention") c.layer_is_full.push_back(0);
      else throw std::runtime_error("qwen config: unknown layer type " + s);
    }
  } else {
    const int interval = (int)t.get_int("full_attention_interval", 4);
    for (int i = 0; i < c.num_layers; ++i) c.layer_is_full.push_back(((i + 1) % interval) == 0 ? 1 : 0);
  }
  return c;
}

QwenConfig QwenConfig::from_file(const std::string& path) {
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << in.rdbuf();
  return from_json(Json::parse(ss.str()));
}

QwenConfig QwenConfig::benchmark_27b() {
  QwenConfig c;
  c.vocab_size = 151936;
  c.hidden_size = 5120;
  c.intermediate_size = 17408;
  c.num_layers = 64;
  for (int i = 0; i < 64; ++i) c.layer_is_full.push_back(((i + 1) % 4) == 0 ? 1 : 0);
  c.num_heads = 40;
  c.num_kv_heads = 8;
  c.head_dim = 128;
  c.rope_theta = 1.0e6;
  c.partial_rotary_factor = 0.25;
  c.linear_key_heads = 16;
  c.linear_value_heads = 32;
  return c;
}

std::string QwenConfig::to_json() const {
  Json j = Json::object();
  j["model_type"] = Json("qwen3_5_text");
  j["vocab_size"] = Json(vocab_size);
  j["hidden_size"] = Json(hidden_size);
  j["intermediate_size"] = Json(intermediate_size);
  j["num_hidden_layers"] = Json((int64_t)num_layers);
  j["max_position_embeddings"] = Json(max_position_embeddings);
  j["mtp_num_hidden_layers"] = Json((int64_t)mtp_num_hidden_layers);
  j["rms_norm_eps"] = Json(rms_norm_eps);
  j["partial_rotary_factor"] = Json(partial_rotary_factor);
  j["rope_theta"] = Json(rope_theta);
  j["linear_num_key_heads"] = Json((int64_t)linear_key_heads);
  j["linear_num_value_heads"] = Json((int64_t)linear_value_heads);
  j["linear_key_head_dim"] = Json((int64_t)linear_key_head_dim);
  j["linear_value_head_dim"] = Json((int64_t)linear_value_head_dim);
  j["linear_conv_kernel_dim"] = Json((int64_t)linear_conv_kernel);
  j["num_attention_heads"] = Json((int64_t)num_heads);
  j["num_key_value_heads"] = Json((int64_t)num_kv_heads);
  j["head_dim"] = Json((int64_t)head_dim);
  j["attn_output_gate"] = Json(attn_output_gate);
  Json lt = Json::array();
  for (int v : layer_is_full) lt.push_back(Json(v ? "full_attention" : "linear_attention"));
  j["layer_types"] = lt;
  return j.dump();
}

}  // namespace pk

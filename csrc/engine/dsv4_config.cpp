#include "dsv4_config.hpp"

#include <fstream>
#include <sstream>
#include <stdexcept>

#include "gguf_reader.hpp"

namespace pk {

namespace {
const char* kArch = "deepseek4";

std::vector<int> default_ratios(int n_layers, int n_mtp) {
  // the published schedule: two window-only layers, then ratio 4 and ratio 128 alternating; MTP blocks are window-only
  std::vector<int> r;
  for (int l = 0; l < n_layers; ++l) r.push_back(l < 2 ? 0 : ((l & 1) ? 128 : 4));
  for (int l = 0; l < n_mtp; ++l) r.push_back(0);
  return r;
}
}  // namespace

Dsv4Config Dsv4Config::from_json(const Json& j) {
  Dsv4Config c;
  c.vocab_size = j.get_int("vocab_size", c.vocab_size);
  c.dim = j.get_int("dim", j.get_int("hidden_size", c.dim));
  c.moe_inter_dim = j.get_int("moe_inter_dim", j.get_int("moe_intermediate_size", c.moe_inter_dim));
  c.n_layers = (int)j.get_int("n_layers", j.get_int("num_hidden_layers", c.n_layers));
  c.n_hash_layers = (int)j.get_int("n_hash_layers", c.n_hash_layers);
  c.n_mtp_layers = (int)j.get_int("n_mtp_layers", j.get_int("num_nextn_predict_layers", c.n_mtp_layers));
  c.n_heads = (int)j.get_int("n_heads", j.get_int("num_attention_heads", c.n_heads));
  c.n_routed_experts = (int)j.get_int("n_routed_experts", c.n_routed_experts);
  c.n_shared_experts = (int)j.get_int("n_shared_experts", c.n_shared_experts);
  c.n_activated_experts = (int)j.get_int("n_activated_experts", j.get_int("num_experts_per_tok", c.n_activated_experts));
  c.score_func = j.get_string("score_func", j.get_string("scoring_func", c.score_func));
  c.route_scale = j.get_double("route_scale", j.get_double("routed_scaling_factor", c.route_scale));
  c.swiglu_limit = j.get_double("swiglu_limit", c.swiglu_limit);
  c.q_lora_rank = (int)j.get_int("q_lora_rank", c.q_lora_rank);
  c.head_dim = (int)j.get_int("head_dim", c.head_dim);
  c.rope_head_dim = (int)j.get_int("rope_head_dim", j.get_int("qk_rope_head_dim", c.rope_head_dim));
  c.norm_eps = j.get_double("norm_eps", j.get_double("rms_norm_eps", c.norm_eps));
  c.o_groups = (int)j.get_int("o_groups", c.o_groups);
  c.o_lora_rank = (int)j.get_int("o_lora_rank", c.o_lora_rank);
  c.window_size = (int)j.get_int("window_size", j.get_int("sliding_window", c.window_size));
  c.compress_rope_theta = j.get_double("compress_rope_theta", c.compress_rope_theta);
  c.rope_theta = j.get_double("rope_theta", c.rope_theta);
  c.rope_factor = j.get_double("rope_factor", c.rope_factor);
  c.original_seq_len = j.get_int("original_seq_len", c.original_seq_len);
  c.max_seq_len = j.get_int("max_seq_len", j.get_int("max_position_embeddings", c.max_seq_len));
  c.beta_fast = (int)j.get_int("beta_fast", c.beta_fast);
  c.beta_slow = (int)j.get_int("beta_slow", c.beta_slow);
  c.index_n_heads = (int)j.get_int("index_n_heads", c.index_n_heads);
  c.index_head_dim = (int)j.get_int("index_head_dim", c.index_head_dim);
  c.index_topk = (int)j.get_int("index_topk", c.index_topk);
  c.hc_mult = (int)j.get_int("hc_mult", c.hc_mult);
  c.hc_sinkhorn_iters = (int)j.get_int("hc_sinkhorn_iters", c.hc_sinkhorn_iters);
  c.hc_eps = j.get_double("hc_eps", c.hc_eps);
  if (const Json* r = j.find("compress_ratios")) {
    for (const Json& v : r->items()) c.compress_ratios.push_back((int)v.as_int());
  } else {
    c.compress_ratios = default_ratios(c.n_layers, c.n_mtp_layers);
  }
  return c;
}

Dsv4Config Dsv4Config::from_file(const std::string& path) {
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << in.rdbuf();
  return from_json(Json::parse(ss.str()));
}

Dsv4Config Dsv4Config::from_gguf(const GgufFile& f) {
  const Json& md = f.metadata();
  if (f.architecture() != kArch) throw std::runtime_error("not a deepseek4 GGUF: architecture '" + f.architecture() + "'");
  const std::string a = kArch;
  const std::string embedded = md.get_string(a + ".pocket_config", "");
  if (!embedded.empty()) return from_json(Json::parse(embedded));
  Dsv4Config c;
  c.n_layers = (int)md.get_int(a + ".block_count", c.n_layers);
  c.n_hash_layers = (int)md.get_int(a + ".hash_layer_count", c.n_hash_layers);
  c.n_routed_experts = (int)md.get_int(a + ".expert_count", c.n_routed_experts);
  c.n_activated_experts = (int)md.get_int(a + ".expert_used_count", c.n_activated_experts);
  c.dim = md.get_int(a + ".embedding_length", c.dim);
  c.vocab_size = md.get_int(a + ".vocab_size", c.vocab_size);
  c.max_seq_len = md.get_int(a + ".context_length", c.max_seq_len);
  c.n_mtp_layers = 0;   // GGUF files carry no MTP blocks
  c.compress_ratios = default_ratios(c.n_layers, 0);
  return c;
}

Json Dsv4Config::to_json() const {
  Json j = Json::object();
  j["vocab_size"] = Json(vocab_size);
  j["dim"] = Json(dim);
  j["moe_inter_dim"] = Json(moe_inter_dim);
  j["n_layers"] = Json(n_layers);
  j["n_hash_layers"] = Json(n_hash_layers);
  j["n_mtp_layers"] = Json(n_mtp_layers);
  j["n_heads"] = Json(n_heads);
  j["n_routed_experts"] = Json(n_routed_experts);
  j["n_shared_experts"] = Json(n_shared_experts);
  j["n_activated_experts"] = Json(n_activated_experts);
  j["score_func"] = Json(score_func);
  j["route_scale"] = Json(route_scale);
  j["swiglu_limit"] = Json(swiglu_limit);
  j["q_lora_rank"] = Json(q_lora_rank);
  j["head_dim"] = Json(head_dim);
  j["rope_head_dim"] = Json(rope_head_dim);
  j["norm_eps"] = Json(norm_eps);
  j["o_groups"] = Json(o_groups);
  j["o_lora_rank"] = Json(o_lora_rank);
  j["window_size"] = Json(window_size);
  Json r = Json::array();
  for (int v : compress_ratios) r.push_back(Json(v));
  j["compress_ratios"] = r;
  j["compress_rope_theta"] = Json(compress_rope_theta);
  j["original_seq_len"] = Json(original_seq_len);
  j["rope_theta"] = Json(rope_theta);
  j["rope_factor"] = Json(rope_factor);
  j["beta_fast"] = Json(beta_fast);
  j["beta_slow"] = Json(beta_slow);
  j["index_n_heads"] = Json(index_n_heads);
  j["index_head_dim"] = Json(index_head_dim);
  j["index_topk"] = Json(index_topk);
  j["hc_mult"] = Json(hc_mult);
  j["hc_sinkhorn_iters"] = Json(hc_sinkhorn_iters);
  j["hc_eps"] = Json(hc_eps);
  j["max_seq_len"] = Json(max_seq_len);
  return j;
}

void Dsv4Config::validate(int tp_world) const {
  auto fail = [](const std::string& what) { throw std::runtime_error("DSV4 config: " + what); };
  if (dim <= 0 || n_layers <= 0 || n_heads <= 0 || head_dim <= 0 || vocab_size <= 0) fail("sizes must be positive");
  if (rope_head_dim <= 0 || rope_head_dim > head_dim || (rope_head_dim & 1)) fail("rope_head_dim must be even and at most head_dim");
  if ((head_dim - rope_head_dim) % 64 != 0) fail("head_dim - rope_head_dim must be a multiple of 64 (FP8 activation blocks)");
  if (n_hash_layers < 0 || n_hash_layers > n_layers) fail("n_hash_layers out of range");
  if (n_activated_experts <= 0 || n_activated_experts > n_routed_experts) fail("n_activated_experts out of range");
  if (o_groups <= 0 || n_heads % o_groups != 0) fail("o_groups must divide n_heads");
  if ((int)compress_ratios.size() < n_layers) fail("compress_ratios needs one entry per layer");
  for (int l = 0; l < n_layers; ++l) {
    const int r = compress_ratios[l];
    if (r != 0 && (r < 2 || (window_size % r != 0 && r % window_size != 0))) fail("compress ratio of layer " + std::to_string(l) + " does not fit the window");
  }
  if (score_func != "sqrtsoftplus" && score_func != "sigmoid" && score_func != "softmax") fail("unknown score_func " + score_func);
  if (tp_world < 1) fail("tp_world must be positive");
  if (n_heads % tp_world || o_groups % tp_world || n_routed_experts % tp_world)
    fail("tp_world " + std::to_string(tp_world) + " must divide heads, output groups and routed experts");
}

}  // namespace pk

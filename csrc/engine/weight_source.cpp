#include "weight_source.hpp"

#include <stdexcept>

namespace pk {

namespace {

// model suffix (after "layers.<l>.") <-> GGUF suffix (after "blk.<l>.")
const std::pair<const char*, const char*> kLayerNames[] = {
    {"attn.attn_sink", "attn_sinks.weight"},
    {"attn.wq_a.weight", "attn_q_a.weight"},
    {"attn.q_norm.weight", "attn_q_a_norm.weight"},
    {"attn.wq_b.weight", "attn_q_b.weight"},
    {"attn.wkv.weight", "attn_kv.weight"},
    {"attn.kv_norm.weight", "attn_kv_a_norm.weight"},
    {"attn.wo_a.weight", "attn_output_a.weight"},
    {"attn.wo_b.weight", "attn_output_b.weight"},
    {"attn_norm.weight", "attn_norm.weight"},
    {"ffn.gate.weight", "ffn_gate_inp.weight"},
    {"ffn.gate.tid2eid", "ffn_gate_tid2eid.weight"},
    {"ffn.gate.bias", "exp_probs_b.bias"},
    {"ffn.shared_experts.w1.weight", "ffn_gate_shexp.weight"},
    {"ffn.shared_experts.w2.weight", "ffn_down_shexp.weight"},
    {"ffn.shared_experts.w3.weight", "ffn_up_shexp.weight"},
    {"ffn_norm.weight", "ffn_norm.weight"},
    {"hc_attn_fn", "hc_attn_fn.weight"},
    {"hc_attn_base", "hc_attn_base.weight"},
    {"hc_attn_scale", "hc_attn_scale.weight"},
    {"hc_ffn_fn", "hc_ffn_fn.weight"},
    {"hc_ffn_base", "hc_ffn_base.weight"},
    {"hc_ffn_scale", "hc_ffn_scale.weight"},
    {"attn.compressor.ape", "attn_compressor_ape.weight"},
    {"attn.compressor.wkv.weight", "attn_compressor_kv.weight"},
    {"attn.compressor.wgate.weight", "attn_compressor_gate.weight"},
    {"attn.compressor.norm.weight", "attn_compressor_norm.weight"},
    {"attn.indexer.wq_b.weight", "indexer.attn_q_b.weight"},
    {"attn.indexer.weights_proj.weight", "indexer.proj.weight"},
    {"attn.indexer.compressor.ape", "indexer_compressor_ape.weight"},
    {"attn.indexer.compressor.wkv.weight", "indexer_compressor_kv.weight"},
    {"attn.indexer.compressor.wgate.weight", "indexer_compressor_gate.weight"},
    {"attn.indexer.compressor.norm.weight", "indexer_compressor_norm.weight"},
};
const std::pair<const char*, const char*> kTopNames[] = {
    {"embed.weight", "token_embd.weight"}, {"head.weight", "output.weight"},       {"norm.weight", "output_norm.weight"},
    {"hc_head_fn", "output_hc_fn.weight"}, {"hc_head_base", "output_hc_base.weight"}, {"hc_head_scale", "output_hc_scale.weight"},
};

const char* expert_tensor(const std::string& part) {
  if (part == "w1") return "ffn_gate_exps.weight";
  if (part == "w3") return "ffn_up_exps.weight";
  if (part == "w2") return "ffn_down_exps.weight";
  throw std::runtime_error("expert part must be w1, w2 or w3, got '" + part + "'");
}

}  // namespace

TensorView WeightSource::require(const std::string& name) const {
  TensorView v = get(name);
  if (!v.found) throw std::runtime_error("missing tensor: " + name);
  return v;
}

// ---- Safetensors ----

SafetensorsSource::SafetensorsSource(const std::string& path) : model_(path) {}

TensorView SafetensorsSource::get(const std::string& name) const {
  TensorView v;
  v.name = name;
  const StTensor* t = model_.find(name);
  if (t == nullptr) return v;
  v.stored_name = t->name;
  v.dtype = st_dtype_name(t->dtype);
  v.shape = t->shape;
  v.data = t->data;
  v.nbytes = t->nbytes;
  v.found = true;
  return v;
}

TensorView SafetensorsSource::expert(int layer, int e, const std::string& part) const {
  (void)expert_tensor(part);   // validates the part name
  return get("layers." + std::to_string(layer) + ".ffn.experts." + std::to_string(e) + "." + part + ".weight");
}

// ---- GGUF ----

GgufSource::GgufSource(const std::string& path) : file_(path), cfg_(Dsv4Config::from_gguf(file_)) {}

std::string GgufSource::stored_name_for(const std::string& name) {
  for (const auto& p : kTopNames)
    if (name == p.first) return p.second;
  if (name.rfind("layers.", 0) != 0) return "";
  const size_t dot = name.find('.', 7);
  if (dot == std::string::npos) return "";
  const std::string layer = name.substr(7, dot - 7), suffix = name.substr(dot + 1);
  if (layer.empty() || layer.find_first_not_of("0123456789") != std::string::npos) return "";
  for (const auto& p : kLayerNames)
    if (suffix == p.first) return "blk." + layer + "." + p.second;
  return "";
}

TensorView GgufSource::view_of(const GgufTensor& t, const std::string& asked) const {
  TensorView v;
  v.name = asked;
  v.stored_name = t.name;
  v.dtype = ggml_type_name(t.type);
  v.shape.assign(t.dims.rbegin(), t.dims.rend());   // GGUF lists the innermost dimension first
  v.data = file_.data(t);
  v.nbytes = t.nbytes;
  v.found = true;
  return v;
}

bool GgufSource::has(const std::string& name) const {
  const std::string s = stored_name_for(name);
  return !s.empty() && file_.find(s) != nullptr;
}

TensorView GgufSource::get(const std::string& name) const {
  TensorView v;
  v.name = name;
  const std::string s = stored_name_for(name);
  if (s.empty()) return v;
  const GgufTensor* t = file_.find(s);
  return t ? view_of(*t, name) : v;
}

TensorView GgufSource::expert(int layer, int e, const std::string& part) const {
  const std::string asked = "layers." + std::to_string(layer) + ".ffn.experts." + std::to_string(e) + "." + part + ".weight";
  TensorView v;
  v.name = asked;
  const GgufTensor* t = file_.find("blk." + std::to_string(layer) + "." + expert_tensor(part));
  if (t == nullptr) return v;
  if (t->dims.size() != 3) throw std::runtime_error("packed expert tensor " + t->name + " is not 3-d");
  const uint64_t n_experts = t->dims[2];
  if (e < 0 || (uint64_t)e >= n_experts) throw std::runtime_error("expert " + std::to_string(e) + " out of range in " + t->name);
  if (t->nbytes % n_experts != 0) throw std::runtime_error("packed expert tensor " + t->name + " does not split evenly");
  v = view_of(*t, asked);
  v.shape = {(int64_t)t->dims[1], (int64_t)t->dims[0]};   // [rows, columns] of one expert
  v.nbytes = t->nbytes / n_experts;
  v.data += v.nbytes * (uint64_t)e;
  return v;
}

std::vector<std::string> GgufSource::names() const {
  std::vector<std::string> out;
  for (const auto& p : kTopNames)
    if (file_.find(p.second) != nullptr) out.push_back(p.first);
  for (int l = 0; l < cfg_.n_layers; ++l)
    for (const auto& p : kLayerNames)
      if (file_.find("blk." + std::to_string(l) + "." + p.second) != nullptr) out.push_back("layers." + std::to_string(l) + "." + p.first);
  return out;
}

bool is_gguf_path(const std::string& path) {
  return path.size() >= 5 && path.compare(path.size() - 5, 5, ".gguf") == 0;
}

std::unique_ptr<WeightSource> open_weight_source(const std::string& path) {
  if (is_gguf_path(path)) return std::make_unique<GgufSource>(path);
  return std::make_unique<SafetensorsSource>(path);
}

}  // namespace pk

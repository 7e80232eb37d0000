#include "qwen_audit.hpp"

#include <set>

namespace pk {

namespace {

std::string shape_text(const std::vector<int64_t>& s) {
  std::string t = "[";
  for (size_t i = 0; i < s.size(); ++i) t += (i ? "," : "") + std::to_string(s[i]);
  return t + "]";
}

struct Auditor {
  const SafetensorsModel& st;
  QwenAuditReport& rep;
  std::set<std::string> seen;

  const StTensor* want(const std::string& name, const std::vector<int64_t>& shape, std::initializer_list<StDtype> dtypes) {
    ++rep.expected;
    seen.insert(name);
    const StTensor* t = st.find(name);
    if (t == nullptr) {
      rep.problems.push_back("missing " + name);
      return nullptr;
    }
    rep.expected_bytes += t->nbytes;
    bool dtype_ok = false;
    for (StDtype d : dtypes) dtype_ok = dtype_ok || t->dtype == d;
    if (!dtype_ok) rep.problems.push_back(std::string("dtype ") + name + " is " + st_dtype_name(t->dtype));
    if (t->shape != shape) rep.problems.push_back("shape " + name + " is " + shape_text(t->shape) + ", expected " + shape_text(shape));
    return t;
  }

  // An FP8 linear [N, K] with its [ceil(N / 128), ceil(K / 128)] scales. `row_cut` / `col_cut`: size of one rank's share
  // along that axis when the axis is split (0 = not split): it must be a multiple of the scale block.
  void fp8_linear(const std::string& name, int64_t N, int64_t K, int64_t row_cut, int64_t col_cut) {
    ++rep.fp8_linears;
    want(name + ".weight", {N, K}, {StDtype::F8_E4M3});
    want(name + ".weight_scale_inv", {(N + 127) / 128, (K + 127) / 128}, {StDtype::F32, StDtype::BF16});
    if (row_cut > 0 && (row_cut % 128) != 0)
      rep.problems.push_back("shard " + name + ": " + std::to_string(row_cut) + " rows per rank do not fall on the 128-row scale blocks");
    if (col_cut > 0 && (col_cut % 128) != 0)
      rep.problems.push_back("shard " + name + ": " + std::to_string(col_cut) + " columns per rank do not fall on the 128-column scale blocks");
  }
};

}  // namespace

QwenAuditReport audit_qwen_checkpoint(const SafetensorsModel& st, const QwenConfig& cfg, int tp_world, bool want_mtp) {
  QwenAuditReport rep;
  Auditor a{st, rep, {}};
  const int W = tp_world < 1 ? 1 : tp_world;
  const int64_t H = cfg.hidden_size, I = cfg.intermediate_size, D = cfg.head_dim;
  const int64_t qrows = (int64_t)cfg.num_heads * D * (cfg.attn_output_gate ? 2 : 1), kvrows = (int64_t)cfg.num_kv_heads * D;
  const int64_t KD = (int64_t)cfg.linear_key_heads * cfg.linear_key_head_dim, VD = (int64_t)cfg.linear_value_heads * cfg.linear_value_head_dim;
  const bool split = W > 1;
  std::string root = "model.language_model.";
  if (!st.has(root + "embed_tokens.weight")) root = "model.";

  auto layer = [&](const std::string& p, bool full) {
    a.want(p + "input_layernorm.weight", {H}, {StDtype::BF16, StDtype::F32});
    a.want(p + "post_attention_layernorm.weight", {H}, {StDtype::BF16, StDtype::F32});
    if (full) {
      a.fp8_linear(p + "self_attn.q_proj", qrows, H, split ? qrows / W : 0, 0);
      a.fp8_linear(p + "self_attn.k_proj", kvrows, H, split ? kvrows / W : 0, 0);
      a.fp8_linear(p + "self_attn.v_proj", kvrows, H, split ? kvrows / W : 0, 0);
      a.fp8_linear(p + "self_attn.o_proj", H, (int64_t)cfg.num_heads * D, 0, split ? (int64_t)cfg.num_heads * D / W : 0);
      a.want(p + "self_attn.q_norm.weight", {D}, {StDtype::BF16, StDtype::F32});
      a.want(p + "self_attn.k_norm.weight", {D}, {StDtype::BF16, StDtype::F32});
    } else {
      // q | k | v rows of in_proj_qkv are cut separately: each part's share must sit on the scale blocks
      a.fp8_linear(p + "linear_attn.in_proj_qkv", 2 * KD + VD, H, split ? KD / W : 0, 0);
      if (split && ((VD / W) % 128) != 0)
        rep.problems.push_back("shard " + p + "linear_attn.in_proj_qkv: " + std::to_string(VD / W) + " value rows per rank do not fall on the 128-row scale blocks");
      a.fp8_linear(p + "linear_attn.in_proj_z", VD, H, split ? VD / W : 0, 0);
      a.fp8_linear(p + "linear_attn.out_proj", H, VD, 0, split ? VD / W : 0);
      a.want(p + "linear_attn.in_proj_a.weight", {(int64_t)cfg.linear_value_heads, H}, {StDtype::BF16});
      a.want(p + "linear_attn.in_proj_b.weight", {(int64_t)cfg.linear_value_heads, H}, {StDtype::BF16});
      const StTensor* cw = st.find(p + "linear_attn.conv1d.weight");
      ++rep.expected;
      a.seen.insert(p + "linear_attn.conv1d.weight");
      if (cw == nullptr) rep.problems.push_back("missing " + p + "linear_attn.conv1d.weight");
      else {
        rep.expected_bytes += cw->nbytes;
        if (cw->numel() != (2 * KD + VD) * cfg.linear_conv_kernel)
          rep.problems.push_back("shape " + p + "linear_attn.conv1d.weight is " + shape_text(cw->shape) + ", expected " +
                                 std::to_string(2 * KD + VD) + " channels of " + std::to_string(cfg.linear_conv_kernel) + " taps");
      }
      a.want(p + "linear_attn.A_log", {(int64_t)cfg.linear_value_heads}, {StDtype::BF16, StDtype::F32});
      a.want(p + "linear_attn.dt_bias", {(int64_t)cfg.linear_value_heads}, {StDtype::BF16, StDtype::F32});
      a.want(p + "linear_attn.norm.weight", {(int64_t)cfg.linear_value_head_dim}, {StDtype::BF16, StDtype::F32});
    }
    a.fp8_linear(p + "mlp.gate_proj", I, H, split ? I / W : 0, 0);
    a.fp8_linear(p + "mlp.up_proj", I, H, split ? I / W : 0, 0);
    a.fp8_linear(p + "mlp.down_proj", H, I, 0, split ? I / W : 0);
  };

  a.want(root + "embed_tokens.weight", {cfg.vocab_size, H}, {StDtype::BF16});
  a.want(root + "norm.weight", {H}, {StDtype::BF16, StDtype::F32});
  a.want("lm_head.weight", {cfg.vocab_size, H}, {StDtype::BF16});
  if (split && (cfg.vocab_size % W) != 0) rep.problems.push_back("shard lm_head.weight: the vocabulary does not divide by the ranks");
  for (int i = 0; i < cfg.num_layers; ++i)
    layer(root + "layers." + std::to_string(i) + ".", i < (int)cfg.layer_is_full.size() && cfg.layer_is_full[i] != 0);
  if (want_mtp) {
    a.want("mtp.fc.weight", {H, 2 * H}, {StDtype::BF16});
    a.want("mtp.pre_fc_norm_embedding.weight", {H}, {StDtype::BF16, StDtype::F32});
    a.want("mtp.pre_fc_norm_hidden.weight", {H}, {StDtype::BF16, StDtype::F32});
    a.want("mtp.norm.weight", {H}, {StDtype::BF16, StDtype::F32});
    layer("mtp.layers.0.", true);
  }
  for (const std::string& n : st.names())
    if (a.seen.count(n) == 0) rep.unused.push_back(n);
  return rep;
}

}  // namespace pk

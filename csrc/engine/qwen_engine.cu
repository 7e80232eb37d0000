#include "qwen_engine.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "mem_guard.hpp"
#include "prefix_plan.hpp"
#include "pk_kernels.h"
#include "safetensors.hpp"
#include "spec_policy.hpp"

namespace pk {

namespace {

constexpr int kHeadDim = 128;
constexpr int kSmallRows = 8;
constexpr int kArgmaxBlocks = 64;
constexpr int kCandStride = 32;   // sampler candidates per rank in the exchange arrays; entry 31 of the index row is the rank's status word

void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

float bf16_to_f32(uint16_t b) {
  uint32_t u = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// ---- host-side shard cutting ----
struct HostMat {
  std::vector<uint8_t> data;
  int rows = 0, cols = 0, elem = 1;
};

HostMat cut(const StTensor& t, int elem, int64_t r0, int64_t nr, int64_t c0, int64_t nc) {
  if (t.shape.size() < 1) throw std::runtime_error("tensor rank: " + t.name);
  const int64_t R = t.shape[0];
  int64_t C = 1;
  for (size_t i = 1; i < t.shape.size(); ++i) C *= t.shape[i];
  if (r0 < 0 || r0 + nr > R || c0 < 0 || c0 + nc > C) throw std::runtime_error("shard out of range: " + t.name);
  if ((size_t)(R * C * elem) != t.nbytes) throw std::runtime_error("dtype size mismatch: " + t.name);
  HostMat m;
  m.rows = (int)nr;
  m.cols = (int)nc;
  m.elem = elem;
  m.data.resize((size_t)nr * nc * elem);
  for (int64_t r = 0; r < nr; ++r)
    memcpy(m.data.data() + (size_t)r * nc * elem, t.data + ((size_t)(r0 + r) * C + c0) * elem, (size_t)nc * elem);
  return m;
}

void append_rows(HostMat& dst, const HostMat& src) {
  if (dst.data.empty()) {
    dst = src;
    return;
  }
  if (dst.cols != src.cols || dst.elem != src.elem) throw std::runtime_error("append_rows: shape mismatch");
  dst.data.insert(dst.data.end(), src.data.begin(), src.data.end());
  dst.rows += src.rows;
}

std::vector<float> bf16_vec_to_f32(const HostMat& m) {
  std::vector<float> out((size_t)m.rows * m.cols);
  const uint16_t* p = (const uint16_t*)m.data.data();
  for (size_t i = 0; i < out.size(); ++i) out[i] = bf16_to_f32(p[i]);
  return out;
}

// fp32 -> E4M3 (round to nearest even, saturating at 448)
uint8_t f32_to_e4m3(float f) {
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a != a) return sign | 0x7f;
  if (a > 448.f) a = 448.f;
  int e = 0;
  (void)std::frexp(a, &e);
  const int E = e - 1;   // a = 1.m * 2^E
  if (a == 0.f || E < -6) return sign | (uint8_t)std::rint(std::ldexp(a, 9));   // zero and subnormals: multiples of 2^-9
  int mant = (int)std::rint((std::ldexp(a, -E) - 1.f) * 8.f), ex = E;
  if (mant == 8) {
    mant = 0;
    ++ex;
  }
  const int code = ((ex + 7) << 3) | mant;
  return sign | (uint8_t)std::min(code, 0x7e);
}

// bf16 [rows, cols] -> E4M3 codes and one fp32 scale per 128 x 128 block (absmax / 448)
void quantize_block128(const HostMat& m, std::vector<uint8_t>& codes, std::vector<float>& scales) {
  const uint16_t* src = (const uint16_t*)m.data.data();
  const int R = m.rows, C = m.cols, rb = (R + 127) / 128, cb = (C + 127) / 128;
  codes.resize((size_t)R * C);
  scales.assign((size_t)rb * cb, 1.f);
  for (int br = 0; br < rb; ++br)
    for (int bc = 0; bc < cb; ++bc) {
      float amax = 0.f;
      const int r1 = std::min(R, br * 128 + 128), c1 = std::min(C, bc * 128 + 128);
      for (int r = br * 128; r < r1; ++r)
        for (int c = bc * 128; c < c1; ++c) amax = std::max(amax, std::fabs(bf16_to_f32(src[(size_t)r * C + c])));
      const float sc = amax > 0.f ? amax / 448.f : 1.f;
      scales[(size_t)br * cb + bc] = sc;
      for (int r = br * 128; r < r1; ++r)
        for (int c = bc * 128; c < c1; ++c) codes[(size_t)r * C + c] = f32_to_e4m3(bf16_to_f32(src[(size_t)r * C + c]) / sc);
    }
}

}  // namespace

void QwenEngine::check(int status, const char* what) const {
  if (status != 0) {
    char buf[160];
    snprintf(buf, sizeof buf, "%s failed: status %d (cuda error %d)", what, status, pk_last_cuda_error());
    throw std::runtime_error(buf);
  }
  ++launches_;
}

void* QwenEngine::dalloc(size_t bytes, bool weight) {
  void* p = nullptr;
  if (bytes >= (size_t(64) << 20)) require_headroom(bytes, weight ? "engine weights" : "engine buffers");
  if (canaries_) {
    // guard words on both sides of every buffer (POCKET_CANARY=1): verify_canaries() tells which one was written across
    const size_t body = (std::max<size_t>(bytes, 16) + 255) / 256 * 256;
    cuda_check(cudaMalloc(&p, body + 2 * kCanaryBytes), "cudaMalloc");
    cuda_check(cudaMemset(p, kCanaryByte, kCanaryBytes), "canary");
    cuda_check(cudaMemset((char*)p + kCanaryBytes + body, kCanaryByte, kCanaryBytes), "canary");
    allocs_.push_back(p);
    guarded_.push_back({(char*)p, body, bytes});
    p = (char*)p + kCanaryBytes;
  } else {
    cuda_check(cudaMalloc(&p, std::max<size_t>(bytes, 16)), "cudaMalloc");
    allocs_.push_back(p);
  }
  if (weight) weight_bytes_ += bytes;
  alloc_bytes_ += bytes;
  return p;
}

// Index of the first buffer (in allocation order) whose guard words were overwritten, or -1. Synchronises the device.
int QwenEngine::verify_canaries(std::string* what) {
  if (!canaries_) return -1;
  cuda_check(cudaDeviceSynchronize(), "sync");
  std::vector<uint8_t> host(2 * kCanaryBytes);
  for (size_t i = 0; i < guarded_.size(); ++i) {
    const Guarded& g = guarded_[i];
    cuda_check(cudaMemcpy(host.data(), g.base, kCanaryBytes, cudaMemcpyDeviceToHost), "canary read");
    cuda_check(cudaMemcpy(host.data() + kCanaryBytes, g.base + kCanaryBytes + g.body, kCanaryBytes, cudaMemcpyDeviceToHost), "canary read");
    for (size_t b = 0; b < host.size(); ++b)
      if (host[b] != kCanaryByte) {
        if (what) {
          char buf[160];
          snprintf(buf, sizeof buf, "buffer %zu (%zu bytes): guard byte %zu %s the buffer was overwritten", i, g.bytes,
                   b < kCanaryBytes ? kCanaryBytes - b : b - kCanaryBytes, b < kCanaryBytes ? "before" : "behind");
          *what = buf;
        }
        return (int)i;
      }
  }
  return -1;
}

void QwenEngine::alloc_fp8(Fp8Linear& l, int N, int K) {
  l.N = N;
  l.K = K;
  l.w = (uint8_t*)dalloc((size_t)N * K, true);
  l.scale = (float*)dalloc((size_t)((N + 127) / 128) * ((K + 127) / 128) * sizeof(float), true);
}

QwenEngine::QwenEngine(const QwenConfig& cfg, const QwenEngineOptions& opt) : cfg_(cfg), opt_(opt) {
  if (const char* cv = getenv("POCKET_CANARY")) canaries_ = cv[0] != '\0' && cv[0] != '0';
  cfg_.validate(opt.tp_world);
  if (opt.tp_world > PK_MAX_RANKS) throw std::runtime_error("tp_world > 8");
  cuda_check(cudaSetDevice(opt.device), "cudaSetDevice");
  cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream");
  cudaDeviceProp prop;
  cuda_check(cudaGetDeviceProperties(&prop, opt.device), "props");
  sm_count_ = prop.multiProcessorCount;
  cuda_check(cudaEventCreate(&ev0_), "event");
  cuda_check(cudaEventCreate(&ev1_), "event");

  const int W = opt.tp_world;
  hidden_ = (int)cfg_.hidden_size;
  inter_l_ = (int)cfg_.intermediate_size / W;
  vocab_l_ = (int)cfg_.vocab_size / W;
  vocab_start_ = vocab_l_ * opt.tp_rank;
  hq_l_ = cfg_.num_heads / W;
  hkv_l_ = cfg_.num_kv_heads / W;
  kh_l_ = cfg_.linear_key_heads / W;
  vh_l_ = cfg_.linear_value_heads / W;
  kd_l_ = kh_l_ * kHeadDim;
  vd_l_ = vh_l_ * kHeadDim;
  conv_c_l_ = 2 * kd_l_ + vd_l_;
  ld_lin_ = (int)align_up(2 * kd_l_ + 2 * vd_l_ + 2 * vh_l_, 8);
  ld_full_ = hq_l_ * 2 * kHeadDim + 2 * hkv_l_ * kHeadDim;
  ld_proj_ = std::max(ld_lin_, ld_full_);
  rows_cap_ = std::max(opt.prefill_chunk, kSmallRows);
  {
    const char* v = getenv("POCKET_PREFILL_ATTN");   // "simt" keeps the split-context kernel for prefill chunks
    tc_prefill_attn_ = !opt.kv_fp8 && opt.attention_window == 0 && !(v != nullptr && std::string(v) == "simt");
  }
  sites_per_epoch_ = 2 * cfg_.num_layers + 1;

  // ---- weights ----
  layers_.resize(cfg_.num_layers);
  for (int i = 0; i < cfg_.num_layers; ++i) alloc_layer(layers_[i], cfg_.layer_is_full[i] != 0);
  embed_ = dalloc((size_t)cfg_.vocab_size * hidden_ * 2, true);
  final_norm_ = (float*)dalloc(hidden_ * sizeof(float), true);
  lm_head_ = dalloc((size_t)vocab_l_ * hidden_ * 2, true);
  if (opt_.mtp) {
    alloc_layer(mtp_layer_, true);
    mtp_norm_e_ = (float*)dalloc(hidden_ * sizeof(float), true);
    mtp_norm_h_ = (float*)dalloc(hidden_ * sizeof(float), true);
    mtp_norm_ = (float*)dalloc(hidden_ * sizeof(float), true);
    mtp_fc_ = dalloc((size_t)hidden_ * 2 * hidden_ * 2, true);
  }
  log_device_memory("weights_allocated", alloc_bytes_);
  alloc_buffers();
  log_device_memory("buffers_allocated", alloc_bytes_);
  reset();
}

void QwenEngine::alloc_layer(QwenLayer& L, bool full) {
  const QwenEngineOptions& opt = opt_;
  {
    L.full = full;
    L.input_norm = (float*)dalloc(hidden_ * sizeof(float), true);
    L.post_norm = (float*)dalloc(hidden_ * sizeof(float), true);
    if (L.full) {
      alloc_fp8(L.qkv, ld_full_, hidden_);
      alloc_fp8(L.o_proj, hidden_, hq_l_ * kHeadDim);
      L.q_norm = (float*)dalloc(kHeadDim * sizeof(float), true);
      L.k_norm = (float*)dalloc(kHeadDim * sizeof(float), true);
      const size_t kv = (size_t)hkv_l_ * opt.max_context * kHeadDim * (opt.kv_fp8 ? 1 : 2);
      L.kcache = dalloc(kv);
      L.vcache = dalloc(kv);
      // finite from the start: the tensor-core prefill attention reads (and masks) rows behind the last position
      cuda_check(cudaMemset(L.kcache, 0, kv), "memset");
      cuda_check(cudaMemset(L.vcache, 0, kv), "memset");
      kv_bytes_ += 2 * kv;
      if (opt.kv_fp8) {
        const size_t sc = (size_t)hkv_l_ * opt.max_context * 2 * sizeof(float);
        L.kscale = (float*)dalloc(sc);
        L.vscale = (float*)dalloc(sc);
        kv_bytes_ += 2 * sc;
      }
    } else {
      alloc_fp8(L.in_proj, 2 * kd_l_ + 2 * vd_l_, hidden_);
      L.in_proj_ab = dalloc((size_t)2 * vh_l_ * hidden_ * 2, true);
      L.conv_w = (float*)dalloc((size_t)conv_c_l_ * 4 * sizeof(float), true);
      L.A_log = (float*)dalloc(vh_l_ * sizeof(float), true);
      L.dt_bias = (float*)dalloc(vh_l_ * sizeof(float), true);
      L.lin_norm = (float*)dalloc(kHeadDim * sizeof(float), true);
      alloc_fp8(L.out_proj, hidden_, vd_l_);
      L.lin_state = (float*)dalloc((size_t)vh_l_ * kHeadDim * kHeadDim * sizeof(float));
      L.conv_state = (float*)dalloc((size_t)conv_c_l_ * 3 * sizeof(float));
    }
    alloc_fp8(L.gate_up, 2 * inter_l_, hidden_);
    alloc_fp8(L.down, hidden_, inter_l_);
  }
}

void QwenEngine::alloc_buffers() {
  const size_t R = rows_cap_;
  for (int i = 0; i < 2; ++i) hidden_buf_[i] = dalloc(R * hidden_ * 2);
  xn_ = opt_.tp_world > 1 ? nullptr : dalloc(R * hidden_ * 2);   // several ranks: inside the comm arena (set below)
  proj_ = dalloc(R * ld_proj_ * 2);
  const int attn_w = std::max(vd_l_, hq_l_ * kHeadDim);
  attn_out_ = dalloc(R * attn_w * 2);
  q_buf_ = dalloc(R * hq_l_ * kHeadDim * 2);
  mlp_h_ = dalloc(R * inter_l_ * 2);
  const size_t ws_small = (size_t)kSmallRows * hq_l_ * opt_.decode_splits * (kHeadDim + 2);
  const size_t ws_big = R * hq_l_ * 1 * (kHeadDim + 2);
  attn_ws_ = (float*)dalloc(std::max(ws_small, ws_big) * sizeof(float));
  lin_ws_ = (float*)dalloc(pk_deltanet_chunk_workspace(rows_cap_, kh_l_, vh_l_) * sizeof(float));
  logits_ = (float*)dalloc((size_t)kSmallRows * vocab_l_ * sizeof(float));
  cand_val_ = (float*)dalloc(kSmallRows * kArgmaxBlocks * sizeof(float));
  cand_idx_ = (int*)dalloc(kSmallRows * kArgmaxBlocks * sizeof(int));
  best_val_ = (float*)dalloc(kSmallRows * sizeof(float));
  best_idx_ = (int*)dalloc(kSmallRows * sizeof(int));
  tokens_dev_ = (int*)dalloc(R * sizeof(int));
  pos_dev_ = (int*)dalloc(R * sizeof(int));
  next_tok_dev_ = (int*)dalloc(kSmallRows * sizeof(int));
  out_cap_ = 1 << 16;
  out_tokens_dev_ = (int*)dalloc(out_cap_ * sizeof(int));
  out_counter_dev_ = (int*)dalloc(sizeof(int));
  gemm_status_ = (uint32_t*)dalloc(sizeof(uint32_t));
  cuda_check(cudaMemset(gemm_status_, 0, sizeof(uint32_t)), "memset");
  if (opt_.mtp) {
    mtp_cat_ = dalloc(R * 2 * hidden_ * 2);
    tgt_hid_ = dalloc(R * hidden_ * 2);
    mtp_out_ = dalloc((size_t)kSmallRows * hidden_ * 2);
    cuda_check(cudaMemset(tgt_hid_, 0, R * hidden_ * 2), "memset");
    cuda_check(cudaMemset(mtp_out_, 0, (size_t)kSmallRows * hidden_ * 2), "memset");
    mtp_tok_dev_ = (int*)dalloc(R * sizeof(int));
    mtp_pos_dev_ = (int*)dalloc(R * sizeof(int));
    mtp_logits_ = (float*)dalloc((size_t)vocab_l_ * sizeof(float));
    mtp_next_dev_ = (int*)dalloc(kSmallRows * sizeof(int));
    cuda_check(cudaMallocHost((void**)&pinned_mtp_, 16 * sizeof(int)), "pinned");
    mtp_seed_ = mtp_out_;
  }
  cuda_check(cudaMallocHost((void**)&pinned_tok_, (size_t)std::max<int>(rows_cap_, out_cap_) * sizeof(int)), "pinned");
  cuda_check(cudaMallocHost((void**)&pinned_status_, 2 * sizeof(uint32_t)), "pinned");
  pinned_status_[0] = pinned_status_[1] = 0u;

  // comm arena: [slot0][slot1][flags0][flags1][cand val][cand idx][cand flags][epoch][status][counter]
  const int W = opt_.tp_world;
  size_t off = 0;
  const size_t slot_bytes = (size_t)W * kSmallRows * hidden_ * sizeof(float);
  for (int s = 0; s < 2; ++s) { off_slot_[s] = off; off = align_up(off + slot_bytes, 256); }
  for (int s = 0; s < 2; ++s) { off_flag_[s] = off; off = align_up(off + PK_MAX_RANKS * 4, 256); }
  const size_t bslot_bytes = W > 1 ? (size_t)W * rows_cap_ * hidden_ * sizeof(float) : 0;
  for (int s = 0; s < 2; ++s) { off_bslot_[s] = off; off = align_up(off + bslot_bytes, 256); }
  off_cval_ = off; off = align_up(off + (size_t)W * kCandStride * 4, 256);
  off_cidx_ = off; off = align_up(off + (size_t)W * kCandStride * 4, 256);
  off_cflag_ = off; off = align_up(off + PK_MAX_RANKS * 4, 256);
  off_epoch_ = off; off = align_up(off + 4, 256);
  off_status_ = off; off = align_up(off + 4, 256);
  off_counter_ = off; off = align_up(off + 4, 256);
  // {value, sequence number} slots of the persistent decode kernel: [world][hidden] 8-byte words per site parity
  for (int s = 0; s < 2; ++s) { off_ll_[s] = off; off = align_up(off + (size_t)W * hidden_ * 8, 256); }
  // tensor-parallel prefill: flags of the all-gather and the buffer of normalised rows that every owner writes into
  for (int s = 0; s < 2; ++s) { off_agflag_[s] = off; off = align_up(off + PK_MAX_RANKS * 4, 256); }
  if (W > 1) { off_xn_ = off; off = align_up(off + (size_t)rows_cap_ * hidden_ * 2, 256); }
  arena_bytes_ = off;
  arena_ = dalloc(arena_bytes_);
  cuda_check(cudaMemset(arena_, 0, std::min<size_t>(arena_bytes_, off_bslot_[0] + 4096)), "memset arena head");
  cuda_check(cudaMemset((char*)arena_ + off_cval_, 0, arena_bytes_ - off_cval_), "memset arena tail");
  for (int r = 0; r < PK_MAX_RANKS; ++r) peers_[r] = nullptr;
  peers_[opt_.tp_rank] = arena_;
  if (W > 1) xn_ = (char*)arena_ + off_xn_;
  peer_cval_dev_ = (float**)dalloc(PK_MAX_RANKS * sizeof(void*));
  peer_cidx_dev_ = (int**)dalloc(PK_MAX_RANKS * sizeof(void*));
  peers_set_ = W == 1;
  if (W == 1) {
    void* a[1] = {arena_};
    set_peer_arenas(a);
  }
}

void QwenEngine::set_peer_arenas(void* const* arenas) {
  float* cv[PK_MAX_RANKS] = {nullptr};
  int* ci[PK_MAX_RANKS] = {nullptr};
  for (int r = 0; r < opt_.tp_world; ++r) {
    peers_[r] = r == opt_.tp_rank ? arena_ : arenas[r];
    if (peers_[r] == nullptr) throw std::runtime_error("set_peer_arenas: null arena");
    cv[r] = (float*)((char*)peers_[r] + off_cval_);
    ci[r] = (int*)((char*)peers_[r] + off_cidx_);
    xn_peer_[r] = opt_.tp_world > 1 ? (char*)peers_[r] + off_xn_ : nullptr;
  }
  cuda_check(cudaMemcpy(peer_cval_dev_, cv, sizeof cv, cudaMemcpyHostToDevice), "peer table");
  cuda_check(cudaMemcpy(peer_cidx_dev_, ci, sizeof ci, cudaMemcpyHostToDevice), "peer table");
  peers_set_ = true;
  persistent_built_ = false;   // the kernel's parameter block holds peer addresses
  if (decode_graph_) {
    cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
}

QwenEngine::~QwenEngine() {
  cudaSetDevice(opt_.device);
  cudaStreamSynchronize(stream_);
  for (auto& st : stored_) {
    for (void* p : st.snap->bufs) cudaFree(p);
    for (void* p : st.snap->kv) cudaFree(p);
  }
  if (decode_graph_) cudaGraphExecDestroy(decode_graph_);
  for (void* p : allocs_) cudaFree(p);
  if (pinned_tok_) cudaFreeHost(pinned_tok_);
  if (pinned_status_) cudaFreeHost(pinned_status_);
  if (pinned_mtp_) cudaFreeHost(pinned_mtp_);
  if (txn_) {
    for (void* p : txn_->bufs) cudaFree(p);
    for (void* p : txn_->kv) cudaFree(p);
  }
  if (ev0_) cudaEventDestroy(ev0_);
  if (ev1_) cudaEventDestroy(ev1_);
  if (stream_) cudaStreamDestroy(stream_);
}

// ---------------------------------------------------------------------------------------
// weights

void QwenEngine::build_prefill_shadow() {
  if (shadow_bytes_ > 0 || act_q_ != nullptr) return;
  int mode = opt_.prefill_bf16_shadow;
  if (const char* v = getenv("POCKET_PREFILL_SHADOW")) mode = atoi(v);
  int gm = opt_.prefill_gemm;
  if (const char* v = getenv("POCKET_PREFILL_GEMM")) {
    const std::string s(v);
    gm = s == "umma" ? 0 : s == "shadow" ? 1 : s == "fp8x2" ? 2 : s == "fp8" ? 3 : gm;
  } else if (gm < 0 && getenv("POCKET_PREFILL_SHADOW") != nullptr) {
    gm = mode != 0 ? 1 : 0;
  }
  if (gm < 0) gm = mode == 1 ? 1 : 2;
  gemm_mode_ = gm;
  if (gm == 2 || gm == 3) {
    // the stored codes are the tensor-core operand: only the activations of the GEMM at hand are quantised, into this scratch
    int kmax = hidden_;
    for (int k : {inter_l_, vd_l_, hq_l_ * kHeadDim}) kmax = std::max(kmax, k);
    kmax = (int)align_up(kmax, 128);
    act_rows_ = (int)align_up(rows_cap_, 128);
    const size_t qb = (size_t)2 * act_rows_ * kmax;
    act_q_ = dalloc(qb);
    act_scale_ = (float*)dalloc((size_t)(kmax / 128) * act_rows_ * sizeof(float));
    cuda_check(cudaMemsetAsync(act_q_, 0, qb, stream_), "memset");
    cuda_check(cudaMemsetAsync(act_scale_, 0, (size_t)(kmax / 128) * act_rows_ * sizeof(float), stream_), "memset");
    cuda_check(cudaStreamSynchronize(stream_), "prefill scratch");
    return;
  }
  if (gm == 0) return;
  if (mode == 0) mode = 1;
  size_t need = 0;
  auto count = [&](const Fp8Linear& l) { need += (size_t)l.N * l.K * 2; };
  std::vector<QwenLayer*> all;
  for (auto& L : layers_) all.push_back(&L);
  if (opt_.mtp) all.push_back(&mtp_layer_);
  for (QwenLayer* lp : all) {
    QwenLayer& L = *lp;
    if (L.full) { count(L.qkv); count(L.o_proj); } else { count(L.in_proj); count(L.out_proj); }
    count(L.gate_up);
    count(L.down);
  }
  if (mode < 0) {
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess || free_b < need + (size_t(16) << 30)) return;   // keep 16 GiB for activations / KV
  }
  auto make = [&](Fp8Linear& l) {
    if (l.N == 0 || (l.K & 15)) return;
    l.wb = dalloc((size_t)l.N * l.K * 2);
    check(pk_fp8_to_bf16(l.w, l.scale, l.N, l.K, l.wb, stream_), "fp8_to_bf16");
  };
  for (QwenLayer* lp : all) {
    QwenLayer& L = *lp;
    if (L.full) { make(L.qkv); make(L.o_proj); } else { make(L.in_proj); make(L.out_proj); }
    make(L.gate_up);
    make(L.down);
  }
  cuda_check(cudaStreamSynchronize(stream_), "prefill shadow");
  shadow_bytes_ = need;
  log_device_memory("prefill_shadow_built", alloc_bytes_);
}

void QwenEngine::init_random(uint64_t seed, float sigma) {
  uint64_t s = seed * 1000003ull + 17;
  auto fp8 = [&](Fp8Linear& l) { check(pk_fill_fp8_gauss(l.w, l.scale, l.N, l.K, sigma, s++, stream_), "fill fp8"); };
  auto f32 = [&](float* p, size_t n, float mean, float sd) { check(pk_fill_f32_gauss(p, n, mean, sd, s++, stream_), "fill f32"); };
  auto b16 = [&](void* p, size_t n, float sd) { check(pk_fill_bf16_gauss(p, n, 0.f, sd, s++, stream_), "fill bf16"); };
  auto fill_layer = [&](QwenLayer& L) {
    f32(L.input_norm, hidden_, 0.f, 0.02f);
    f32(L.post_norm, hidden_, 0.f, 0.02f);
    if (L.full) {
      fp8(L.qkv);
      fp8(L.o_proj);
      f32(L.q_norm, kHeadDim, 0.f, 0.02f);
      f32(L.k_norm, kHeadDim, 0.f, 0.02f);
    } else {
      fp8(L.in_proj);
      b16(L.in_proj_ab, (size_t)2 * vh_l_ * hidden_, sigma);
      f32(L.conv_w, (size_t)conv_c_l_ * 4, 0.f, 0.3f);
      f32(L.A_log, vh_l_, 0.f, 0.5f);
      f32(L.dt_bias, vh_l_, 0.f, 0.5f);
      f32(L.lin_norm, kHeadDim, 1.f, 0.02f);
      fp8(L.out_proj);
    }
    fp8(L.gate_up);
    fp8(L.down);
  };
  for (auto& L : layers_) fill_layer(L);
  // The embedding is replicated, so every rank must draw the same table.
  check(pk_fill_bf16_gauss(embed_, (size_t)cfg_.vocab_size * hidden_, 0.f, sigma, seed * 7919ull + 1, stream_), "fill embed");
  check(pk_fill_f32_gauss(final_norm_, hidden_, 0.f, 0.02f, seed * 7919ull + 2, stream_), "fill norm");
  b16(lm_head_, (size_t)vocab_l_ * hidden_, sigma);
  if (opt_.mtp) {
    fill_layer(mtp_layer_);
    // replicated tensors: the same draw on every rank
    check(pk_fill_f32_gauss(mtp_norm_e_, hidden_, 0.f, 0.02f, seed * 7919ull + 3, stream_), "fill norm");
    check(pk_fill_f32_gauss(mtp_norm_h_, hidden_, 0.f, 0.02f, seed * 7919ull + 4, stream_), "fill norm");
    check(pk_fill_f32_gauss(mtp_norm_, hidden_, 0.f, 0.02f, seed * 7919ull + 5, stream_), "fill norm");
    check(pk_fill_bf16_gauss(mtp_fc_, (size_t)hidden_ * 2 * hidden_, 0.f, sigma, seed * 7919ull + 6, stream_), "fill fc");
  }
  cuda_check(cudaStreamSynchronize(stream_), "init_random");
  build_prefill_shadow();
}

void QwenEngine::load_safetensors(const std::string& path) {
  SafetensorsModel st(path);
  const int W = opt_.tp_world, R = opt_.tp_rank;
  std::string root = "model.language_model.";
  if (!st.has(root + "embed_tokens.weight")) root = "model.";
  if (!st.has(root + "embed_tokens.weight")) throw std::runtime_error("checkpoint has no embed_tokens.weight");

  auto upload = [&](void* dst, const void* src, size_t n) {
    cuda_check(cudaMemcpy(dst, src, n, cudaMemcpyHostToDevice), "upload");
  };
  auto norm_vec = [&](const std::string& name, float* dst, int64_t r0, int64_t n) {
    const StTensor& t = st.get(name);
    std::vector<float> v;
    if (t.dtype == StDtype::BF16) v = bf16_vec_to_f32(cut(t, 2, r0, n, 0, t.numel() / t.shape[0]));
    else if (t.dtype == StDtype::F32) {
      HostMat m = cut(t, 4, r0, n, 0, t.numel() / t.shape[0]);
      v.resize(m.data.size() / 4);
      memcpy(v.data(), m.data.data(), m.data.size());
    } else throw std::runtime_error("unsupported dtype for " + name);
    upload(dst, v.data(), v.size() * sizeof(float));
  };
  // One FP8 linear shard: weight rows [r0, r0+nr), cols [c0, c0+nc) and the matching scales.
  struct Piece { HostMat w; std::vector<float> s; int sb_rows, sb_cols; };
  auto fp8_piece = [&](const std::string& name, int64_t r0, int64_t nr, int64_t c0, int64_t nc) {
    const StTensor& w = st.get(name + ".weight");
    if (r0 % 128 || c0 % 128 || nr % 128 || nc % 128)
      throw std::runtime_error("FP8 shard of " + name + " is not aligned to the 128x128 scale blocks");
    Piece p;
    if (w.dtype == StDtype::BF16) {
      // bf16 linears (the predictor's layer in some checkpoints) are quantised here to the engine's FP8 block format
      HostMat m = cut(w, 2, r0, nr, c0, nc);
      p.w.rows = m.rows;
      p.w.cols = m.cols;
      p.w.elem = 1;
      quantize_block128(m, p.w.data, p.s);
      p.sb_rows = (int)(nr / 128);
      p.sb_cols = (int)(nc / 128);
      return p;
    }
    if (w.dtype != StDtype::F8_E4M3) throw std::runtime_error(name + ".weight is neither F8_E4M3 nor BF16");
    const StTensor& s = st.get(name + ".weight_scale_inv");
    p.w = cut(w, 1, r0, nr, c0, nc);
    p.sb_rows = (int)(nr / 128);
    p.sb_cols = (int)(nc / 128);
    if (s.dtype == StDtype::BF16) p.s = bf16_vec_to_f32(cut(s, 2, r0 / 128, nr / 128, c0 / 128, nc / 128));
    else if (s.dtype == StDtype::F32) {
      HostMat m = cut(s, 4, r0 / 128, nr / 128, c0 / 128, nc / 128);
      p.s.resize(m.data.size() / 4);
      memcpy(p.s.data(), m.data.data(), m.data.size());
    } else throw std::runtime_error("unsupported scale dtype for " + name);
    return p;
  };
  auto upload_fp8 = [&](Fp8Linear& dst, std::vector<Piece>& pieces) {
    size_t roff = 0, soff = 0;
    for (auto& p : pieces) {
      if (p.w.cols != dst.K) throw std::runtime_error("fp8 upload: K mismatch");
      upload(dst.w + roff * dst.K, p.w.data.data(), p.w.data.size());
      upload(dst.scale + soff, p.s.data(), p.s.size() * sizeof(float));
      roff += p.w.rows;
      soff += p.s.size();
    }
    if ((int)roff != dst.N) throw std::runtime_error("fp8 upload: N mismatch");
  };

  auto load_full_attention = [&](QwenLayer& L, const std::string& p) {
    const int64_t qrows = (int64_t)hq_l_ * 2 * kHeadDim, kvrows = (int64_t)hkv_l_ * kHeadDim;
    std::vector<Piece> pcs;
    pcs.push_back(fp8_piece(p + "self_attn.q_proj", R * qrows, qrows, 0, hidden_));
    pcs.push_back(fp8_piece(p + "self_attn.k_proj", R * kvrows, kvrows, 0, hidden_));
    pcs.push_back(fp8_piece(p + "self_attn.v_proj", R * kvrows, kvrows, 0, hidden_));
    upload_fp8(L.qkv, pcs);
    std::vector<Piece> o;
    o.push_back(fp8_piece(p + "self_attn.o_proj", 0, hidden_, (int64_t)R * hq_l_ * kHeadDim, (int64_t)hq_l_ * kHeadDim));
    upload_fp8(L.o_proj, o);
    norm_vec(p + "self_attn.q_norm.weight", L.q_norm, 0, kHeadDim);
    norm_vec(p + "self_attn.k_norm.weight", L.k_norm, 0, kHeadDim);
  };
  auto load_mlp = [&](QwenLayer& L, const std::string& p) {
    std::vector<Piece> gu;
    gu.push_back(fp8_piece(p + "mlp.gate_proj", (int64_t)R * inter_l_, inter_l_, 0, hidden_));
    gu.push_back(fp8_piece(p + "mlp.up_proj", (int64_t)R * inter_l_, inter_l_, 0, hidden_));
    upload_fp8(L.gate_up, gu);
    std::vector<Piece> d;
    d.push_back(fp8_piece(p + "mlp.down_proj", 0, hidden_, (int64_t)R * inter_l_, inter_l_));
    upload_fp8(L.down, d);
  };

  {
    const StTensor& e = st.get(root + "embed_tokens.weight");
    if (e.dtype != StDtype::BF16) throw std::runtime_error("embed_tokens must be BF16");
    upload(embed_, e.data, e.nbytes);
    norm_vec(root + "norm.weight", final_norm_, 0, hidden_);
    const StTensor& h = st.get("lm_head.weight");
    HostMat hm = cut(h, 2, (int64_t)vocab_start_, vocab_l_, 0, hidden_);
    upload(lm_head_, hm.data.data(), hm.data.size());
  }
  const int64_t KD = (int64_t)cfg_.linear_key_heads * kHeadDim, VD = (int64_t)cfg_.linear_value_heads * kHeadDim;
  for (int i = 0; i < cfg_.num_layers; ++i) {
    QwenLayer& L = layers_[i];
    const std::string p = root + "layers." + std::to_string(i) + ".";
    norm_vec(p + "input_layernorm.weight", L.input_norm, 0, hidden_);
    norm_vec(p + "post_attention_layernorm.weight", L.post_norm, 0, hidden_);
    if (L.full) {
      load_full_attention(L, p);
    } else {
      std::vector<Piece> pcs;
      pcs.push_back(fp8_piece(p + "linear_attn.in_proj_qkv", (int64_t)R * kd_l_, kd_l_, 0, hidden_));
      pcs.push_back(fp8_piece(p + "linear_attn.in_proj_qkv", KD + (int64_t)R * kd_l_, kd_l_, 0, hidden_));
      pcs.push_back(fp8_piece(p + "linear_attn.in_proj_qkv", 2 * KD + (int64_t)R * vd_l_, vd_l_, 0, hidden_));
      pcs.push_back(fp8_piece(p + "linear_attn.in_proj_z", (int64_t)R * vd_l_, vd_l_, 0, hidden_));
      upload_fp8(L.in_proj, pcs);
      std::vector<Piece> o;
      o.push_back(fp8_piece(p + "linear_attn.out_proj", 0, hidden_, (int64_t)R * vd_l_, vd_l_));
      upload_fp8(L.out_proj, o);
      HostMat ab = cut(st.get(p + "linear_attn.in_proj_a.weight"), 2, (int64_t)R * vh_l_, vh_l_, 0, hidden_);
      append_rows(ab, cut(st.get(p + "linear_attn.in_proj_b.weight"), 2, (int64_t)R * vh_l_, vh_l_, 0, hidden_));
      upload(L.in_proj_ab, ab.data.data(), ab.data.size());
      const StTensor& cw = st.get(p + "linear_attn.conv1d.weight");
      HostMat c = cut(cw, 2, (int64_t)R * kd_l_, kd_l_, 0, 4);
      append_rows(c, cut(cw, 2, KD + (int64_t)R * kd_l_, kd_l_, 0, 4));
      append_rows(c, cut(cw, 2, 2 * KD + (int64_t)R * vd_l_, vd_l_, 0, 4));
      std::vector<float> cf = bf16_vec_to_f32(c);
      upload(L.conv_w, cf.data(), cf.size() * sizeof(float));
      norm_vec(p + "linear_attn.A_log", L.A_log, (int64_t)R * vh_l_, vh_l_);
      norm_vec(p + "linear_attn.dt_bias", L.dt_bias, (int64_t)R * vh_l_, vh_l_);
      norm_vec(p + "linear_attn.norm.weight", L.lin_norm, 0, kHeadDim);
    }
    load_mlp(L, p);
  }
  if (opt_.mtp) {
    if (!st.has("mtp.fc.weight")) throw std::runtime_error("the checkpoint has no mtp.* tensors (multi-token predictor requested)");
    norm_vec("mtp.pre_fc_norm_embedding.weight", mtp_norm_e_, 0, hidden_);
    norm_vec("mtp.pre_fc_norm_hidden.weight", mtp_norm_h_, 0, hidden_);
    norm_vec("mtp.norm.weight", mtp_norm_, 0, hidden_);
    const StTensor& fc = st.get("mtp.fc.weight");
    if (fc.dtype != StDtype::BF16 || fc.nbytes != (size_t)hidden_ * 2 * hidden_ * 2) throw std::runtime_error("mtp.fc.weight must be BF16 [hidden, 2 * hidden]");
    upload(mtp_fc_, fc.data, fc.nbytes);
    const std::string p = "mtp.layers.0.";
    norm_vec(p + "input_layernorm.weight", mtp_layer_.input_norm, 0, hidden_);
    norm_vec(p + "post_attention_layernorm.weight", mtp_layer_.post_norm, 0, hidden_);
    load_full_attention(mtp_layer_, p);
    load_mlp(mtp_layer_, p);
  }
  (void)W;
  cuda_check(cudaDeviceSynchronize(), "load_safetensors");
  build_prefill_shadow();
}

// ---------------------------------------------------------------------------------------
// state

void QwenEngine::reset() {
  for (auto& L : layers_) {
    if (!L.full) {
      cuda_check(cudaMemsetAsync(L.lin_state, 0, (size_t)vh_l_ * kHeadDim * kHeadDim * sizeof(float), stream_), "memset");
      cuda_check(cudaMemsetAsync(L.conv_state, 0, (size_t)conv_c_l_ * 3 * sizeof(float), stream_), "memset");
    }
  }
  cuda_check(cudaMemsetAsync(out_counter_dev_, 0, sizeof(int), stream_), "memset");
  cuda_check(cudaStreamSynchronize(stream_), "reset");
  pos_ = 0;
  history_.clear();
  last_token_ = -1;
  pending_site_ = -1;
  mtp_pos_ = 0;
  mtp_ready_ = false;
  tgt_rows_ = 0;
}

std::unique_ptr<QwenEngine::Snapshot> QwenEngine::snapshot(bool with_kv) {
  auto s = std::make_unique<Snapshot>();
  if (with_kv && pos_ > 0) {
    // rows [0, pos) of every head: codes (1 or 2 bytes per channel) and, with the FP8 cache, the scales
    const size_t esz = opt_.kv_fp8 ? 1 : 2;
    const size_t row = (size_t)pos_ * kHeadDim * esz, pitch = (size_t)opt_.max_context * kHeadDim * esz;
    const size_t srow = (size_t)pos_ * 2 * sizeof(float), spitch = (size_t)opt_.max_context * 2 * sizeof(float);
    for (auto& L : layers_) {
      if (!L.full) continue;
      for (void* cache : {L.kcache, L.vcache}) {
        void* b = nullptr;
        cuda_check(cudaMalloc(&b, row * hkv_l_), "snapshot kv alloc");
        cuda_check(cudaMemcpy2DAsync(b, row, cache, pitch, row, (size_t)hkv_l_, cudaMemcpyDeviceToDevice, stream_), "snapshot kv");
        s->kv.push_back(b);
      }
      if (opt_.kv_fp8)
        for (float* sc : {L.kscale, L.vscale}) {
          void* b = nullptr;
          cuda_check(cudaMalloc(&b, srow * hkv_l_), "snapshot kv alloc");
          cuda_check(cudaMemcpy2DAsync(b, srow, sc, spitch, srow, (size_t)hkv_l_, cudaMemcpyDeviceToDevice, stream_), "snapshot kv");
          s->kv.push_back(b);
        }
    }
  }
  for (auto& L : layers_) {
    if (L.full) continue;
    const size_t sb = (size_t)vh_l_ * kHeadDim * kHeadDim * sizeof(float), cb = (size_t)conv_c_l_ * 3 * sizeof(float);
    void* a = nullptr;
    void* b = nullptr;
    cuda_check(cudaMalloc(&a, sb), "snapshot alloc");
    cuda_check(cudaMalloc(&b, cb), "snapshot alloc");
    cuda_check(cudaMemcpyAsync(a, L.lin_state, sb, cudaMemcpyDeviceToDevice, stream_), "snapshot");
    cuda_check(cudaMemcpyAsync(b, L.conv_state, cb, cudaMemcpyDeviceToDevice, stream_), "snapshot");
    s->bufs.push_back(a);
    s->bufs.push_back(b);
  }
  s->pos = pos_;
  s->last_token = last_token_;
  return s;
}

void QwenEngine::update_snapshot(Snapshot& s) {
  size_t i = 0;
  for (auto& L : layers_) {
    if (L.full) continue;
    const size_t sb = (size_t)vh_l_ * kHeadDim * kHeadDim * sizeof(float), cb = (size_t)conv_c_l_ * 3 * sizeof(float);
    cuda_check(cudaMemcpyAsync(s.bufs[i++], L.lin_state, sb, cudaMemcpyDeviceToDevice, stream_), "snapshot");
    cuda_check(cudaMemcpyAsync(s.bufs[i++], L.conv_state, cb, cudaMemcpyDeviceToDevice, stream_), "snapshot");
  }
  s.pos = pos_;
  s.last_token = last_token_;
}

void QwenEngine::restore(const Snapshot& s) {
  size_t i = 0;
  for (auto& L : layers_) {
    if (L.full) continue;
    const size_t sb = (size_t)vh_l_ * kHeadDim * kHeadDim * sizeof(float), cb = (size_t)conv_c_l_ * 3 * sizeof(float);
    cuda_check(cudaMemcpyAsync(L.lin_state, s.bufs[i++], sb, cudaMemcpyDeviceToDevice, stream_), "restore");
    cuda_check(cudaMemcpyAsync(L.conv_state, s.bufs[i++], cb, cudaMemcpyDeviceToDevice, stream_), "restore");
  }
  if (!s.kv.empty()) {
    const size_t esz = opt_.kv_fp8 ? 1 : 2;
    const size_t row = (size_t)s.pos * kHeadDim * esz, pitch = (size_t)opt_.max_context * kHeadDim * esz;
    const size_t srow = (size_t)s.pos * 2 * sizeof(float), spitch = (size_t)opt_.max_context * 2 * sizeof(float);
    size_t k = 0;
    for (auto& L : layers_) {
      if (!L.full) continue;
      for (void* cache : {L.kcache, L.vcache})
        cuda_check(cudaMemcpy2DAsync(cache, pitch, s.kv[k++], row, row, (size_t)hkv_l_, cudaMemcpyDeviceToDevice, stream_), "restore kv");
      if (opt_.kv_fp8)
        for (float* sc : {L.kscale, L.vscale})
          cuda_check(cudaMemcpy2DAsync(sc, spitch, s.kv[k++], srow, srow, (size_t)hkv_l_, cudaMemcpyDeviceToDevice, stream_), "restore kv");
    }
  }
  // decode() reads its input token from slot 0 of the device token buffer
  cuda_check(cudaMemcpyAsync(next_tok_dev_, &s.last_token, sizeof(int), cudaMemcpyHostToDevice, stream_), "restore token");
  cuda_check(cudaStreamSynchronize(stream_), "restore");
  pos_ = s.pos;
  if ((int)history_.size() > s.pos) history_.resize((size_t)s.pos);
  last_token_ = s.last_token;
  mtp_ready_ = false;     // the predictor's boundary row belongs to the abandoned position
  mtp_pos_ = s.pos;
}

void QwenEngine::free_snapshot(Snapshot& s) {
  cudaStreamSynchronize(stream_);
  for (void* p : s.bufs) cudaFree(p);
  for (void* p : s.kv) cudaFree(p);
  s.bufs.clear();
  s.kv.clear();
}

uint32_t QwenEngine::comm_status() {
  uint32_t v[2] = {0, 0};
  cuda_check(cudaMemcpy(&v[0], (char*)arena_ + off_status_, 4, cudaMemcpyDeviceToHost), "status");
  cuda_check(cudaMemcpy(&v[1], gemm_status_, 4, cudaMemcpyDeviceToHost), "status");
  // bits 0-7: peer waits, 8-15: tensor-core GEMM waits, 16-23: matvec ring waits
  return v[0] | (v[1] << 8) | ((pk_matvec_ring_status() & 0xffu) << 16);
}

void QwenEngine::clear_comm_status() {
  cuda_check(cudaMemsetAsync((char*)arena_ + off_status_, 0, 4, stream_), "clear status");
  cuda_check(cudaMemsetAsync(gemm_status_, 0, 4, stream_), "clear status");
  cuda_check(cudaStreamSynchronize(stream_), "clear status");
  (void)pk_matvec_ring_status();   // reading clears it
  pinned_status_[0] = pinned_status_[1] = 0u;
}

void QwenEngine::queue_status_read() {
  cuda_check(cudaMemcpyAsync(&pinned_status_[0], (char*)arena_ + off_status_, 4, cudaMemcpyDeviceToHost, stream_), "status");
  cuda_check(cudaMemcpyAsync(&pinned_status_[1], gemm_status_, 4, cudaMemcpyDeviceToHost, stream_), "status");
}

void QwenEngine::raise_if_step_failed(const char* what) {
  if (pinned_status_[0] == 0u && pinned_status_[1] == 0u) return;
  const uint32_t peer = pinned_status_[0], gemm = pinned_status_[1];
  clear_comm_status();
  // tokens of this step are not handed out; a graph that holds the failed kernels' state is rebuilt on the next decode
  last_token_ = -1;
  // The status word travels with the sampler exchange, so every rank arrives here in the same step: all of them leave
  // the peer-store path together.
  const bool to_nccl = peer != 0u && nccl_ != nullptr && !nccl_mode_;
  if (to_nccl) switch_to_nccl();
  char buf[260];
  snprintf(buf, sizeof buf, "%s: a bounded device wait ran out (peer word %u, tensor-core word %u); the step is discarded%s", what, peer, gemm,
           to_nccl ? "; later steps use NCCL collectives" : "");
  throw CommTimeout(buf);
}

void QwenEngine::enable_nccl_fallback(const std::string& id_path, int timeout_ms) {
  if (opt_.tp_world < 2) return;
  if (!NcclComm::available()) throw std::runtime_error("NCCL was not found (libnccl.so.2)");
  nccl_ = std::make_shared<NcclComm>(id_path, opt_.tp_rank, opt_.tp_world, opt_.device, timeout_ms);
}

void QwenEngine::switch_to_nccl() {
  if (nccl_mode_) return;
  if (nccl_ == nullptr) throw std::runtime_error("switch_to_nccl: enable_nccl_fallback was not called");
  cuda_check(cudaStreamSynchronize(stream_), "sync");
  nccl_mode_ = true;
  // one launch per projection from here on: the persistent kernel and a captured graph hold peer pointers and flags
  persistent_built_ = true;
  persistent_ok_ = false;
  if (decode_graph_) {
    cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
  opt_.use_cuda_graph = false;
  clear_comm_status();
}

void QwenEngine::set_tap_layers(const int* layers, int n) {
  if (opt_.tp_world > 1) throw std::runtime_error("target taps are captured on one rank only");
  for (int i = 0; i < n; ++i)
    if (layers[i] < 0 || layers[i] >= cfg_.num_layers) throw std::runtime_error("tap layer outside the model");
  cuda_check(cudaStreamSynchronize(stream_), "sync");
  tap_layers_.assign(layers, layers + n);
  taps_ = nullptr;
  if (n > 0) taps_ = dalloc((size_t)rows_cap_ * n * hidden_ * 2);
  tap_rows_ = 0;
  set_persistent_decode(n > 0 ? 0 : opt_.persistent_decode);   // per-projection decode while taps are on; drops a captured graph
}

void QwenEngine::capture_tap(int layer, const void* rows, int M) {
  for (size_t s = 0; s < tap_layers_.size(); ++s)
    if (tap_layers_[s] == layer) {
      const size_t pitch = tap_layers_.size() * (size_t)hidden_ * 2;
      cuda_check(cudaMemcpy2DAsync((char*)taps_ + s * (size_t)hidden_ * 2, pitch, rows, (size_t)hidden_ * 2, (size_t)hidden_ * 2, (size_t)M,
                                   cudaMemcpyDeviceToDevice, stream_),
                 "tap copy");
      ++launches_;
    }
}

void QwenEngine::copy_taps(void* dst_device, int first_row, int rows) {
  if (tap_layers_.empty()) throw std::runtime_error("no tap layers set");
  if (first_row < 0 || rows < 1 || first_row + rows > tap_rows_) throw std::runtime_error("copy_taps: rows outside the last forward");
  const size_t pitch = tap_layers_.size() * (size_t)hidden_ * 2;
  cuda_check(cudaMemcpyAsync(dst_device, (char*)taps_ + (size_t)first_row * pitch, (size_t)rows * pitch, cudaMemcpyDeviceToDevice, stream_), "taps");
  cuda_check(cudaStreamSynchronize(stream_), "taps");
}

void QwenEngine::copy_logits(float* out_host, int row) {
  cuda_check(cudaStreamSynchronize(stream_), "sync");
  cuda_check(cudaMemcpy(out_host, logits_ + (size_t)row * vocab_l_, (size_t)vocab_l_ * sizeof(float), cudaMemcpyDeviceToHost), "logits");
}

void QwenEngine::copy_mtp_logits(float* out_host) {
  if (!opt_.mtp) throw std::runtime_error("the engine was built without the multi-token predictor");
  cuda_check(cudaStreamSynchronize(stream_), "sync");
  cuda_check(cudaMemcpy(out_host, mtp_logits_, (size_t)vocab_l_ * sizeof(float), cudaMemcpyDeviceToHost), "logits");
}

// ---------------------------------------------------------------------------------------
// comm helpers

float* QwenEngine::slot_parts(int site, bool big) const {
  return (float*)((char*)arena_ + (big ? off_bslot_[site & 1] : off_slot_[site & 1]));
}

PkWait QwenEngine::make_wait(int site) const {
  PkWait w{};
  w.flag = opt_.tp_world > 1 ? (const uint32_t*)((char*)arena_ + off_flag_[site & 1]) : nullptr;
  w.epoch = (const uint32_t*)((char*)arena_ + off_epoch_);
  w.sites_per_epoch = sites_per_epoch_;
  w.site = site;
  w.world = opt_.tp_world;
  w.status = (uint32_t*)((char*)arena_ + off_status_);
  w.timeout_us = opt_.comm_timeout_us;
  return w;
}

PkPush QwenEngine::make_push(int site, bool big, int rows_per_rank) const {
  PkPush p{};
  if (nccl_mode_) {
    // this rank's partial rows go to the first slot of its own arena, unflagged; NCCL adds the ranks' slots in place
    p.dst[0] = (float*)((char*)arena_ + (big ? off_bslot_[site & 1] : off_slot_[site & 1]));
    p.block_counter = (uint32_t*)((char*)arena_ + off_counter_);
    p.epoch = (const uint32_t*)((char*)arena_ + off_epoch_);
    p.sites_per_epoch = sites_per_epoch_;
    p.site = site;
    p.world = 1;
    p.rank = 0;
    return p;
  }
  p.rows_per_rank = rows_per_rank;
  for (int r = 0; r < opt_.tp_world; ++r) {
    p.dst[r] = (float*)((char*)peers_[r] + (big ? off_bslot_[site & 1] : off_slot_[site & 1]));
    p.flag[r] = opt_.tp_world > 1 ? (uint32_t*)((char*)peers_[r] + off_flag_[site & 1]) : nullptr;
  }
  p.block_counter = (uint32_t*)((char*)arena_ + off_counter_);
  p.epoch = (const uint32_t*)((char*)arena_ + off_epoch_);
  p.sites_per_epoch = sites_per_epoch_;
  p.site = site;
  p.world = opt_.tp_world;
  p.rank = opt_.tp_rank;
  return p;
}

// ---------------------------------------------------------------------------------------
// forward, weight-streaming path (1..8 rows)

void QwenEngine::run_small(int M, bool all_logits, bool mtp) {
  if (!peers_set_) throw std::runtime_error("peer arenas not registered");
  const float eps = (float)cfg_.rms_norm_eps;
  const int W = opt_.tp_world;
  const int* posd = mtp ? mtp_pos_dev_ : pos_dev_;
  const int n_layers = mtp ? 1 : cfg_.num_layers;
  if (!mtp) tap_rows_ = tap_layers_.empty() ? 0 : M;
  check(pk_bump_epoch((uint32_t*)((char*)arena_ + off_epoch_), stream_), "epoch");
  if (mtp) {
    check(pk_mtp_concat_norm(mtp_tok_dev_, M, embed_, mtp_in_, hidden_, mtp_norm_e_, mtp_norm_h_, eps, mtp_cat_, stream_), "mtp_concat_norm");
    check(pk_matvec(nullptr, nullptr, mtp_fc_, 0, hidden_, 2 * hidden_, M, mtp_cat_, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 0,
                    hidden_buf_[cur_], hidden_, nullptr, sm_count_, stream_),
          "matvec(mtp fc)");
  } else {
    check(pk_embedding(tokens_dev_, M, embed_, hidden_, 0, (int)cfg_.vocab_size, hidden_buf_[cur_], nullptr, stream_), "embedding");
  }
  int pending = -1;  // site whose partial sums still wait to be added to the residual stream

  auto consume = [&](const Fp8Linear* w, const void* wb, int nb, const float* gamma, int epi, void* y, int ldy,
                     const PkPush* push) {
    // x = hidden (+ pending partials) -> norm -> linear. The summed hidden goes to the other buffer.
    const float* parts = pending >= 0 ? slot_parts(pending) : nullptr;
    PkWait wt = make_wait(pending >= 0 ? pending : 0);
    void* hout = pending >= 0 ? hidden_buf_[cur_ ^ 1] : nullptr;
    check(pk_matvec(w ? w->w : nullptr, w ? w->scale : nullptr, wb, w ? w->N : 0, nb, hidden_, M, hidden_buf_[cur_], parts,
                    kernel_world(), hout, gamma, 1, eps, pending >= 0 && !nccl_mode_ ? &wt : nullptr, epi, y, ldy, push, sm_count_, stream_),
          "matvec(consume)");
    if (pending >= 0) cur_ ^= 1;
    // the summed residual stream now holds the output of the layer whose down projection was pending
    if (!mtp && !tap_layers_.empty() && pending >= 0 && (pending & 1)) capture_tap(pending >> 1, hidden_buf_[cur_], M);
    pending = -1;
  };
  auto produce = [&](const Fp8Linear& w, const void* x, int site) {
    PkPush ps = make_push(site);
    check(pk_matvec(w.w, w.scale, nullptr, w.N, 0, w.K, M, x, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 3,
                    nullptr, hidden_, &ps, sm_count_, stream_),
          "matvec(produce)");
    if (nccl_mode_) nccl_->all_reduce_sum(slot_parts(site), (size_t)M * hidden_, NcclComm::Dtype::F32, stream_);
    pending = site;
  };

  for (int i = 0; i < n_layers; ++i) {
    QwenLayer& L = mtp ? mtp_layer_ : layers_[i];
    if (L.full) {
      consume(&L.qkv, nullptr, 0, L.input_norm, 0, proj_, ld_proj_, nullptr);
      check(pk_qk_norm_rope_append_kv(proj_, ld_proj_, M, hq_l_, hkv_l_, kHeadDim, posd, L.q_norm, L.k_norm, eps,
                                      cfg_.rotary_dim(), (float)cfg_.rope_theta, q_buf_, L.kcache, L.vcache, L.kscale, L.vscale,
                                      opt_.max_context, stream_),
            "qk_norm_rope_append");
      check(pk_gqa_decode_kv(q_buf_, L.kcache, L.vcache, L.kscale, L.vscale, posd, M, hq_l_, hkv_l_, kHeadDim, opt_.max_context,
                             1.f / sqrtf((float)kHeadDim), opt_.decode_splits, opt_.attention_window, opt_.attention_sink,
                             attn_ws_, cfg_.attn_output_gate ? proj_ : nullptr, ld_proj_, attn_out_, stream_),
            "gqa_decode");
      ++launches_;  // two kernels in that call
      produce(L.o_proj, attn_out_, 2 * i);
    } else {
      consume(&L.in_proj, L.in_proj_ab, 2 * vh_l_, L.input_norm, 0, proj_, ld_proj_, nullptr);
      check(pk_deltanet_seq(proj_, ld_proj_, M, kh_l_, vh_l_, kHeadDim, kHeadDim, L.conv_w, L.conv_state, L.A_log,
                            L.dt_bias, L.lin_norm, eps, L.lin_state, attn_out_, stream_),
            "deltanet_seq");
      produce(L.out_proj, attn_out_, 2 * i);
    }
    consume(&L.gate_up, nullptr, 0, L.post_norm, 1, mlp_h_, inter_l_, nullptr);
    produce(L.down, mlp_h_, 2 * i + 1);
  }
  if (opt_.mtp) {
    // The normalised rows are kept: the target's feed the predictor, the predictor's last one seeds its next row.
    const float* parts = slot_parts(pending);
    PkWait wt = make_wait(pending);
    void* y = mtp ? mtp_out_ : tgt_hid_;
    check(pk_rmsnorm(hidden_buf_[cur_], parts, kernel_world(), M, hidden_, hidden_buf_[cur_], mtp ? mtp_norm_ : final_norm_, 1, eps, y,
                     nccl_mode_ ? nullptr : &wt, stream_),
          "final norm");
    if (!mtp && !tap_layers_.empty() && (pending & 1)) capture_tap(pending >> 1, hidden_buf_[cur_], M);
    pending = -1;
    const bool all = !mtp && (all_logits || M == 1);
    const int rows = all ? M : 1;
    const char* x = (const char*)y + (all ? 0 : (size_t)(M - 1) * hidden_ * 2);
    float* lg = mtp ? mtp_logits_ : logits_;
    check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, rows, x, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 2, lg,
                    vocab_l_, nullptr, sm_count_, stream_),
          "lm_head");
    sample_rows(rows, lg, mtp ? mtp_next_dev_ : next_tok_dev_);
    if (mtp) mtp_seed_ = x;
    else tgt_rows_ = M;
    return;
  }
  // final norm + lm_head on every row (speculative verify) or on the last row only
  if (all_logits || M == 1) {
    consume(nullptr, lm_head_, vocab_l_, final_norm_, 2, logits_, vocab_l_, nullptr);
    sample_rows(M, logits_, next_tok_dev_);
  } else {
    // Fold the pending partials into the hidden state first, then project the last row.
    const float* parts = slot_parts(pending);
    PkWait wt = make_wait(pending);
    check(pk_rmsnorm(hidden_buf_[cur_], parts, kernel_world(), M, hidden_, hidden_buf_[cur_], final_norm_, 1, eps, nullptr,
                     nccl_mode_ ? nullptr : &wt, stream_),
          "fold");
    if (!tap_layers_.empty() && (pending & 1)) capture_tap(pending >> 1, hidden_buf_[cur_], M);
    pending = -1;
    const char* last = (const char*)hidden_buf_[cur_] + (size_t)(M - 1) * hidden_ * 2;
    check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, last, nullptr, 0, nullptr, final_norm_, 1, eps,
                    nullptr, 2, logits_, vocab_l_, nullptr, sm_count_, stream_),
          "lm_head");
    sample_rows(1, logits_, next_tok_dev_);
  }
}

// Greedy token of `M` logits rows -> out[0..M).
void QwenEngine::sample_rows(int M, const float* logits, int* out) {
  const int W = opt_.tp_world;
  check(pk_argmax(logits, vocab_l_, M, vocab_l_, vocab_start_, kArgmaxBlocks, cand_val_,
                  cand_idx_, best_val_, W == 1 ? out : best_idx_, stream_),
        "argmax");
  ++launches_;
  if (W > 1 && nccl_mode_) {
    // each rank's row of candidates into its own arena, then one all-gather per array, then the same merge
    PkPush ps{};
    ps.world = 1;
    ps.rank = opt_.tp_rank;
    ps.block_counter = (uint32_t*)((char*)arena_ + off_counter_);
    ps.epoch = (const uint32_t*)((char*)arena_ + off_epoch_);
    ps.sites_per_epoch = sites_per_epoch_;
    uint32_t* status = (uint32_t*)((char*)arena_ + off_status_);
    check(pk_cand_push(best_val_, best_idx_, M, &ps, peer_cval_dev_ + opt_.tp_rank, peer_cidx_dev_ + opt_.tp_rank, status, kCandStride, stream_), "cand_push");
    float* cval = (float*)((char*)arena_ + off_cval_);
    int* cidx = (int*)((char*)arena_ + off_cidx_);
    nccl_->all_gather(cval + (size_t)opt_.tp_rank * kCandStride, cval, kCandStride, NcclComm::Dtype::F32, stream_);
    nccl_->all_gather(cidx + (size_t)opt_.tp_rank * kCandStride, cidx, kCandStride, NcclComm::Dtype::I32, stream_);
    PkWait wt = make_wait(2 * cfg_.num_layers);
    wt.flag = nullptr;
    check(pk_cand_merge_wait(cval, cidx, M, W, &wt, out, status, kCandStride, stream_), "cand_merge");
  } else if (W > 1) {
    // Exchange {logit, token} of every rank through peer memory and merge (lowest id on ties).
    const int site = 2 * cfg_.num_layers;
    PkPush ps = make_push(site);
    for (int r = 0; r < W; ++r) ps.flag[r] = (uint32_t*)((char*)peers_[r] + off_cflag_);
    uint32_t* status = (uint32_t*)((char*)arena_ + off_status_);
    check(pk_cand_push(best_val_, best_idx_, M, &ps, peer_cval_dev_, peer_cidx_dev_, status, kCandStride, stream_), "cand_push");
    PkWait wt = make_wait(site);
    wt.flag = (const uint32_t*)((char*)arena_ + off_cflag_);
    check(pk_cand_merge_wait((const float*)((char*)arena_ + off_cval_), (const int*)((char*)arena_ + off_cidx_), M, W,
                             &wt, out, status, kCandStride, stream_),
          "cand_merge");
  }
}

// ---------------------------------------------------------------------------------------
// forward, tensor-core path (more than 8 rows, one rank)

void QwenEngine::run_chunk(int M, bool mtp) {
  if (!peers_set_) throw std::runtime_error("peer arenas not registered");
  const float eps = (float)cfg_.rms_norm_eps;
  const int W = opt_.tp_world;
  const int* posd = mtp ? mtp_pos_dev_ : pos_dev_;
  const int n_layers = mtp ? 1 : cfg_.num_layers;
  void* hid = hidden_buf_[cur_];
  if (!mtp) tap_rows_ = tap_layers_.empty() ? 0 : M;
  if (W > 1) check(pk_bump_epoch((uint32_t*)((char*)arena_ + off_epoch_), stream_), "epoch");
  if (mtp) {
    check(pk_mtp_concat_norm(mtp_tok_dev_, M, embed_, mtp_in_, hidden_, mtp_norm_e_, mtp_norm_h_, eps, mtp_cat_, stream_), "mtp_concat_norm");
    int rc = pk_gemm_bf16(mtp_cat_, 2 * hidden_, mtp_fc_, M, hidden_, 2 * hidden_, 0, hid, nullptr, hidden_, gemm_status_, nullptr, sm_count_, stream_);
    if (rc == 4) rc = pk_gemm_umma(mtp_cat_, 2 * hidden_, mtp_fc_, nullptr, 1, M, hidden_, 2 * hidden_, 0, hid, nullptr, hidden_, gemm_status_, nullptr, stream_);
    check(rc, "gemm(mtp fc)");
  } else {
    check(pk_embedding(tokens_dev_, M, embed_, hidden_, 0, (int)cfg_.vocab_size, hid, nullptr, stream_), "embedding");
  }
  int pending = -1;  // site whose partial sums still wait to be added to the residual stream
  // Native FP8: quantise the rows of A (one or two E4M3 terms per value, a scale per row and 128-wide k block), then run
  // tcgen05 kind::f8f6f4 on them and on the stored weight codes. Shapes the kernel does not take fall through.
  // true while act_q_ / act_scale_ hold the quantised rows of xn_ (written by the norm kernel itself)
  bool xn_quantised = false;
  auto gemm_native = [&](const void* A, int lda, const Fp8Linear& w, int epi, void* C, const void* resid, int ldc, const PkPush* ps) -> bool {
    if (act_q_ == nullptr || w.w == nullptr || w.scale == nullptr || (w.K & 127) != 0 || (lda & 3) != 0 || M > act_rows_) return false;   // bf16-only linears have no codes
    if (epi == 1 && ((w.N >> 1) & 127) != 0) return false;
    const int terms = gemm_mode_ == 3 ? 1 : 2;
    if (!(xn_quantised && A == xn_ && lda == hidden_ && w.K == hidden_)) {
      check(pk_quant_act_fp8(A, lda, M, w.K, terms, act_q_, act_rows_, act_scale_, act_rows_, stream_), "quant_act_fp8");
      xn_quantised = false;
    }
    check(pk_gemm_fp8(act_q_, terms, act_rows_, act_scale_, act_rows_, w.w, w.scale, M, w.N, w.K, epi, C, resid, ldc, gemm_status_, ps, sm_count_,
                      stream_), "gemm_fp8");
    return true;
  };
  auto gemm = [&](const void* A, int lda, const Fp8Linear& w, int epi, void* C, const void* resid, int ldc) {
    if (gemm_native(A, lda, w, epi, C, resid, ldc, nullptr)) return;
    if (w.wb != nullptr) {
      // persistent 128x256 kernel; shapes it does not take (SwiGLU halves not a multiple of 128) go to the 128x128 one
      int rc = pk_gemm_bf16(A, lda, w.wb, M, w.N, w.K, epi, C, resid, ldc, gemm_status_, nullptr, sm_count_, stream_);
      if (rc == 4) rc = pk_gemm_umma(A, lda, w.wb, nullptr, 1, M, w.N, w.K, epi, C, resid, ldc, gemm_status_, nullptr, stream_);
      check(rc, "gemm_bf16");
    } else
      check(pk_gemm_umma(A, lda, w.w, w.scale, 0, M, w.N, w.K, epi, C, resid, ldc, gemm_status_, nullptr, stream_), "gemm_umma");
  };
  // Row-parallel projection back into the residual stream. One rank: residual add in the epilogue. Several ranks:
  // reduce-scatter + all-gather around the norm. Rows are owned in blocks of rpr = ceil(M / W); the GEMM epilogue
  // stores each fp32 partial row into its OWNER's slot only, tile by tile (1 / W of the bytes of a push to everyone);
  // the owner's norm kernel adds the W partials and the residual for its rows, keeps the new residual rows to itself,
  // and writes the normalised bf16 rows into every rank's activation buffer (the all-gather), then waits until the
  // other owners' rows have arrived. The residual stream of rows a rank does not own is never needed there.
  const int rpr = (M + W - 1) / W;
  auto gemm_out = [&](const void* A, int lda, const Fp8Linear& w, int site) {
    if (W == 1) {
      gemm(A, lda, w, 2, hid, hid, hidden_);
    } else if (nccl_mode_) {
      // fp32 partial rows into this rank's slot, summed over the ranks in place; the next norm adds them to the residual
      float* slot = slot_parts(site, true);
      gemm(A, lda, w, 3, slot, nullptr, hidden_);
      nccl_->all_reduce_sum(slot, (size_t)M * hidden_, NcclComm::Dtype::F32, stream_);
      pending = site;
    } else {
      PkPush ps = make_push(site, true, rpr);
      if (gemm_native(A, lda, w, 4, nullptr, nullptr, hidden_, &ps)) {
      } else if (w.wb != nullptr)
        check(pk_gemm_bf16(A, lda, w.wb, M, w.N, w.K, 4, nullptr, nullptr, hidden_, gemm_status_, &ps, sm_count_, stream_), "gemm_bf16(push)");
      else
        check(pk_gemm_umma(A, lda, w.w, w.scale, 0, M, w.N, w.K, 4, nullptr, nullptr, hidden_, gemm_status_, &ps, stream_), "gemm_umma(push)");
      pending = site;
    }
  };
  // y == nullptr with pending partials folds them into the owners' residual rows only.
  auto norm = [&](const float* gamma, void* y) {
    if (pending >= 0 && nccl_mode_) {
      check(pk_rmsnorm(hid, slot_parts(pending, true), 1, M, hidden_, hid, gamma, 1, eps, y, nullptr, stream_), "rmsnorm(+reduced rows)");
      pending = -1;
    } else if (pending >= 0) {
      PkWait wrs = make_wait(pending);
      PkPush pag = make_push(pending, true);
      PkWait wag = make_wait(pending);
      for (int r = 0; r < W; ++r) pag.flag[r] = (uint32_t*)((char*)peers_[r] + off_agflag_[pending & 1]);
      wag.flag = (const uint32_t*)((char*)arena_ + off_agflag_[pending & 1]);
      check(pk_rmsnorm_rs_ag(hid, slot_parts(pending, true), W, opt_.tp_rank, rpr, M, hidden_, gamma, 1, eps, xn_peer_, &wrs, &pag, &wag,
                             sm_count_, stream_),
            "rmsnorm(reduce-scatter, all-gather)");
      // the gathered rows live in the arena buffer; callers that want them elsewhere get a copy
      if (y != nullptr && y != xn_)
        cuda_check(cudaMemcpyAsync(y, xn_, (size_t)M * hidden_ * 2, cudaMemcpyDeviceToDevice, stream_), "copy normalised rows");
      pending = -1;
    } else if (y == xn_ && act_q_ != nullptr && (gemm_mode_ == 2 || gemm_mode_ == 3) && (hidden_ & 127) == 0 && M <= act_rows_) {
      // the rows feed a native FP8 GEMM next: the norm kernel quantises them on the way out
      check(pk_rmsnorm_quant(hid, M, hidden_, gamma, 1, eps, y, gemm_mode_ == 3 ? 1 : 2, act_q_, act_rows_, act_scale_, act_rows_, stream_),
            "rmsnorm(+quantise)");
      xn_quantised = true;
    } else {
      check(pk_rmsnorm(hid, nullptr, 0, M, hidden_, nullptr, gamma, 1, eps, y, nullptr, stream_), "rmsnorm");
      xn_quantised = false;
    }
  };
  for (int i = 0; i < n_layers; ++i) {
    QwenLayer& L = mtp ? mtp_layer_ : layers_[i];
    norm(L.input_norm, xn_);
    if (L.full) {
      gemm(xn_, hidden_, L.qkv, 0, proj_, nullptr, ld_proj_);
      check(pk_qk_norm_rope_append_kv(proj_, ld_proj_, M, hq_l_, hkv_l_, kHeadDim, posd, L.q_norm, L.k_norm, eps,
                                      cfg_.rotary_dim(), (float)cfg_.rope_theta, q_buf_, L.kcache, L.vcache, L.kscale, L.vscale,
                                      opt_.max_context, stream_),
            "qk_norm_rope_append");
      if (tc_prefill_attn_ && M >= 16) {
        // causal flash attention on the tensor cores (bf16 cache, full attention); the rows behind the chunk that its last
        // tile reads are masked and were zeroed when the cache was allocated
        check(pk_gqa_prefill_umma(q_buf_, L.kcache, L.vcache, posd, M, hq_l_, hkv_l_, kHeadDim, opt_.max_context, 1.f / sqrtf((float)kHeadDim),
                                  cfg_.attn_output_gate ? proj_ : nullptr, ld_proj_, attn_out_, gemm_status_, stream_),
              "gqa_prefill_umma");
      } else {
        check(pk_gqa_decode_kv(q_buf_, L.kcache, L.vcache, L.kscale, L.vscale, posd, M, hq_l_, hkv_l_, kHeadDim, opt_.max_context,
                               1.f / sqrtf((float)kHeadDim), 1, opt_.attention_window, opt_.attention_sink, attn_ws_,
                               cfg_.attn_output_gate ? proj_ : nullptr, ld_proj_, attn_out_, stream_),
              "gqa_prefill");
        ++launches_;
      }
      gemm_out(attn_out_, hq_l_ * kHeadDim, L.o_proj, 2 * i);
    } else {
      gemm(xn_, hidden_, L.in_proj, 0, proj_, nullptr, ld_proj_);
      check(pk_gemm_umma(xn_, hidden_, L.in_proj_ab, nullptr, 1, M, 2 * vh_l_, hidden_, 0,
                         (char*)proj_ + (size_t)L.in_proj.N * 2, nullptr, ld_proj_, gemm_status_, nullptr, stream_),
            "gemm_umma(ab)");
      if (M >= 32) {
        check(pk_deltanet_chunked(proj_, ld_proj_, M, kh_l_, vh_l_, kHeadDim, kHeadDim, L.conv_w, L.conv_state, L.A_log,
                                  L.dt_bias, L.lin_norm, eps, L.lin_state, attn_out_, lin_ws_, stream_),
              "deltanet_chunked");
        launches_ += 4;  // five kernels in that call
      } else {
        check(pk_deltanet_seq(proj_, ld_proj_, M, kh_l_, vh_l_, kHeadDim, kHeadDim, L.conv_w, L.conv_state, L.A_log,
                              L.dt_bias, L.lin_norm, eps, L.lin_state, attn_out_, stream_),
              "deltanet_seq");
      }
      gemm_out(attn_out_, vd_l_, L.out_proj, 2 * i);
    }
    norm(L.post_norm, xn_);
    gemm(xn_, hidden_, L.gate_up, 1, mlp_h_, nullptr, inter_l_);
    gemm_out(mlp_h_, inter_l_, L.down, 2 * i + 1);
    if (!mtp && W == 1 && !tap_layers_.empty()) capture_tap(i, hid, M);   // one rank: the epilogue added the residual in place
  }
  if (opt_.mtp && !mtp) {
    // every normalised row feeds the predictor; the last one also gives the logits
    norm(final_norm_, tgt_hid_);
    tgt_rows_ = M;
    const char* x = (const char*)tgt_hid_ + (size_t)(M - 1) * hidden_ * 2;
    check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, x, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 2, logits_,
                    vocab_l_, nullptr, sm_count_, stream_),
          "lm_head");
    sample_rows(1, logits_, next_tok_dev_);
    return;
  }
  if (W > 1) {
    // several ranks: only the owner of the last row has its residual; the final norm is the reduce-scatter /
    // all-gather kind, and every rank reads the gathered last row
    const char* xlast = (const char*)xn_ + (size_t)(M - 1) * hidden_ * 2;
    if (mtp) {
      norm(mtp_norm_, xn_);
      cuda_check(cudaMemcpyAsync(mtp_out_, xlast, (size_t)hidden_ * 2, cudaMemcpyDeviceToDevice, stream_), "copy predictor row");
      check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, mtp_out_, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 2,
                      mtp_logits_, vocab_l_, nullptr, sm_count_, stream_),
            "lm_head(mtp)");
      sample_rows(1, mtp_logits_, mtp_next_dev_);
      mtp_seed_ = mtp_out_;
      return;
    }
    norm(final_norm_, xn_);
    check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, xlast, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 2, logits_,
                    vocab_l_, nullptr, sm_count_, stream_),
          "lm_head");
    sample_rows(1, logits_, next_tok_dev_);
    return;
  }
  const char* last = (const char*)hid + (size_t)(M - 1) * hidden_ * 2;
  if (mtp) {
    check(pk_rmsnorm(last, nullptr, 0, 1, hidden_, nullptr, mtp_norm_, 1, eps, mtp_out_, nullptr, stream_), "mtp norm");
    check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, mtp_out_, nullptr, 0, nullptr, nullptr, 0, eps, nullptr, 2,
                    mtp_logits_, vocab_l_, nullptr, sm_count_, stream_),
          "lm_head(mtp)");
    sample_rows(1, mtp_logits_, mtp_next_dev_);
    mtp_seed_ = mtp_out_;
    return;
  }
  check(pk_matvec(nullptr, nullptr, lm_head_, 0, vocab_l_, hidden_, 1, last, nullptr, 0, nullptr, final_norm_, 1, eps,
                  nullptr, 2, logits_, vocab_l_, nullptr, sm_count_, stream_),
        "lm_head");
  sample_rows(1, logits_, next_tok_dev_);
}

// ---------------------------------------------------------------------------------------
// public entry points

int QwenEngine::prefill(const int* tokens_host, int n) {
  for (int t = 0; t < n; ++t)
    if (tokens_host[t] < 0 || tokens_host[t] >= cfg_.vocab_size)
      throw std::runtime_error("token id " + std::to_string(tokens_host[t]) + " is outside the vocabulary of " + std::to_string(cfg_.vocab_size));
  if (n < 1) throw std::runtime_error("prefill: empty prompt");
  if (pos_ + n + 1 > opt_.max_context) throw std::runtime_error("prefill: prompt exceeds max_context");
  cuda_check(cudaEventRecord(ev0_, stream_), "event");
  const long long l0 = launches_;
  int done = 0;
  // The prompt is staged in pinned memory once (in pieces only when it is longer than the staging buffer), so the chunks
  // queue back to back and the host never waits for the device inside the loop.
  const int stage_cap = std::max<int>(rows_cap_, out_cap_);
  int stage_base = 0, stage_end = 0;
  while (done < n) {
    if (done >= stage_end) {
      if (stage_end > 0) cuda_check(cudaStreamSynchronize(stream_), "prefill staging");   // copies out of the buffer are over
      stage_base = done;
      stage_end = done + std::min(n - done, stage_cap);
      memcpy(pinned_tok_, tokens_host + stage_base, (size_t)(stage_end - stage_base) * sizeof(int));
    }
    int M = std::min(std::min(n - done, rows_cap_), stage_end - done);
    cuda_check(cudaMemcpyAsync(tokens_dev_, pinned_tok_ + (done - stage_base), (size_t)M * sizeof(int), cudaMemcpyHostToDevice, stream_), "h2d tokens");
    check(pk_iota_int(pos_dev_, M, nullptr, pos_, stream_), "iota");
    if (M <= kSmallRows) run_small(M, false);
    else run_chunk(M);
    if (opt_.mtp) {
      // prime the predictor: row i pairs the target's hidden of position i with the token of position i + 1; the
      // very last row takes the token the target has just produced
      if (M > 1) check(pk_copy_int(tokens_dev_ + 1, mtp_tok_dev_, M - 1, stream_), "shift tokens");
      if (done + M < n) check(pk_iota_int(mtp_tok_dev_ + (M - 1), 1, nullptr, tokens_host[done + M], stream_), "next token");
      else check(pk_copy_int(next_tok_dev_, mtp_tok_dev_ + (M - 1), 1, stream_), "first output token");
      mtp_forward(M, tgt_hid_, pos_);
    }
    pos_ += M;
    done += M;
  }
  cuda_check(cudaMemcpyAsync(pinned_tok_, next_tok_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h token");
  if (opt_.mtp) cuda_check(cudaMemcpyAsync(pinned_mtp_, mtp_next_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h draft");
  cuda_check(cudaEventRecord(ev1_, stream_), "event");
  queue_status_read();
  cuda_check(cudaStreamSynchronize(stream_), "prefill");
  raise_if_step_failed("prefill");
  float ms = 0;
  cudaEventElapsedTime(&ms, ev0_, ev1_);
  timings_.prefill_ms = ms;
  timings_.prefill_tokens = n;
  timings_.kernel_launches += launches_ - l0;
  history_.insert(history_.end(), tokens_host, tokens_host + n);
  last_token_ = pinned_tok_[0];
  if (opt_.mtp) {
    mtp_ready_ = true;
    mtp_seed_token_ = last_token_;
    mtp_next_token_ = pinned_mtp_[0];
  }
  return last_token_;
}

// The persistent kernel's view of the model: one descriptor per layer in device memory and a parameter block with
// the activation buffers, the grid barrier words and every rank's slots and flags.
void QwenEngine::build_persistent() {
  persistent_built_ = true;
  persistent_ok_ = false;
  int mode = opt_.persistent_decode;
  if (const char* v = getenv("POCKET_DECODE_PERSISTENT")) mode = atoi(v);
  // The predictor's verify rows run on the per-projection kernels; plain decode then uses them too, so that both
  // see the same rounding and speculative tokens equal plain ones.
  if (mode == 0 || (mode < 0 && opt_.mtp) || nccl_mode_) return;   // NCCL collectives sit between launches: one launch per projection
  if (!peers_set_) throw std::runtime_error("peer arenas not registered");
  int max_k = hidden_, max_rows = vocab_l_;
  auto lin = [&](const Fp8Linear& l) {
    PkDecLinear d{};
    d.w = l.w;
    d.scale = l.scale;
    d.N = l.N;
    d.K = l.K;
    d.elem = 1;
    max_k = std::max(max_k, l.K);
    max_rows = std::max(max_rows, l.N);
    return d;
  };
  std::vector<PkDecLayer> hl(cfg_.num_layers);
  for (int i = 0; i < cfg_.num_layers; ++i) {
    const QwenLayer& L = layers_[i];
    PkDecLayer& d = hl[i];
    memset(&d, 0, sizeof d);
    d.full = L.full ? 1 : 0;
    d.input_norm = L.input_norm;
    d.post_norm = L.post_norm;
    if (L.full) {
      d.lin[0] = lin(L.qkv);
      d.lin[1].elem = 2;
      d.lin[1].K = hidden_;
      d.lin[2] = lin(L.o_proj);
      d.q_norm = L.q_norm;
      d.k_norm = L.k_norm;
      d.kcache = L.kcache;
      d.vcache = L.vcache;
      d.kscale = L.kscale;
      d.vscale = L.vscale;
    } else {
      d.lin[0] = lin(L.in_proj);
      d.lin[1].w = L.in_proj_ab;
      d.lin[1].N = 2 * vh_l_;
      d.lin[1].K = hidden_;
      d.lin[1].elem = 2;
      d.lin[2] = lin(L.out_proj);
      d.conv_w = L.conv_w;
      d.conv_state = L.conv_state;
      d.A_log = L.A_log;
      d.dt_bias = L.dt_bias;
      d.lin_norm = L.lin_norm;
      d.lin_state = L.lin_state;
    }
    d.lin[3] = lin(L.gate_up);
    d.lin[4] = lin(L.down);
  }
  if (dec_layers_dev_ == nullptr) {
    dec_layers_dev_ = (PkDecLayer*)dalloc(hl.size() * sizeof(PkDecLayer));
    dec_o_raw_ = (float*)dalloc((size_t)std::max(vd_l_, 1) * sizeof(float));
    dec_cand_val_ = (float*)dalloc((size_t)sm_count_ * sizeof(float));
    dec_cand_idx_ = (int*)dalloc((size_t)sm_count_ * sizeof(int));
    dec_bar_ = (unsigned long long*)dalloc(2 * sizeof(unsigned long long));
    cuda_check(cudaMemset(dec_bar_, 0, 2 * sizeof(unsigned long long)), "memset");
  }
  cuda_check(cudaMemcpy(dec_layers_dev_, hl.data(), hl.size() * sizeof(PkDecLayer), cudaMemcpyHostToDevice), "decode table");

  PkDecParams& p = dec_params_;
  memset(&p, 0, sizeof p);
  p.layers = dec_layers_dev_;
  p.n_layers = cfg_.num_layers;
  p.hidden = hidden_;
  p.inter_l = inter_l_;
  p.vocab_l = vocab_l_;
  p.vocab_start = vocab_start_;
  p.hq_l = hq_l_;
  p.hkv_l = hkv_l_;
  p.kh_l = kh_l_;
  p.vh_l = vh_l_;
  p.ld_proj = ld_proj_;
  p.eps = (float)cfg_.rms_norm_eps;
  p.rotary_dim = cfg_.rotary_dim();
  p.theta = (float)cfg_.rope_theta;
  p.ctx_cap = opt_.max_context;
  p.max_splits = std::min(64, kSmallRows * opt_.decode_splits);
  p.window = opt_.attention_window;
  p.sink = opt_.attention_sink;
  p.attn_gate = cfg_.attn_output_gate ? 1 : 0;
  p.kv_fp8 = opt_.kv_fp8 ? 1 : 0;
  p.max_k = max_k;
  p.max_rows = max_rows;
  p.embed = embed_;
  p.final_norm = final_norm_;
  p.lm_head.w = lm_head_;
  p.lm_head.scale = nullptr;
  p.lm_head.N = vocab_l_;
  p.lm_head.K = hidden_;
  p.lm_head.elem = 2;
  p.token = tokens_dev_;
  p.pos = pos_dev_;
  p.hidden_buf[0] = hidden_buf_[0];
  p.hidden_buf[1] = hidden_buf_[1];
  p.proj = proj_;
  p.o_raw = dec_o_raw_;
  p.attn_out = attn_out_;
  p.mlp_h = mlp_h_;
  p.attn_ws = attn_ws_;
  p.logits = logits_;
  p.norm_out = opt_.mtp ? tgt_hid_ : nullptr;
  p.cand_val = dec_cand_val_;
  p.cand_idx = dec_cand_idx_;
  p.next_tok = next_tok_dev_;
  p.out_tokens = out_tokens_dev_;
  p.out_counter = out_counter_dev_;
  p.out_cap = out_cap_;
  p.bar_count = dec_bar_;
  p.bar_base = dec_bar_ + 1;
  p.world = opt_.tp_world;
  p.rank = opt_.tp_rank;
  for (int r = 0; r < opt_.tp_world; ++r) {
    for (int s = 0; s < 2; ++s) p.slot[s][r] = (uint2*)((char*)peers_[r] + off_ll_[s]);
    p.cand_val_peer[r] = (float*)((char*)peers_[r] + off_cval_);
    p.cand_idx_peer[r] = (int*)((char*)peers_[r] + off_cidx_);
    p.cand_flag[r] = (uint32_t*)((char*)peers_[r] + off_cflag_);
  }
  // two-stage sums (POCKET_DECODE_TWO_STAGE=1): off by default. Measured at TP8 on the 27B shape: 4.83 ms per token with it,
  // 4.58 without; the second hop inside the GPU costs more than reading 8 x 40 KB of words per block saves.
  {
    int two = 0;
    if (const char* v = getenv("POCKET_DECODE_TWO_STAGE")) two = atoi(v) != 0 && opt_.tp_world > 1;
    p.two_stage = two;
    p.red[0] = p.red[1] = nullptr;
    if (two) {
      if (dec_red_ == nullptr) {
        dec_red_ = dalloc((size_t)2 * hidden_ * sizeof(uint2));
        cuda_check(cudaMemset(dec_red_, 0, (size_t)2 * hidden_ * sizeof(uint2)), "memset");
      }
      p.red[0] = (uint2*)dec_red_;
      p.red[1] = (uint2*)dec_red_ + hidden_;
    }
  }
  p.epoch = (const uint32_t*)((char*)arena_ + off_epoch_);
  p.sites_per_epoch = sites_per_epoch_;
  p.status = (uint32_t*)((char*)arena_ + off_status_);
  p.timeout_us = opt_.comm_timeout_us;
  if (const char* t = getenv("POCKET_DECODE_TRACE")) {
    if (t[0] == '1' && dec_dbg_ == nullptr) {
      dec_dbg_cap_ = 32 * cfg_.num_layers + 64;
      dec_dbg_ = (unsigned long long*)dalloc((size_t)dec_dbg_cap_ * 2 * sizeof(unsigned long long));
    }
  }
  if (dec_dbg_) cuda_check(cudaMemset(dec_dbg_, 0, (size_t)dec_dbg_cap_ * 2 * sizeof(unsigned long long)), "memset");
  p.dbg = dec_dbg_;
  p.dbg_cap = dec_dbg_cap_;
  dec_grid_ = sm_count_;
  persistent_ok_ = pk_decode_persistent_smem(&p, dec_grid_) != 0;
  if (!persistent_ok_ && mode > 0) throw std::runtime_error("the persistent decode kernel does not take these shapes");
}

void QwenEngine::set_persistent_decode(int mode) {
  opt_.persistent_decode = mode;
  persistent_built_ = false;
  if (decode_graph_) {
    cudaStreamSynchronize(stream_);
    cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
}

int QwenEngine::copy_decode_trace(unsigned long long* out, int cap) {
  if (dec_dbg_ == nullptr) return 0;
  cuda_check(cudaStreamSynchronize(stream_), "sync");
  const int n = std::min(cap, dec_dbg_cap_);
  cuda_check(cudaMemcpy(out, dec_dbg_, (size_t)n * 2 * sizeof(unsigned long long), cudaMemcpyDeviceToHost), "trace");
  int used = 0;
  while (used < n && out[2 * used + 1] != 0ull) ++used;
  return used;
}

void QwenEngine::enqueue_decode_step() {
  if (!persistent_built_) build_persistent();
  if (persistent_ok_) {
    check(pk_decode_persistent_prepare((uint32_t*)((char*)arena_ + off_epoch_), next_tok_dev_, tokens_dev_, dec_bar_, dec_bar_ + 1, stream_),
          "decode prepare");
    check(pk_decode_persistent_step(&dec_params_, dec_grid_, stream_), "persistent decode step");
    return;
  }
  check(pk_copy_int(next_tok_dev_, tokens_dev_, 1, stream_), "copy token");
  run_small(1, true);
  check(pk_add_int(pos_dev_, 1, 1, stream_), "advance pos");
  check(pk_store_token(next_tok_dev_, out_tokens_dev_, out_counter_dev_, out_cap_, stream_), "store token");
}

// ---------------------------------------------------------------------------------------
// prefix reuse across requests

void QwenEngine::clear_prefix_cache() {
  for (auto& st : stored_) {
    free_snapshot(*st.snap);
  }
  stored_.clear();
  prefix_stats_.snapshots = 0;
  prefix_stats_.snapshot_bytes = 0;
}

void QwenEngine::drop_states_after(int pos) {
  for (size_t i = 0; i < stored_.size();) {
    if (stored_[i].snap->pos > pos) {
      free_snapshot(*stored_[i].snap);
      stored_.erase(stored_.begin() + (long)i);
    } else {
      ++i;
    }
  }
}

void QwenEngine::store_state() {
  if (opt_.max_snapshots <= 0 || pos_ <= 0) return;
  for (auto& st : stored_)
    if (st.snap->pos == pos_) {   // same position again (a repeated prompt): refresh its age
      st.stamp = ++stamp_;
      return;
    }
  if ((int)stored_.size() >= opt_.max_snapshots) {
    std::vector<int> positions;
    std::vector<long long> stamps;
    for (auto& st : stored_) {
      positions.push_back(st.snap->pos);
      stamps.push_back(st.stamp);
    }
    const int v = snapshot_to_evict(positions, stamps, opt_.snapshot_interval);
    if (v >= 0) {
      free_snapshot(*stored_[(size_t)v].snap);
      stored_.erase(stored_.begin() + v);
    }
  }
  StoredState st;
  st.snap = snapshot(false);
  st.stamp = ++stamp_;
  stored_.push_back(std::move(st));
}

int QwenEngine::prefill_cached(const int* tokens_host, int n) {
  if (n < 1) throw std::runtime_error("prefill: empty prompt");
  QwenPrefixStats& ps = prefix_stats_;
  ps.prompt_tokens = n;
  if (!opt_.prefix_cache) {
    reset();
    ps.reused_tokens = 0;
    ps.computed_tokens = n;
    ps.matched_tokens = 0;
    ps.resume_source = "empty";
    return prefill(tokens_host, n);
  }
  std::vector<int> positions;
  for (auto& st : stored_) positions.push_back(st.snap->pos);
  const PrefixDecision d = plan_prefix(history_, pos_, positions, tokens_host, n);
  ps.matched_tokens = d.matched;
  ps.resume_source = prefix_source_name(d.source);
  if (d.source == PrefixDecision::kLive) {
    // continue where the engine stands; the pending token (generated, not yet consumed) is simply dropped
  } else if (d.source == PrefixDecision::kSnapshot) {
    StoredState& st = stored_[(size_t)d.snapshot_index];
    st.stamp = ++stamp_;
    restore(*st.snap);
  } else {
    // nothing reusable: the stored states describe another sequence from position 0 on
    const std::vector<int> keep;
    (void)keep;
    clear_prefix_cache();
    reset();
  }
  drop_states_after(d.resume_pos);   // positions past the resume point are about to be overwritten
  if (d.resume_pos > 0) ++ps.hits; else ++ps.misses;
  ps.reused_tokens = d.resume_pos;
  ps.computed_tokens = n - d.resume_pos;
  int first = -1;
  double ms = 0;
  int from = d.resume_pos;
  for (int to : snapshot_points(d.resume_pos, n, opt_.snapshot_interval)) {
    // the last piece ends at the request boundary; its state is stored too, for prompts that share this one as a prefix
    first = prefill(tokens_host + from, to - from);
    ms += timings_.prefill_ms;
    store_state();
    from = to;
  }
  timings_.prefill_ms = ms;
  timings_.prefill_tokens = n - d.resume_pos;
  ps.snapshots = (int)stored_.size();
  unsigned long long bytes = 0;
  for (auto& L : layers_)
    if (!L.full) bytes += (unsigned long long)vh_l_ * kHeadDim * kHeadDim * sizeof(float) + (unsigned long long)conv_c_l_ * 3 * sizeof(float);
  ps.snapshot_bytes = bytes * stored_.size();
  return first;
}

void QwenEngine::capture_decode_graph() {
  cudaGraph_t g = nullptr;
  if (!persistent_built_) build_persistent();   // allocations and copies stay outside the capture
  const long long l0 = launches_;
  cuda_check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "begin capture");
  try {
    cur_ = 0;
    enqueue_decode_step();
  } catch (...) {
    cudaStreamEndCapture(stream_, &g);
    if (g) cudaGraphDestroy(g);
    throw;
  }
  cuda_check(cudaStreamEndCapture(stream_, &g), "end capture");
  graph_nodes_ = launches_ - l0;
  launches_ = l0;
  cuda_check(cudaGraphInstantiate(&decode_graph_, g, 0), "graph instantiate");
  cudaGraphDestroy(g);
}

void QwenEngine::decode(int steps, int* out_host, bool sync_each_step) {
  if (last_token_ < 0) throw std::runtime_error("decode before prefill");
  if (steps < 1) return;
  if (pos_ + steps + 1 > opt_.max_context) throw std::runtime_error("decode: exceeds max_context");
  if (steps > out_cap_) throw std::runtime_error("decode: too many steps in one call");
  // The hidden ping-pong index must be the same at capture and at every replay: a forward
  // flips it an even number of times only if it starts from a fixed buffer.
  cur_ = 0;
  if (opt_.use_cuda_graph && decode_graph_ == nullptr) capture_decode_graph();
  cur_ = 0;
  cuda_check(cudaMemsetAsync(out_counter_dev_, 0, sizeof(int), stream_), "memset");
  check(pk_iota_int(pos_dev_, 1, nullptr, pos_, stream_), "iota");
  --launches_;
  cuda_check(cudaEventRecord(ev0_, stream_), "event");
  const long long l0 = launches_;
  for (int s = 0; s < steps; ++s) {
    if (decode_graph_) {
      cuda_check(cudaGraphLaunch(decode_graph_, stream_), "graph launch");
      launches_ += graph_nodes_;
    } else {
      cur_ = 0;
      enqueue_decode_step();
    }
    if (sync_each_step) {
      cuda_check(cudaMemcpyAsync(pinned_tok_ + s, next_tok_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h");
      cuda_check(cudaStreamSynchronize(stream_), "decode step");
    }
  }
  if (!sync_each_step)
    cuda_check(cudaMemcpyAsync(pinned_tok_, out_tokens_dev_, (size_t)steps * sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h");
  cuda_check(cudaEventRecord(ev1_, stream_), "event");
  queue_status_read();
  cuda_check(cudaStreamSynchronize(stream_), "decode");
  raise_if_step_failed("decode");
  float ms = 0;
  cudaEventElapsedTime(&ms, ev0_, ev1_);
  timings_.decode_ms = ms;
  timings_.decode_tokens = steps;
  timings_.kernel_launches += launches_ - l0;
  pos_ += steps;
  // consumed by these steps: the token that was pending, then every new token but the last
  history_.push_back(last_token_);
  history_.insert(history_.end(), pinned_tok_, pinned_tok_ + (steps - 1));
  last_token_ = pinned_tok_[steps - 1];
  mtp_ready_ = false;   // the predictor has not seen these positions
  mtp_pos_ = pos_;
  tgt_rows_ = 1;
  if (out_host) memcpy(out_host, pinned_tok_, (size_t)steps * sizeof(int));
}

void QwenEngine::forward_rows(const int* tokens_host, int M, int* out_tokens_host) {
  for (int t = 0; t < M; ++t)
    if (tokens_host[t] < 0 || tokens_host[t] >= cfg_.vocab_size) throw std::runtime_error("forward_rows: token id outside the vocabulary");
  if (M < 1 || M > kSmallRows) throw std::runtime_error("forward_rows: 1..8 rows");
  if (pos_ + M + 1 > opt_.max_context) throw std::runtime_error("forward_rows: exceeds max_context");
  memcpy(pinned_tok_, tokens_host, (size_t)M * sizeof(int));
  cuda_check(cudaMemcpyAsync(tokens_dev_, pinned_tok_, (size_t)M * sizeof(int), cudaMemcpyHostToDevice, stream_), "h2d");
  check(pk_iota_int(pos_dev_, M, nullptr, pos_, stream_), "iota");
  run_small(M, true);
  cuda_check(cudaMemcpyAsync(pinned_tok_, next_tok_dev_, (size_t)M * sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h");
  // decode() continues from slot 0 of the token buffer
  if (M > 1) check(pk_copy_int(next_tok_dev_ + (M - 1), next_tok_dev_, 1, stream_), "copy token");
  queue_status_read();
  cuda_check(cudaStreamSynchronize(stream_), "forward_rows");
  raise_if_step_failed("forward_rows");
  pos_ += M;
  history_.insert(history_.end(), tokens_host, tokens_host + M);
  last_token_ = pinned_tok_[M - 1];
  mtp_ready_ = false;
  mtp_pos_ = pos_;
  if (out_tokens_host) memcpy(out_tokens_host, pinned_tok_, (size_t)M * sizeof(int));
}

// ---------------------------------------------------------------------------------------
// multi-token predictor and speculative decode

void QwenEngine::mtp_forward(int M, const void* hidden_rows, int position) {
  mtp_in_ = hidden_rows;
  check(pk_iota_int(mtp_pos_dev_, M, nullptr, position, stream_), "iota");
  if (M <= kSmallRows) run_small(M, false, true);
  else run_chunk(M, true);
  mtp_pos_ = position + M;
}

int QwenEngine::mtp_row(int token, const void* hidden_row, int position) {
  check(pk_iota_int(mtp_tok_dev_, 1, nullptr, token, stream_), "token");
  mtp_forward(1, hidden_row, position);
  cuda_check(cudaMemcpyAsync(pinned_mtp_, mtp_next_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_), "d2h draft");
  queue_status_read();
  cuda_check(cudaStreamSynchronize(stream_), "mtp row");
  raise_if_step_failed("predictor row");
  mtp_seed_token_ = token;
  mtp_next_token_ = pinned_mtp_[0];
  mtp_ready_ = true;
  return mtp_next_token_;
}

// Drafts after `input_token` (generated, not yet consumed by the target at position pos_). The first draft is the
// boundary row's prediction when that row was given this token, else the row is rebuilt from the target's last hidden;
// further drafts recurse on the predictor's own output.
void QwenEngine::draft_tokens(int count, int input_token, int produced, std::vector<int>& drafts, QwenSpecStats& st) {
  drafts.clear();
  if (!(mtp_ready_ && mtp_seed_token_ == input_token)) {
    const char* last = (const char*)tgt_hid_ + (size_t)std::max(tgt_rows_ - 1, 0) * hidden_ * 2;
    mtp_row(input_token, last, pos_ - 1);
    ++st.predictor_rows;
  }
  auto pick = [&](int predicted) {
    const size_t at = (size_t)produced + drafts.size();
    return at < replay_.size() ? replay_[at] : predicted;
  };
  drafts.push_back(pick(mtp_next_token_));
  while ((int)drafts.size() < count) {
    const int next = mtp_row(drafts.back(), mtp_seed_, mtp_pos_);
    ++st.predictor_rows;
    drafts.push_back(pick(next));
  }
}

void QwenEngine::spec_decode(int steps, int max_draft, int* out_host, QwenSpecStats* stats_out) {
  if (!opt_.mtp) throw std::runtime_error("spec_decode: the engine was built without the multi-token predictor");
  if (last_token_ < 0) throw std::runtime_error("spec_decode before prefill");
  if (steps < 1) return;
  if (pos_ + steps + kSmallRows + 1 > opt_.max_context) throw std::runtime_error("spec_decode: exceeds max_context");
  max_draft = std::max(1, std::min(max_draft, kSmallRows - 1));
  QwenSpecStats st;
  if (!txn_) txn_ = snapshot(false);
  std::vector<int> out, drafts, rows(kSmallRows), preds(kSmallRows);
  out.reserve(steps + kSmallRows);
  cuda_check(cudaEventRecord(ev0_, stream_), "event");
  const long long l0 = launches_;
  int K = 1;
  while ((int)out.size() < steps) {
    const int remaining = steps - (int)out.size();
    if (remaining == 1) {
      int t = last_token_, next = 0;
      forward_rows(&t, 1, &next);
      out.push_back(next);
      ++st.plain_steps;
      continue;
    }
    const int k = drafts_this_round(K, remaining, max_draft);
    const int committed = pos_, input = last_token_;
    draft_tokens(k, input, (int)out.size(), drafts, st);
    update_snapshot(*txn_);
    rows[0] = input;
    for (int i = 0; i < k; ++i) rows[i + 1] = drafts[i];
    forward_rows(rows.data(), k + 1, preds.data());
    int correct = 0;
    while (correct < k && preds[correct] == drafts[correct]) ++correct;
    int bonus = preds[correct];
    ++st.rounds;
    st.proposed += k;
    if (correct < k) {
      // rows after the first mismatch have advanced the recurrent state: rewind and replay the accepted prefix.
      // The replay is what the state ends up holding, so its picks are the ones handed out. A pass over fewer rows may
      // run other kernels than the verify pass (1-2 rows stream through the rings, 3-8 through registers) and add in a
      // different order: on a near-tie a pick can fall the other way. Then only the prefix both passes agree on is kept
      // and the replay runs again over it (each round is shorter, so this ends).
      for (;;) {
        ++st.rollbacks;
        st.replay_tokens += correct + 1;
        restore(*txn_);
        forward_rows(rows.data(), correct + 1, preds.data());
        int agree = 0;
        while (agree < correct && preds[agree] == drafts[agree]) ++agree;
        if (agree == correct) break;
        correct = agree;
      }
      bonus = preds[correct];
    }
    st.accepted += correct;
    // pos_ == committed + correct + 1; the target's hidden of the last committed row is row `correct` of tgt_hid_.
    // Rebind the predictor's boundary row to the bonus token (not yet consumed by the target).
    mtp_row(bonus, (const char*)tgt_hid_ + (size_t)correct * hidden_ * 2, committed + correct);
    ++st.predictor_rows;
    for (int i = 0; i < correct; ++i) out.push_back(drafts[i]);
    out.push_back(bonus);
    last_token_ = bonus;
    K = next_draft_len(K, k, correct, max_draft);
  }
  // a round may overshoot by nothing: k <= remaining - 1, so at most `remaining` tokens are added
  cuda_check(cudaEventRecord(ev1_, stream_), "event");
  cuda_check(cudaStreamSynchronize(stream_), "spec_decode");
  float ms = 0;
  cudaEventElapsedTime(&ms, ev0_, ev1_);
  timings_.decode_ms = ms;
  timings_.decode_tokens = steps;
  timings_.kernel_launches += launches_ - l0;
  if (out_host) memcpy(out_host, out.data(), (size_t)steps * sizeof(int));
  if (stats_out) *stats_out = st;
}

}  // namespace pk

// Native inference engine for the hybrid Gated-DeltaNet / GQA decoder: weights (FP8
// block-scaled Safetensors or random init), KV + recurrent state, chunked prefill, CUDA
// graph decode, tensor parallelism over peer memory. Counterpart of the reference's
// QwenEngine (cpp_engine/src/qwen_engine.cpp:295-557, 910-1303, 1733-2270) with a
// different execution model: one fused launch per projection, collectives folded into the
// producing and consuming kernels, and a captured graph per decode step.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../common/pk_comm_types.h"
#include "../kernels/pk_decode_persistent.h"
#include "nccl_comm.hpp"
#include "qwen_config.hpp"

namespace pk {

struct QwenEngineOptions {
  int tp_rank = 0;
  int tp_world = 1;
  int device = 0;
  int max_context = 4096;
  int prefill_chunk = 512;
  int decode_splits = 8;       // context splits of the decode attention kernel
  bool use_cuda_graph = true;
  int attention_window = 0;    // 0 = full attention
  int attention_sink = 0;
  uint32_t comm_timeout_us = 2000000;
  // bf16 copies of the FP8 linears for the tensor-core prefill path (the decode path keeps streaming FP8):
  // -1 = when HBM has room for them (twice the FP8 bytes plus a reserve), 0 = never, 1 = always.
  // POCKET_PREFILL_SHADOW in the environment overrides.
  int prefill_bf16_shadow = -1;
  // Which GEMM the many-row (prefill, verify) path uses on the FP8 linears:
  //   -1  automatic: the native FP8 kernel with two-term activations, unless prefill_bf16_shadow == 1 asks for the copies
  //    0  weights decoded to bf16 inside shared memory (128 x 128 tiles), bf16 activations
  //    1  bf16 copies of the weights in HBM (see prefill_bf16_shadow), bf16 activations
  //    2  native FP8 tensor-core math on the stored codes, activations as two E4M3 terms per value (bf16-like accuracy)
  //    3  native FP8, one E4M3 term per activation (fastest; activations carry 4 significant bits)
  // POCKET_PREFILL_GEMM = umma | shadow | fp8x2 | fp8 in the environment overrides.
  int prefill_gemm = -1;
  // Multi-token predictor (`mtp.*` tensors: two input norms, fc, one full-attention layer, norm) for speculative decoding.
  bool mtp = false;
  // Single-row decode steps as one persistent cooperative kernel per token (weights ring that never drains, grid and
  // peer-flag barriers instead of kernel boundaries): -1 = when the shapes fit its shared-memory plan, 0 = never
  // (one launch per projection), 1 = required. POCKET_DECODE_PERSISTENT in the environment overrides.
  int persistent_decode = -1;
  // Exact prefix reuse across sequential requests (prefill_cached): the KV cache is position indexed and stays, the
  // recurrent state continues live or rolls back to a stored copy. Copies are taken every `snapshot_interval` tokens
  // of a prefill (0: only at request boundaries), at most `max_snapshots` of them.
  // FP8 KV cache: E4M3 codes with one fp32 scale per 64 channels (amax / 448) instead of bf16; a little over half the bytes
  // per position (reference: --kv-cache-dtype fp8, cpp_engine/src/qwen_engine.cpp:410-438).
  bool kv_fp8 = false;
  bool prefix_cache = true;
  int snapshot_interval = 4096;
  int max_snapshots = 82;
};

// Outcome of the last prefill_cached().
struct QwenPrefixStats {
  int reused_tokens = 0;        // prompt tokens that needed no forward pass
  int computed_tokens = 0;
  int prompt_tokens = 0;
  int matched_tokens = 0;       // common prefix with the consumed sequence, before rounding to a resume point
  const char* resume_source = "empty";   // "empty", "live" or "snapshot"
  int snapshots = 0;
  unsigned long long snapshot_bytes = 0;
  long long hits = 0, misses = 0;
};

// Counters of spec_decode().
struct QwenSpecStats {
  long long rounds = 0;         // draft + verify rounds
  long long proposed = 0;       // draft tokens sent to the target
  long long accepted = 0;       // of those, matched by the target
  long long rollbacks = 0;      // rounds that restored the recurrent state and replayed
  long long replay_tokens = 0;
  long long plain_steps = 0;    // tokens produced by single-row decode
  long long predictor_rows = 0; // rows run through the predictor (priming excluded)
};

struct Fp8Linear {
  uint8_t* w = nullptr;   // [N, K] e4m3
  float* scale = nullptr; // [ceil(N/128), ceil(K/128)]
  void* wb = nullptr;     // optional bf16 [N, K] copy used by the prefill GEMM
  int N = 0, K = 0;
};

struct QwenLayer {
  bool full = false;
  float* input_norm = nullptr;
  float* post_norm = nullptr;
  // linear attention
  Fp8Linear in_proj;           // q|k|v|z rows of this rank
  void* in_proj_ab = nullptr;  // bf16 [2*Hv_l, hidden]
  float* conv_w = nullptr;     // [C_l, 4]
  float* A_log = nullptr;
  float* dt_bias = nullptr;
  float* lin_norm = nullptr;
  Fp8Linear out_proj;
  float* lin_state = nullptr;  // [Hv_l, 128, 128]
  float* conv_state = nullptr; // [C_l, 3]
  // full attention
  Fp8Linear qkv;
  float* q_norm = nullptr;
  float* k_norm = nullptr;
  Fp8Linear o_proj;
  void* kcache = nullptr;      // bf16 [Hkv_l, ctx, 128], or E4M3 codes [Hkv_l, ctx, 128] with the FP8 cache
  void* vcache = nullptr;
  float* kscale = nullptr;     // FP8 cache: [Hkv_l, ctx, 2]
  float* vscale = nullptr;
  // mlp
  Fp8Linear gate_up;
  Fp8Linear down;
};

// Thrown by the engine's step functions when a bounded device wait ran out during the step (this rank's or, learned
// through the sampler exchange, another rank's): the step's tokens are not returned, the status words are cleared and
// the request state is undefined until reset().
struct CommTimeout : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct QwenTimings {
  double prefill_ms = 0;      // device time of the last prefill
  double decode_ms = 0;       // device time of the last decode run
  int prefill_tokens = 0;
  int decode_tokens = 0;
  long long kernel_launches = 0;  // launches issued (graph nodes count once per replay)
};

class QwenEngine {
 public:
  QwenEngine(const QwenConfig& cfg, const QwenEngineOptions& opt);
  ~QwenEngine();
  QwenEngine(const QwenEngine&) = delete;
  QwenEngine& operator=(const QwenEngine&) = delete;

  // Weights: from a checkpoint directory / file (this rank's shard is cut on the host), or
  // N(0, sigma) values quantised on the device.
  void load_safetensors(const std::string& path);
  void init_random(uint64_t seed, float sigma);

  // Peer memory. The arena holds the all-reduce slots, flags and sampler candidates; its
  // address is exported to the other ranks, and theirs are registered here.
  void* comm_arena() const { return arena_; }
  size_t comm_arena_bytes() const { return arena_bytes_; }
  void set_peer_arenas(void* const* arenas);  // [tp_world], entry tp_rank may be own

  void reset();
  // Runs the prompt in chunks; returns the first generated token (greedy).
  int prefill(const int* tokens_host, int n);
  // A new request: reuses the longest prefix of `tokens_host` that the engine has already consumed (see prefix_plan.hpp),
  // runs the rest, and stores recurrent-state copies on the way. With the cache switched off: reset() + prefill().
  int prefill_cached(const int* tokens_host, int n);
  const QwenPrefixStats& prefix_stats() const { return prefix_stats_; }
  void clear_prefix_cache();
  void configure_prefix_cache(bool enable, int snapshot_interval, int max_snapshots) {
    clear_prefix_cache();
    opt_.prefix_cache = enable;
    opt_.snapshot_interval = snapshot_interval;
    opt_.max_snapshots = max_snapshots;
  }
  // Greedy decode of `steps` tokens following the last generated one. Tokens are
  // written to out_host (may be null). `sync_each_step` reads every token back as soon as
  // its step ends (streaming); otherwise one read at the end.
  void decode(int steps, int* out_host, bool sync_each_step);
  // Verify-style forward over M (<= 8) given tokens at consecutive positions; returns
  // the greedy token after each row. State advances by M tokens.
  void forward_rows(const int* tokens_host, int M, int* out_tokens_host);
  // Greedy decode of `steps` tokens with drafts from the multi-token predictor, verified by the target in one
  // multi-row pass per round. The tokens equal those of decode(). Draft length starts at 1, doubles after a
  // fully accepted round up to `max_draft` (<= 7), and shrinks to max(1, min(K / 2, accepted + 1)) after a reject;
  // the last token comes from a plain step.
  void spec_decode(int steps, int max_draft, int* out_host, QwenSpecStats* stats);
  bool mtp_enabled() const { return opt_.mtp; }
  // The predictor's current pick for the token after last_token() (-1 when its boundary row is stale), and the fp32
  // logits behind it (this rank's vocabulary shard).
  int mtp_next_token() const { return mtp_ready_ ? mtp_next_token_ : -1; }
  void copy_mtp_logits(float* out_host);
  // Test hook: the known continuation (tokens that follow the first generated one). While set, spec_decode drafts
  // come from it instead of the predictor's picks (the predictor still runs, so its state stays consistent).
  void set_draft_replay(const int* tokens, int n) { replay_.assign(tokens, tokens + n); }

  int position() const { return pos_; }
  int last_token() const { return last_token_; }
  const QwenTimings& timings() const { return timings_; }
  uint32_t comm_status();
  void clear_comm_status();
  // fp32 logits of the last forward's final row: this rank's vocab shard.
  void copy_logits(float* out_host, int row);
  int vocab_local() const { return vocab_l_; }
  const QwenConfig& config() const { return cfg_; }
  const QwenEngineOptions& options() const { return opt_; }
  size_t weight_bytes() const { return weight_bytes_; }
  size_t shadow_bytes() const { return shadow_bytes_; }
  // Fallback collectives: joins the NCCL communicator of this tensor-parallel group now (every rank must call it;
  // rendezvous through files under `id_path`). After a bounded peer wait has run out, the failed step raises CommTimeout
  // as before and every later step runs its row-parallel sums, the prefill gathers and the sampler exchange through
  // NCCL instead of peer stores (role of the reference's NCCL path, cpp_engine/src/tp_comm.cpp:40-269, which is its only one).
  void enable_nccl_fallback(const std::string& id_path, int timeout_ms = 600000);
  void switch_to_nccl();               // also callable directly (a rank that learnt of the failure on the host)
  // Budget of every device-side wait on a peer (microseconds); takes effect with the next step.
  void set_comm_timeout_us(uint32_t us) {
    opt_.comm_timeout_us = us;
    set_persistent_decode(opt_.persistent_decode);   // the persistent kernel's parameter block and the graph carry the old budget
  }
  bool nccl_mode() const { return nccl_mode_; }
  // POCKET_CANARY=1 at construction puts 256 guard bytes before and behind every device buffer of the engine; returns the
  // index of the first buffer whose guards changed (-1: all intact, or canaries off).
  int verify_canaries(std::string* what = nullptr);
  bool canaries_enabled() const { return canaries_; }
  // Target taps for an external block drafter: the residual stream after each of the given layers, for every row of the
  // last forward (prefill chunk, verify rows, decode step), concatenated per row in the order given: [rows, n * hidden]
  // bf16. One rank only. Decode steps run one launch per projection while taps are on (the persistent kernel keeps the
  // residual stream in shared memory). Reference: cpp_engine/src/qwen_engine.cpp:1555-1726 (tap capture for DSpark).
  void set_tap_layers(const int* layers, int n);
  int tap_count() const { return (int)tap_layers_.size(); }
  int tap_rows() const { return tap_rows_; }                       // rows written by the last forward
  void copy_taps(void* dst_device, int first_row, int rows);       // [rows, n * hidden] bf16 into device memory
  int prefill_gemm_mode() const { return gemm_mode_; }
  // Before the weights are loaded or initialised: choose the many-row GEMM (QwenEngineOptions::prefill_gemm).
  void set_prefill_gemm(int mode) {
    if (shadow_bytes_ > 0 || act_q_ != nullptr) throw std::runtime_error("prefill GEMM already set up");
    opt_.prefill_gemm = mode;
  }   // 0 umma, 1 bf16 copies, 2 FP8 two terms, 3 FP8 one term
  size_t kv_cache_bytes() const { return kv_bytes_; }   // K and V of every full-attention layer, scales included
  // true once a decode step has been planned on the persistent kernel
  bool persistent_decode_active() const { return persistent_built_ && persistent_ok_; }
  // -1 automatic, 0 one launch per projection, 1 persistent kernel required; takes effect at the next decode.
  void set_persistent_decode(int mode);
  // Phase trace of the last persistent decode step (POCKET_DECODE_TRACE=1 when the engine first decodes): up to `cap`
  // pairs {phase id, ns}; returns the number of pairs.
  int copy_decode_trace(unsigned long long* out, int cap);
  cudaStream_t stream() const { return stream_; }

  // Recurrent-state snapshot (DeltaNet state + conv tails of every linear layer); KV is
  // position indexed and needs no copy. Used by speculative decoding and the prefix cache.
  struct Snapshot {
    std::vector<void*> bufs;
    std::vector<void*> kv;      // with_kv: K then V rows [0, pos) of every full-attention layer, [Hkv][pos][128] bf16
    int pos = 0;
    int last_token = 0;
  };
  // with_kv also copies the KV rows of positions [0, pos): needed when other requests run in between
  // (prefix cache); a speculative rewind inside one request does not need it.
  std::unique_ptr<Snapshot> snapshot(bool with_kv = false);
  void update_snapshot(Snapshot& s);   // re-capture into existing buffers (no allocation)
  void restore(const Snapshot& s);
  void free_snapshot(Snapshot& s);

 private:
  void alloc_buffers();
  void build_prefill_shadow();   // after the weights are in place
  void alloc_fp8(Fp8Linear& l, int N, int K);
  void* dalloc(size_t bytes, bool weight = false);
  // `mtp` runs the predictor stack (input = [norm(embed(mtp_tok_dev_)) | norm(mtp_in_)] through fc, one layer,
  // mtp.norm, logits of the last row) instead of the target.
  void run_small(int M, bool all_logits, bool mtp = false);    // M <= 8 rows: weight-streaming path
  void run_chunk(int M, bool mtp = false);                     // M > 8 rows: tensor-core path
  void sample_rows(int M, const float* logits, int* out);
  void mtp_forward(int M, const void* hidden_rows, int position);   // tokens already in mtp_tok_dev_
  int mtp_row(int token, const void* hidden_row, int position);     // one row; returns the predicted token
  void draft_tokens(int count, int input_token, int produced, std::vector<int>& drafts, QwenSpecStats& st);
  void alloc_layer(QwenLayer& L, bool full);
  void capture_decode_graph();
  void queue_status_read();        // async copy of the status words into pinned memory (before the step's last sync)
  void raise_if_step_failed(const char* what);   // after that sync
  void enqueue_decode_step();      // one greedy single-row step on stream_ (persistent kernel or per-projection launches)
  void build_persistent();         // descriptor table and parameters of the persistent decode kernel
  PkWait make_wait(int site) const;
  PkPush make_push(int site, bool big = false, int rows_per_rank = 0) const;
  float* slot_parts(int site, bool big = false) const;
  void check(int status, const char* what) const;

  QwenConfig cfg_;
  QwenEngineOptions opt_;
  cudaStream_t stream_ = nullptr;
  int sm_count_ = 148;

  // local (per rank) dims
  int hidden_, inter_l_, vocab_l_, vocab_start_;
  int hq_l_, hkv_l_, kh_l_, vh_l_, kd_l_, vd_l_, conv_c_l_;
  int ld_lin_, ld_full_, ld_proj_;
  int rows_cap_;  // rows of the activation buffers (prefill chunk)

  std::vector<QwenLayer> layers_;
  void* embed_ = nullptr;     // bf16 [vocab, hidden] (replicated)
  float* final_norm_ = nullptr;
  void* lm_head_ = nullptr;   // bf16 [vocab_l, hidden]
  size_t weight_bytes_ = 0;
  size_t alloc_bytes_ = 0;   // everything obtained through dalloc
  size_t shadow_bytes_ = 0;
  static constexpr size_t kCanaryBytes = 256;
  static constexpr int kCanaryByte = 0xC5;
  struct Guarded { char* base; size_t body, bytes; };
  std::vector<Guarded> guarded_;
  bool canaries_ = false;
  std::shared_ptr<NcclComm> nccl_;
  bool nccl_mode_ = false;
  int kernel_world() const { return nccl_mode_ ? 1 : opt_.tp_world; }   // what the kernels see as the number of slots to add
  int gemm_mode_ = 0;
  std::vector<int> tap_layers_;
  void* taps_ = nullptr;           // [rows_cap_, taps * hidden] bf16
  int tap_rows_ = 0;
  void capture_tap(int layer, const void* rows, int M);   // rows [M, hidden] bf16 = the residual stream after `layer`
  void* dec_red_ = nullptr;        // persistent decode, two-stage sums: [2][hidden] {value, sequence} words
  bool tc_prefill_attn_ = false;   // prefill chunks through pk_gqa_prefill_umma (bf16 cache, no window)
  void* act_q_ = nullptr;        // [2][rows_cap_ up to 128][K max] E4M3 terms of the GEMM input being multiplied
  float* act_scale_ = nullptr;   // [K max / 128][that row count]
  int act_rows_ = 0;
  size_t kv_bytes_ = 0;
  std::vector<void*> allocs_;

  // activations
  void* hidden_buf_[2] = {nullptr, nullptr};
  int cur_ = 0;
  void* xn_ = nullptr;
  void* proj_ = nullptr;
  void* attn_out_ = nullptr;
  void* q_buf_ = nullptr;
  void* mlp_h_ = nullptr;
  float* attn_ws_ = nullptr;
  float* lin_ws_ = nullptr;   // chunked DeltaNet scan workspace
  float* logits_ = nullptr;   // [8, vocab_l]
  float* cand_val_ = nullptr;
  int* cand_idx_ = nullptr;
  float* best_val_ = nullptr;
  int* best_idx_ = nullptr;
  int* tokens_dev_ = nullptr; // [rows_cap]
  int* pos_dev_ = nullptr;    // [rows_cap]
  int* next_tok_dev_ = nullptr;  // [8]
  int* out_tokens_dev_ = nullptr;
  int* out_counter_dev_ = nullptr;
  int out_cap_ = 0;
  uint32_t* gemm_status_ = nullptr;
  int* pinned_tok_ = nullptr;   // pinned host staging for token ids / results
  uint32_t* pinned_status_ = nullptr;   // [2]: peer-wait word of the arena, tensor-core GEMM word

  // comm arena layout (all inside arena_): slots, flags, sampler candidates, epoch, status
  void* arena_ = nullptr;
  size_t arena_bytes_ = 0;
  size_t off_bslot_[2];   // prefill-size slots [world][rows_cap][hidden] fp32
  size_t off_ll_[2];
  size_t off_agflag_[2] = {0, 0}, off_xn_ = 0;   // all-gather flags and the peer-visible buffer of normalised prefill rows
  void** xn_peer_dev_ = nullptr;   // unused on the device; host table below
  void* xn_peer_[PK_MAX_RANKS] = {nullptr};
  size_t off_slot_[2], off_flag_[2], off_cval_, off_cidx_, off_cflag_, off_epoch_, off_status_, off_counter_;
  void* peers_[PK_MAX_RANKS] = {nullptr};
  float** peer_cval_dev_ = nullptr;
  int** peer_cidx_dev_ = nullptr;
  bool peers_set_ = false;
  int sites_per_epoch_ = 0;
  int pending_site_ = -1;   // site whose partials still have to be added to the hidden state

  // multi-token predictor
  QwenLayer mtp_layer_;
  float* mtp_norm_e_ = nullptr;
  float* mtp_norm_h_ = nullptr;
  float* mtp_norm_ = nullptr;
  void* mtp_fc_ = nullptr;        // bf16 [hidden, 2 * hidden], replicated
  void* mtp_cat_ = nullptr;       // [rows_cap, 2 * hidden]
  void* tgt_hid_ = nullptr;       // [rows_cap, hidden]: the target's last forward after the final norm
  void* mtp_out_ = nullptr;       // [8, hidden]: the predictor's last forward after mtp.norm
  const void* mtp_in_ = nullptr;  // hidden rows the next predictor pass reads
  const void* mtp_seed_ = nullptr;  // row of mtp_out_ that seeds the next recursive draft
  int* mtp_tok_dev_ = nullptr;
  int* mtp_pos_dev_ = nullptr;
  float* mtp_logits_ = nullptr;   // [vocab_l]
  int* mtp_next_dev_ = nullptr;
  int* pinned_mtp_ = nullptr;
  int tgt_rows_ = 0;              // rows of tgt_hid_ written by the last target forward
  int mtp_pos_ = 0;
  int mtp_seed_token_ = -1;       // token the predictor's boundary row was given
  int mtp_next_token_ = -1;       // its prediction
  bool mtp_ready_ = false;
  std::unique_ptr<Snapshot> txn_;
  std::vector<int> replay_;

  // persistent decode kernel
  bool persistent_built_ = false;
  bool persistent_ok_ = false;
  PkDecParams dec_params_{};
  PkDecLayer* dec_layers_dev_ = nullptr;
  float* dec_o_raw_ = nullptr;
  float* dec_cand_val_ = nullptr;
  int* dec_cand_idx_ = nullptr;
  unsigned long long* dec_bar_ = nullptr;   // [0] arrival counter, [1] its value before the current step
  unsigned long long* dec_dbg_ = nullptr;   // phase trace of the last step (POCKET_DECODE_TRACE=1)
  int dec_dbg_cap_ = 0;
  int dec_grid_ = 0;

  // prefix reuse: tokens consumed so far (positions 0 .. pos_-1) and stored recurrent states
  std::vector<int> history_;
  struct StoredState {
    std::unique_ptr<Snapshot> snap;
    long long stamp = 0;
  };
  std::vector<StoredState> stored_;
  long long stamp_ = 0;
  QwenPrefixStats prefix_stats_;
  void store_state();            // copy of the recurrent state at pos_
  void drop_states_after(int pos);

  int pos_ = 0;
  int last_token_ = -1;
  cudaGraphExec_t decode_graph_ = nullptr;
  long long graph_nodes_ = 0;
  mutable long long launches_ = 0;
  QwenTimings timings_;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
};

}  // namespace pk

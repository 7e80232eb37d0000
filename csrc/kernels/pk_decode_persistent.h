// Persistent single-token decode of the hybrid Gated-DeltaNet / GQA decoder: one cooperative launch runs the
// whole token (embedding row, every layer, final norm, lm_head, greedy pick, sampler exchange between ranks).
//
// Why one kernel: at one row per step a projection streams a few MB per SM-group and the fixed cost of a
// kernel boundary (drain, launch, re-stage, re-fill the memory pipeline) is as long as the streaming itself.
// Here every warp owns a shared-memory ring that bulk asynchronous copies keep full of weight bytes. The order
// in which a warp will need weights is fixed for the whole token, so the ring keeps filling across phase
// boundaries, while the warp waits at a grid barrier or on the other ranks' flags. Phases are separated by
//   * a grid barrier (monotonic 64-bit arrival counter, bounded acquire poll), or
//   * after a row-parallel projection, nothing but the data itself: the epilogue stores every fp32 partial sum
//     into every rank's slot as an 8-byte word {value, sequence number of this site} (one store, so the number
//     cannot arrive without the value: no fence, no flag), and the next norm prologue polls the words it is about
//     to add until they carry the site's number. The all-reduce wait and the grid barrier are the same wait, on
//     one rank as on eight.
// Every wait has a time budget; on expiry the kernel records a status code, drains its copies and returns.
//
// Reference counterpart: the per-token loop of cpp_engine/src/qwen_engine.cpp:894-1303 (about 700 kernel
// launches and 129 NCCL all-reduces per token).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/pk_comm_types.h"

// One weight-streaming segment: rows of FP8 E4M3 codes with 128x128 fp32 block scales, or plain bf16 rows.
struct PkDecLinear {
  const void* w;
  const float* scale;   // fp8: [ceil(N/128)][ceil(K/128)]; null for bf16
  int N, K;
  int elem;             // bytes per weight: 1 (fp8) or 2 (bf16)
  int pad;
};

// lin[0] in_proj (q|k|v|z) or qkv, lin[1] in_proj a|b rows (bf16; N = 0 on full-attention layers),
// lin[2] out_proj / o_proj, lin[3] gate|up, lin[4] down.
struct PkDecLayer {
  int full;
  int pad;
  const float* input_norm;
  const float* post_norm;
  PkDecLinear lin[5];
  // Gated DeltaNet
  const float* conv_w;    // [C, 4]
  float* conv_state;      // [C, 3]
  const float* A_log;
  const float* dt_bias;
  const float* lin_norm;  // [128]
  float* lin_state;       // [Hv, 128, 128]
  // full attention
  const float* q_norm;
  const float* k_norm;
  void* kcache;           // bf16 [Hkv, ctx_cap, 128], or E4M3 codes (one byte per channel) with kv_fp8
  void* vcache;
  float* kscale;          // kv_fp8: fp32 [Hkv, ctx_cap, 2], one scale per 64 channels (amax / 448)
  float* vscale;
};

struct PkDecParams {
  const PkDecLayer* layers;   // device array
  int n_layers;
  int hidden, inter_l, vocab_l, vocab_start;
  int hq_l, hkv_l, kh_l, vh_l;
  int ld_proj;
  float eps;
  int rotary_dim;
  float theta;
  int ctx_cap;
  int max_splits;             // attention context splits the workspace allows
  int window, sink;
  int attn_gate;              // 1: sigmoid gate from the q projection
  int kv_fp8;                 // 1: FP8 KV cache
  int max_k;                  // largest K of any segment (sizes the staged activation row)
  int max_rows;               // largest row count of any segment (sizes the per-block accumulators)
  const void* embed;          // bf16 [vocab, hidden]
  const float* final_norm;
  PkDecLinear lm_head;
  // activations (device)
  const int* token;           // [1] token to feed
  int* pos;                   // [1] its position; incremented at the end of the step
  void* hidden_buf[2];        // bf16 [hidden] ping-pong residual stream
  void* proj;                 // bf16 [ld_proj]
  float* o_raw;               // fp32 [vh_l * 128]: DeltaNet output before the gated norm
  void* attn_out;             // bf16 [hq_l * 128]
  void* mlp_h;                // bf16 [inter_l]
  float* attn_ws;             // fp32 [hq_l][max_splits][130]
  float* logits;              // fp32 [vocab_l]
  void* norm_out;             // bf16 [hidden] normalised last hidden state (may be null)
  float* cand_val;            // [grid] per-block greedy candidates
  int* cand_idx;
  int* next_tok;              // [1]
  int* out_tokens;
  int* out_counter;
  int out_cap;
  // grid barrier
  unsigned long long* bar_count;        // arrival counter, only ever incremented
  const unsigned long long* bar_base;   // its value before this launch (written by the preparing kernel)
  // tensor parallelism (world == 1: the slot of "rank 0" is local and no flag is used)
  int world, rank;
  // peer r's partial-sum slots, by site parity: [world][hidden] words of {fp32 value, sequence number}. A producer
  // writes value and sequence number with ONE 8-byte store, so the arrival of the sequence number is the arrival of
  // the value: no fence, no separate flag, and the consumer's wait on the data is the only synchronisation of a site.
  uint2* slot[2][PK_MAX_RANKS];
  // two-stage sums on many ranks: this GPU's own {value, sequence} words of the reduced residual stream, by site parity
  // ([hidden] words each; null or two_stage == 0: every block adds the world's slots itself)
  uint2* red[2];
  int two_stage;
  float* cand_val_peer[PK_MAX_RANKS];   // peer r's sampler candidates: rows of 32 per rank (index row: entry 31 = status)
  int* cand_idx_peer[PK_MAX_RANKS];
  uint32_t* cand_flag[PK_MAX_RANKS];    // peer r's sampler flags [world]
  const uint32_t* epoch;                // local word, bumped once per forward
  uint32_t sites_per_epoch;
  uint32_t* status;                     // local status word, 0 = ok
  uint32_t timeout_us;
  // optional phase trace of block 0: pairs {phase id, %globaltimer ns} (null in normal use)
  unsigned long long* dbg;
  int dbg_cap;                          // pairs
};

// Status codes written to *status by the persistent kernel (besides PK_COMM_TIMEOUT from the peer waits).
#define PK_DEC_ERR_GRID_BARRIER 2u
#define PK_DEC_ERR_RING 3u

extern "C" {
// Epoch bump, token hand-over (next_tok -> token) and barrier base snapshot; stream-ordered before the step.
int pk_decode_persistent_prepare(uint32_t* epoch, const int* next_tok, int* token, const unsigned long long* bar_count,
                                 unsigned long long* bar_base, cudaStream_t stream);
// One token. `grid` must not exceed the number of blocks that can be resident at once (one per SM); returns
// PK_ERR_UNSUPPORTED when the shapes do not fit the kernel's shared-memory plan.
int pk_decode_persistent_step(const PkDecParams* params, int grid, cudaStream_t stream);
// Shared-memory bytes the kernel needs for these shapes on a grid of `grid` blocks (0 when unsupported).
size_t pk_decode_persistent_smem(const PkDecParams* params, int grid);
}

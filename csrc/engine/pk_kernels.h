// C declarations of every kernel launcher exported by libpocket_kernels. All pointers are
// device pointers unless a comment says otherwise; every function returns a PkStatus.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/pk_comm_types.h"

extern "C" {

int pk_last_cuda_error();
const char* pk_build_arch();

int pk_matvec(const void* W, const float* scale, const void* Wb, int N, int Nb, int K, int M, const void* x_in,
              const float* parts, int nparts, void* hidden_out, const float* gamma, int norm_mode, float eps,
              const PkWait* wait, int epi, void* y, int ldy, const PkPush* push, int sm_count,
              cudaStream_t stream);

unsigned pk_matvec_ring_status();

int pk_gemm_umma(const void* A, int lda, const void* W, const float* scale, int wfmt, int M, int N, int K,
                 int epi, void* C, const void* resid, int ldc, uint32_t* status, const PkPush* push,
                 cudaStream_t stream);

int pk_deltanet_seq(const void* proj, int ld, int T, int key_heads, int value_heads, int key_dim,
                    int value_dim, const float* conv_w, float* conv_state, const float* A_log,
                    const float* dt_bias, const float* norm_w, float eps, float* state, void* out,
                    cudaStream_t stream);

size_t pk_deltanet_chunk_workspace(int T, int key_heads, int value_heads);
int pk_deltanet_chunked(const void* proj, int ld, int T, int key_heads, int value_heads, int key_dim,
                        int value_dim, const float* conv_w, float* conv_state, const float* A_log,
                        const float* dt_bias, const float* norm_w, float eps, float* state, void* out, float* ws,
                        cudaStream_t stream);

int pk_qk_norm_rope_append(const void* proj, int ld, int M, int Hq, int Hkv, int head_dim, const int* pos,
                           const float* q_gamma, const float* k_gamma, float eps, int rotary_dim, float theta,
                           void* q_out, void* kcache, void* vcache, int ctx_cap, cudaStream_t stream);

int pk_gqa_decode(const void* q, const void* kcache, const void* vcache, const int* pos, int M, int Hq,
                  int Hkv, int head_dim, int ctx_cap, float scale, int nsplit, int window, int sink, float* ws,
                  const void* gate_proj, int ld, void* out, cudaStream_t stream);

int pk_qk_norm_rope_append_kv(const void* proj, int ld, int M, int Hq, int Hkv, int head_dim, const int* pos,
                              const float* q_gamma, const float* k_gamma, float eps, int rotary_dim, float theta,
                              void* q_out, void* kcache, void* vcache, float* kscale, float* vscale, int ctx_cap, cudaStream_t stream);
int pk_gqa_decode_kv(const void* q, const void* kcache, const void* vcache, const float* kscale, const float* vscale, const int* pos,
                     int M, int Hq, int Hkv, int head_dim, int ctx_cap, float scale, int nsplit, int window, int sink, float* ws,
                     const void* gate_proj, int ld, void* out, cudaStream_t stream);

int pk_embedding(const int* tokens, int M, const void* table, int dim, int vocab_start, int vocab_rows,
                 void* out_bf16, float* out_f32, cudaStream_t stream);

int pk_rmsnorm(const void* x, const float* parts, int nparts, int M, int K, void* hidden_out,
               const float* gamma, int mode, float eps, void* y, const PkWait* wait, cudaStream_t stream);

int pk_rmsnorm_rs_ag(void* hidden, const float* parts, int world, int rank, int rows_per_rank, int M, int K, const float* gamma,
                     int mode, float eps, void* const* y_peer, const PkWait* wait_rs, const PkPush* pub_ag, const PkWait* wait_ag,
                     int sm_count, cudaStream_t stream);

int pk_mtp_concat_norm(const int* tokens, int M, const void* table, const void* hidden, int K, const float* gamma_e,
                       const float* gamma_h, float eps, void* out, cudaStream_t stream);

int pk_silu_mul(const void* gate_up, int M, int inter, void* out, float limit, cudaStream_t stream);

int pk_argmax(const float* logits, int ld, int M, int n, int id_offset, int nblocks, float* cand_val,
              int* cand_idx, float* out_val, int* out_idx, cudaStream_t stream);
int pk_argmax_merge(const float* cand_val, const int* cand_idx, int M, int ncand, float* out_val,
                    int* out_idx, cudaStream_t stream);

int pk_bump_epoch(uint32_t* epoch, cudaStream_t stream);
int pk_add_int(int* p, int n, int delta, cudaStream_t stream);
int pk_copy_int(const int* src, int* dst, int n, cudaStream_t stream);

int pk_fill_fp8_gauss(void* w, float* scale, int N, int K, float sigma, uint64_t seed, cudaStream_t stream);
int pk_fill_bf16_gauss(void* w, size_t n, float mean, float sigma, uint64_t seed, cudaStream_t stream);
int pk_fill_f32_gauss(float* w, size_t n, float mean, float sigma, uint64_t seed, cudaStream_t stream);
int pk_iota_int(int* p, int n, const int* base_dev, int base_host, cudaStream_t stream);
int pk_store_token(const int* token, int* out, int* counter, int cap, cudaStream_t stream);
int pk_cand_push(const float* val, const int* idx, int M, const PkPush* push, float* const* peer_val,
                 int* const* peer_idx, const uint32_t* status, int stride, cudaStream_t stream);
int pk_cand_merge_wait(const float* cand_val, const int* cand_idx, int M, int world, const PkWait* wait,
                       int* out_idx, uint32_t* status, int stride, cudaStream_t stream);
int pk_fp8_to_bf16(const void* w, const float* scale, int N, int K, void* out, cudaStream_t stream);
int pk_rmsnorm_quant(const void* x, int M, int K, const float* gamma, int mode, float eps, void* y, int terms, void* q, int m_pad,
                     float* scale_t, int s_ld, cudaStream_t stream);
int pk_quant_act_fp8(const void* x, int ldx, int M, int K, int terms, void* q, int m_pad, float* scale_t, int s_ld, cudaStream_t stream);
int pk_gemm_fp8(const void* Aq, int terms, int m_pad, const float* a_scale, int a_ld, const void* W, const float* w_scale, int M, int N,
                int K, int epi, void* C, const void* resid, int ldc, uint32_t* status, const PkPush* push, int sm_count, cudaStream_t stream);
int pk_gqa_prefill_umma(const void* q, const void* kcache, const void* vcache, const int* pos, int M, int Hq, int Hkv, int head_dim, int ctx_cap,
                        float scale, const void* gate_proj, int ld, void* out, uint32_t* status, cudaStream_t stream);
int pk_gemm_bf16_grouped(const void* A, int lda, const void* W, const int* seg, int n_groups, int R, int N, int K, int epi, void* C, int ldc,
                         uint32_t* status, int sm_count, cudaStream_t stream);
int pk_scatter_rows(const void* src, const int* slots, int n, int row_bytes, void* pool, cudaStream_t stream);
int pk_topk_select(const float* score, const int* lengths, int M, int n, int ld, int k, int* out, cudaStream_t stream);
int pk_gemm_bf16(const void* A, int lda, const void* W, int M, int N, int K, int epi, void* C, const void* resid, int ldc,
                 uint32_t* status, const PkPush* push, int sm_count, cudaStream_t stream);
}

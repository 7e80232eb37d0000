// Kernels of the external block drafter ("DSpark") of the Qwen hybrid model:
//   * per-head RMSNorm of q / k rows (plain gamma) + half-split rotation over the WHOLE head from tables that already carry
//     the YaRN frequencies and the attention factor, q written as bf16 rows, k and v appended to a position-indexed cache;
//   * the Markov head: logits[v] += w2[v, :] . e for the embedding e = w1[previous token] of one row, with the block maxima
//     of the corrected logits, and the pick that turns them into the next previous token and its embedding.
// Block attention over context + block is the split-context GQA kernel with every row's extent set to the end of the block
// (the block's K / V are appended behind the context first), so it needs no kernel of its own.
//
// Reference counterpart: cpp_engine/cuda/qwen_dspark_ops.cu (YaRN RoPE, dual-source GQA, Markov bias, confidence) and
// cpp_engine/src/qwen_dspark.cpp:598-640,686-829.
#include "../common/pk_common.cuh"

namespace {

using namespace pk;
constexpr int kD = 128;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// grid (rows, Hq + Hkv), 128 threads: head hh < Hq is a query head, else a key head (its value head is copied alongside).
__global__ void __launch_bounds__(kD)
dspark_qk_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ k, int ldk, const bf16* __restrict__ v, int ldv, const int* __restrict__ pos,
                 const float* __restrict__ q_gamma, const float* __restrict__ k_gamma, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                 int Hq, int Hkv, int cap, float eps, bf16* __restrict__ q_out, bf16* __restrict__ kcache, bf16* __restrict__ vcache) {
  const int m = blockIdx.x, hh = blockIdx.y, d = threadIdx.x;
  __shared__ float red[4];
  __shared__ float sy[kD];
  const bool is_q = hh < Hq;
  const int hk = hh - Hq;
  const float x = is_q ? __bfloat162float(q[(size_t)m * ldq + hh * kD + d]) : __bfloat162float(k[(size_t)m * ldk + hk * kD + d]);
  float ss = warp_sum_f(x * x);
  if ((d & 31) == 0) red[d >> 5] = ss;
  __syncthreads();
  ss = red[0] + red[1] + red[2] + red[3];
  const float y = x * rsqrtf(ss / (float)kD + eps) * (is_q ? q_gamma[d] : k_gamma[d]);
  sy[d] = y;
  __syncthreads();
  const int p = pos[m];
  const int half = kD / 2, j = d < half ? d : d - half;
  const float cs = cos_t[(size_t)p * half + j], sn = sin_t[(size_t)p * half + j];
  const float other = d < half ? sy[d + half] : sy[d - half];
  const float r = d < half ? y * cs - other * sn : y * cs + other * sn;
  if (is_q) {
    q_out[((size_t)m * Hq + hh) * kD + d] = __float2bfloat16(r);
  } else if (p >= 0 && p < cap) {
    const size_t ci = ((size_t)hk * cap + p) * kD + d;
    kcache[ci] = __float2bfloat16(r);
    vcache[ci] = v[(size_t)m * ldv + hk * kD + d];
  } else if (d == 0) {
    PK_DEBUG_RECORD(101, p, cap);
  }
}

// One warp per vocabulary row: logits[v] += w2[v, :] . e; block maximum (value, lowest index) to cand[blockIdx.x].
__global__ void __launch_bounds__(256)
dspark_markov_kernel(float* __restrict__ logits, const bf16* __restrict__ w2, const float* __restrict__ e, int vocab, int rank, float* __restrict__ cand_val,
                     int* __restrict__ cand_idx) {
  extern __shared__ float es[];
  for (int i = threadIdx.x; i < rank; i += 256) es[i] = e[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int vrow = blockIdx.x * 8 + warp; vrow < vocab; vrow += gridDim.x * 8) {
    const bf16* w = w2 + (size_t)vrow * rank;
    float acc = 0.f;
    for (int c = lane * 2; c < rank; c += 64) {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(w + c);
      acc = fmaf(__uint_as_float(u << 16), es[c], acc);
      acc = fmaf(__uint_as_float(u & 0xffff0000u), es[c + 1], acc);
    }
    acc = warp_sum_f(acc);
    const float val = logits[vrow] + acc;
    if (lane == 0) logits[vrow] = val;
    if (val > best || (val == best && vrow < bi)) {
      best = val;
      bi = vrow;
    }
  }
  __shared__ float bv[8];
  __shared__ int bx[8];
  if (lane == 0) {
    bv[warp] = best;
    bx[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (bv[w] > best || (bv[w] == best && bx[w] < bi)) {
        best = bv[w];
        bi = bx[w];
      }
    cand_val[blockIdx.x] = best;
    cand_idx[blockIdx.x] = bi;
  }
}

// Final pick over the block candidates (lowest index on ties): token out, and the next row's embedding e = w1[token].
__global__ void __launch_bounds__(256)
dspark_pick_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx, int n, const bf16* __restrict__ w1, int rank, int* __restrict__ token_out,
                   float* __restrict__ e_out) {
  __shared__ float sv[256];
  __shared__ int si[256];
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += 256) {
    const float v = cand_val[i];
    const int id = cand_idx[i];
    if (v > best || (v == best && id < bi)) {
      best = v;
      bi = id;
    }
  }
  sv[threadIdx.x] = best;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      const float ov = sv[threadIdx.x + s];
      const int oi = si[threadIdx.x + s];
      if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
        sv[threadIdx.x] = ov;
        si[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  const int tok = si[0];
  if (threadIdx.x == 0) *token_out = tok;
  for (int i = threadIdx.x; i < rank; i += 256) e_out[i] = __bfloat162float(w1[(size_t)tok * rank + i]);
}

__global__ void __launch_bounds__(256) dspark_gather_kernel(const int* __restrict__ token, const bf16* __restrict__ w1, int rank, float* __restrict__ e_out) {
  const int tok = *token;
  for (int i = threadIdx.x; i < rank; i += 256) e_out[i] = __bfloat162float(w1[(size_t)tok * rank + i]);
}

}  // namespace

// q [M, Hq * 128], k / v [M, Hkv * 128] bf16 (row strides in elements), pos [M], tables [positions, 64] (cos and sin of the
// YaRN angles times the attention factor), caches [Hkv, cap, 128] bf16. q_out [M, Hq, 128] bf16.
PK_API int pk_dspark_qk_norm_rope_append(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const int* pos, int M, int Hq, int Hkv,
                                         int head_dim, const float* q_gamma, const float* k_gamma, const float* cos_t, const float* sin_t, float eps,
                                         void* q_out, void* kcache, void* vcache, int cap, cudaStream_t stream) {
  if (head_dim != kD) return PK_ERR_UNSUPPORTED;
  if (M < 1 || Hq < 0 || Hkv < 0 || Hq + Hkv < 1 || cap < 1 || pos == nullptr) return PK_ERR_BAD_ARG;
  dspark_qk_kernel<<<dim3(M, Hq + Hkv), kD, 0, stream>>>((const pk::bf16*)q, ldq, (const pk::bf16*)k, ldk, (const pk::bf16*)v, ldv, pos, q_gamma, k_gamma, cos_t,
                                                         sin_t, Hq, Hkv, cap, eps, (pk::bf16*)q_out, (pk::bf16*)kcache, (pk::bf16*)vcache);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// One row of the Markov head: logits [vocab] fp32 += w2 [vocab, rank] bf16 . e [rank]; token_out = argmax (lowest index on
// ties); e_next = w1[token_out] as fp32 [rank] (may alias e). cand_*: scratch of `blocks` entries.
PK_API int pk_dspark_markov_row(float* logits, const void* w2, const void* w1, const float* e, int vocab, int rank, float* cand_val, int* cand_idx, int blocks,
                                int* token_out, float* e_next, cudaStream_t stream) {
  if (vocab < 1 || rank < 2 || (rank & 1) != 0 || blocks < 1 || blocks > 4096 || (size_t)rank * 4 > 48 * 1024) return PK_ERR_BAD_ARG;
  dspark_markov_kernel<<<blocks, 256, (size_t)rank * sizeof(float), stream>>>(logits, (const pk::bf16*)w2, e, vocab, rank, cand_val, cand_idx);
  PK_CHECK_LAUNCH();
  dspark_pick_kernel<<<1, 256, 0, stream>>>(cand_val, cand_idx, blocks, (const pk::bf16*)w1, rank, token_out, e_next);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// e_out = w1[*token] as fp32 [rank] (the embedding of the anchor token, read from the device).
PK_API int pk_dspark_markov_embed(const int* token, const void* w1, int rank, float* e_out, cudaStream_t stream) {
  if (token == nullptr || w1 == nullptr || e_out == nullptr || rank < 1) return PK_ERR_BAD_ARG;
  dspark_gather_kernel<<<1, 256, 0, stream>>>(token, (const pk::bf16*)w1, rank, e_out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

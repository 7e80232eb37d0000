// Linear layers and routed experts on RAW GGUF blocks: the quantised weights stay in their
// file layout in HBM and are decoded in registers, eight weights per lane, on their way
// into the FMA. One warp walks one output row (or a gate/up row pair) 256 weights per step.
//
//   pk_gguf_linear   y[m, n] = sum_k x[m, k] W[n, k]        (1..8 rows; bf16 / fp32 / SwiGLU out)
//   pk_gguf_moe_w13  h[route, j] = silu(W1_e x_t) * (W3_e x_t) * route weight
//   pk_gguf_moe_w2   y[t] += W2_e h[route]                   (fp32 atomics, or per-route partials)
//
// Device type ids follow the reference's table (src/loader/gguf/quant_types.py): iq2_xxs 0,
// q2_k 1, iq1_m 2, q4_k 3, q5_k 4, iq2_xs 5, iq3_xxs 6, iq4_xs 7, q6_k 8, plus q8_0 9 and
// bf16 10 here. Replaces its DP4A / float kernels (src/csrc/cuda_kernel_impl.cu:6545-6632,
// 7039-8275: gguf_quant_gemm*, gguf_moe_w13*, gguf_moe_w2*, gguf_moe_single_*).
#include <mutex>

#include "../common/pk_common.cuh"

namespace {

using namespace pk;

#include "gguf_codebooks.inc"

enum : int { T_IQ2_XXS = 0, T_Q2_K = 1, T_IQ1_M = 2, T_Q4_K = 3, T_Q5_K = 4, T_IQ2_XS = 5, T_IQ3_XXS = 6,
             T_IQ4_XS = 7, T_Q6_K = 8, T_Q8_0 = 9, T_BF16 = 10, T_MXFP4 = 11 };
constexpr int T_LAST = T_MXFP4;

__host__ __device__ constexpr int block_bytes(int t) {
  return t == T_IQ2_XXS ? 66 : t == T_Q2_K ? 84 : t == T_IQ1_M ? 56 : t == T_Q4_K ? 144 : t == T_Q5_K ? 176
       : t == T_IQ2_XS ? 74 : t == T_IQ3_XXS ? 98 : t == T_IQ4_XS ? 136 : t == T_Q6_K ? 210 : t == T_Q8_0 ? 272 : t == T_MXFP4 ? 136 : 512;
}

__device__ __forceinline__ float ld_f16(const uint8_t* p) {
  const uint16_t v = (uint16_t)p[0] | ((uint16_t)p[1] << 8);
  return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) {
  return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }

__device__ __forceinline__ void k4_scale_min(const uint8_t* s, int j, float& sc, float& mn) {
  if (j < 4) {
    sc = (float)(s[j] & 63);
    mn = (float)(s[j + 4] & 63);
  } else {
    sc = (float)((s[j + 4] & 15) | ((s[j - 4] >> 6) << 4));
    mn = (float)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
  }
}

__device__ const float kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// Weights [8p, 8p + 8) of one 256-weight super block (for q8_0: eight 34-byte blocks).
template <int TYPE>
__device__ __forceinline__ void decode8(const uint8_t* b, int p, float (&w)[8]) {
  if constexpr (TYPE == T_Q8_0) {
    const uint8_t* blk = b + (p >> 2) * 34;
    const float d = ld_f16(blk);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)(int8_t)blk[2 + (p & 3) * 8 + i];
  } else if constexpr (TYPE == T_BF16) {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = __uint_as_float(ld_u16(b + (p * 8 + i) * 2) << 16);
  } else if constexpr (TYPE == T_MXFP4) {
    // eight 17-byte groups: one E8M0 scale, then 32 E2M1 nibbles (element 2j low, 2j+1 high)
    const uint8_t* blk = b + (p >> 2) * 17;
    const float d = e8m0_to_float(blk[0]);
    const uint8_t* q = blk + 1 + (p & 3) * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[2 * i] = d * e2m1_to_float(q[i] & 15);
      w[2 * i + 1] = d * e2m1_to_float(q[i] >> 4);
    }
  } else if constexpr (TYPE == T_Q2_K) {
    const int g = p >> 1, half = g >> 3, gi = g & 7, shift = (gi >> 1) * 2;
    const uint8_t* q = b + 16 + half * 32 + (gi & 1) * 16 + (p & 1) * 8;
    const uint8_t s = b[g];
    const float d = ld_f16(b + 80) * (float)(s & 15), m = ld_f16(b + 82) * (float)(s >> 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * (float)((q[i] >> shift) & 3) - m;
  } else if constexpr (TYPE == T_Q4_K || TYPE == T_Q5_K) {
    const int pr = p >> 3, h = (p >> 2) & 1, l0 = (p & 3) * 8, j = 2 * pr + h;
    float sc, mn;
    k4_scale_min(b + 4, j, sc, mn);
    const float d = ld_f16(b) * sc, m = ld_f16(b + 2) * mn;
    const uint8_t* q = b + (TYPE == T_Q4_K ? 16 : 48) + pr * 32 + l0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int v = h ? (q[i] >> 4) : (q[i] & 15);
      if constexpr (TYPE == T_Q5_K) v += ((b[16 + l0 + i] >> j) & 1) << 4;
      w[i] = d * (float)v - m;
    }
  } else if constexpr (TYPE == T_Q6_K) {
    const int n = p >> 4, idx = (p & 15) * 8, k = idx >> 5, l0 = idx & 31;
    const uint8_t* ql = b + 64 * n + (k & 1) * 32 + l0;
    const uint8_t* qh = b + 128 + 32 * n + l0;
    const float d = ld_f16(b + 208) * (float)(int8_t)b[192 + 8 * n + 2 * k + (l0 >> 4)];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int lo = k < 2 ? (ql[i] & 15) : (ql[i] >> 4);
      w[i] = d * (float)((lo | (((qh[i] >> (2 * k)) & 3) << 4)) - 32);
    }
  } else if constexpr (TYPE == T_IQ2_XXS) {
    const int sub = p >> 2, part = p & 3;
    const uint8_t* q = b + 2 + sub * 8;
    const uint32_t aux = ld_u32(q + 4);
    const float d = ld_f16(b) * 0.125f * (float)(2 * (aux >> 28) + 1);
    const uint64_t g = kIq2xxsGrid[q[part]];
    const uint8_t sg = kKsigns[(aux >> (7 * part)) & 127];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v = d * (float)((g >> (8 * i)) & 0xff);
      w[i] = (sg >> i) & 1 ? -v : v;
    }
  } else if constexpr (TYPE == T_IQ2_XS) {
    const int sub = p >> 2, part = p & 3;
    const uint32_t q = ld_u16(b + 2 + (sub * 4 + part) * 2);
    const uint32_t nib = (b[66 + sub] >> (4 * (part >> 1))) & 15;
    const float d = ld_f16(b) * 0.25f * ((float)nib + 0.5f);
    const uint64_t g = kIq2xsGrid[q & 511];
    const uint8_t sg = kKsigns[q >> 9];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v = d * (float)((g >> (8 * i)) & 0xff);
      w[i] = (sg >> i) & 1 ? -v : v;
    }
  } else if constexpr (TYPE == T_IQ3_XXS) {
    const int sub = p >> 2, pr = p & 3;
    const uint32_t aux = ld_u32(b + 66 + sub * 4);
    const float d = ld_f16(b) * 0.5f * ((float)(aux >> 28) + 0.5f);
    const uint32_t g0 = kIq3xxsGrid[b[2 + sub * 8 + pr * 2]], g1 = kIq3xxsGrid[b[2 + sub * 8 + pr * 2 + 1]];
    const uint8_t sg = kKsigns[(aux >> (7 * pr)) & 127];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float v0 = d * (float)((g0 >> (8 * i)) & 0xff), v1 = d * (float)((g1 >> (8 * i)) & 0xff);
      w[i] = (sg >> i) & 1 ? -v0 : v0;
      w[4 + i] = (sg >> (4 + i)) & 1 ? -v1 : v1;
    }
  } else if constexpr (TYPE == T_IQ4_XS) {
    const int ib = p >> 2, q = p & 3;
    const uint32_t sh = ld_u16(b + 2);
    const int ls = ((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 15) | (((sh >> (2 * ib)) & 3) << 4);
    const float d = ld_f16(b) * (float)(ls - 32);
    const uint8_t* qs = b + 8 + 16 * ib + 8 * (q & 1);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * kIq4nl[q < 2 ? (qs[i] & 15) : (qs[i] >> 4)];
  } else if constexpr (TYPE == T_IQ1_M) {
    const int ib = p >> 2, g = p & 3;
    const uint32_t s0 = ld_u16(b + 48), s1 = ld_u16(b + 50), s2 = ld_u16(b + 52), s3 = ld_u16(b + 54);
    const uint16_t dbits = (uint16_t)((s0 >> 12) | ((s1 >> 8) & 0xf0) | ((s2 >> 4) & 0xf00) | (s3 & 0xf000));
    const uint32_t sw = ld_u16(b + 48 + (ib >> 1) * 2) >> (6 * (ib & 1));
    const float dl = __half2float(__ushort_as_half(dbits)) * (float)(2 * ((sw >> (3 * (g >> 1))) & 7) + 1);
    const uint32_t h = b[32 + 2 * ib + (g >> 1)];
    const uint32_t idx = b[4 * ib + g] | (((g & 1) ? (h << 4) : (h << 8)) & 0x700);
    const float delta = (h & ((g & 1) ? 0x80 : 0x08)) ? -0.125f : 0.125f;
    const uint64_t gr = kIq1Grid[idx];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = dl * ((float)(int8_t)((gr >> (8 * i)) & 0xff) + delta);
  }
}

constexpr int kThreads = 256;
constexpr int kWarps = 8;

// The decoders read single bytes; from global memory that is one load instruction per byte, each a round trip to L2.
// A warp therefore first brings a stretch of its row into shared memory with 16-byte loads and decodes from there.
constexpr int kStageBlocks = 8;                                  // 2048 weights per stretch
// Bytes of one warp's stage buffer for rows of `type` with K weights: a stretch of up to kStageBlocks blocks plus the
// misalignment of its start, rounded to 16. Sized per launch so that small block types leave room for more resident blocks.
__host__ __device__ inline int stage_bytes_per_warp(int type, int K) {
  const int nb = (K >> 8) < kStageBlocks ? (K >> 8) : kStageBlocks;
  return ((nb * block_bytes(type) + 15) & ~15) + 16;
}

// One warp: dot products of one raw row with M staged activation rows (fp32, [M][K]). `stage` is this warp's
// stage_bytes_per_warp(TYPE, K) bytes of shared memory.
template <int TYPE, int M>
__device__ __forceinline__ void row_dot(const uint8_t* wrow, const float* xs, int K, int lane, float (&acc)[M], uint8_t* stage) {
  constexpr int BB = block_bytes(TYPE);
  const int nblk = K >> 8;
  if (stage == nullptr) {
    // Several activation rows share every decoded weight, which hides the byte loads: decode straight from global memory
    // (and keep the shared memory for a second resident block).
    for (int blk = 0; blk < nblk; ++blk) {
      float w[8];
      decode8<TYPE>(wrow + (size_t)blk * BB, lane, w);
      const int k = (blk << 8) + (lane << 3);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 a = *reinterpret_cast<const float4*>(xs + m * K + k);
        const float4 c = *reinterpret_cast<const float4*>(xs + m * K + k + 4);
        acc[m] += w[0] * a.x + w[1] * a.y + w[2] * a.z + w[3] * a.w + w[4] * c.x + w[5] * c.y + w[6] * c.z + w[7] * c.w;
      }
    }
    return;
  }
  for (int blk0 = 0; blk0 < nblk; blk0 += kStageBlocks) {
    const int nb = min(kStageBlocks, nblk - blk0);
    const uint8_t* src = wrow + (size_t)blk0 * BB;
    const int mis = (int)((uintptr_t)src & 15);
    const uint8_t* src_al = src - mis;           // the bytes before `src` belong to the previous row or block of the same tensor
    const int total = mis + nb * BB;
    __syncwarp();                                // the previous stretch has been decoded by every lane
    for (int off = lane << 4; off < total; off += 512) {
      if (off + 16 <= total) {
        *reinterpret_cast<uint4*>(stage + off) = __ldg(reinterpret_cast<const uint4*>(src_al + off));
      } else {
        for (int i = off < mis ? mis - off : 0; off + i < total; ++i) stage[off + i] = src_al[off + i];   // never past the row's end
      }
    }
    __syncwarp();
    for (int b = 0; b < nb; ++b) {
      float w[8];
      decode8<TYPE>(stage + mis + b * BB, lane, w);
      const int k = ((blk0 + b) << 8) + (lane << 3);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 a = *reinterpret_cast<const float4*>(xs + m * K + k);
        const float4 c = *reinterpret_cast<const float4*>(xs + m * K + k + 4);
        acc[m] += w[0] * a.x + w[1] * a.y + w[2] * a.z + w[3] * a.w + w[4] * c.x + w[5] * c.y + w[6] * c.z + w[7] * c.w;
      }
    }
  }
}

struct LinearParams {
  const uint8_t* W;   // [N, K/256 blocks]
  int type, N, K, M;
  const bf16* x;      // [M, K]
  const float* gamma; // optional fused RMSNorm (plain gamma)
  float eps;
  int epi;            // 0 bf16, 1 swiglu (rows j and j + N/2), 2 fp32
  void* y;
  int ldy;
  int stage_bytes;    // per warp, behind the staged activations in dynamic shared memory (one- and two-row launches)
};

template <int M>
__device__ __forceinline__ void dispatch_row(int type, const uint8_t* wrow, const float* xs, int K, int lane, float (&acc)[M], uint8_t* stage) {
  switch (type) {
    case T_IQ2_XXS: row_dot<T_IQ2_XXS, M>(wrow, xs, K, lane, acc, stage); break;
    case T_Q2_K: row_dot<T_Q2_K, M>(wrow, xs, K, lane, acc, stage); break;
    case T_IQ1_M: row_dot<T_IQ1_M, M>(wrow, xs, K, lane, acc, stage); break;
    case T_Q4_K: row_dot<T_Q4_K, M>(wrow, xs, K, lane, acc, stage); break;
    case T_Q5_K: row_dot<T_Q5_K, M>(wrow, xs, K, lane, acc, stage); break;
    case T_IQ2_XS: row_dot<T_IQ2_XS, M>(wrow, xs, K, lane, acc, stage); break;
    case T_IQ3_XXS: row_dot<T_IQ3_XXS, M>(wrow, xs, K, lane, acc, stage); break;
    case T_IQ4_XS: row_dot<T_IQ4_XS, M>(wrow, xs, K, lane, acc, stage); break;
    case T_Q6_K: row_dot<T_Q6_K, M>(wrow, xs, K, lane, acc, stage); break;
    case T_Q8_0: row_dot<T_Q8_0, M>(wrow, xs, K, lane, acc, stage); break;
    case T_MXFP4: row_dot<T_MXFP4, M>(wrow, xs, K, lane, acc, stage); break;
    default: row_dot<T_BF16, M>(wrow, xs, K, lane, acc, stage); break;
  }
}

__host__ __device__ inline size_t row_bytes(int type, int K) { return (size_t)(K >> 8) * block_bytes(type); }

template <int M>
__global__ void __launch_bounds__(kThreads) gguf_linear_kernel(const LinearParams p) {
  extern __shared__ __align__(16) float xs[];  // [M][K]
  __shared__ float red[40];
  constexpr bool kStaged = M <= 2;     // one or two rows: the byte loads of the decoders dominate, stage the weights
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* stage = kStaged ? reinterpret_cast<uint8_t*>(xs + (size_t)M * p.K) + (size_t)warp * p.stage_bytes : nullptr;
  for (int m = 0; m < M; ++m) {
    float ss = 0.f;
    for (int k = tid; k < p.K; k += kThreads) {
      // the template may be wider than the number of rows given: pad with zeros
      const float v = m < p.M ? __bfloat162float(p.x[(size_t)m * p.K + k]) : 0.f;
      xs[m * p.K + k] = v;
      ss += v * v;
    }
    if (p.gamma != nullptr) {
      ss = block_sum(ss, red);
      const float rs = rsqrtf(ss / (float)p.K + p.eps);
      for (int k = tid; k < p.K; k += kThreads)
        xs[m * p.K + k] = __bfloat162float(__float2bfloat16(xs[m * p.K + k] * rs * p.gamma[k]));
    }
  }
  __syncthreads();
  const size_t rb = row_bytes(p.type, p.K);
  const int half_n = p.N >> 1;
  const int groups = p.epi == 1 ? half_n : p.N;
  for (int g = blockIdx.x * kWarps + warp; g < groups; g += gridDim.x * kWarps) {
    float a0[M], a1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { a0[m] = 0.f; a1[m] = 0.f; }
    dispatch_row<M>(p.type, p.W + (size_t)g * rb, xs, p.K, lane, a0, stage);
    if (p.epi == 1) dispatch_row<M>(p.type, p.W + (size_t)(g + half_n) * rb, xs, p.K, lane, a1, stage);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      a0[m] = warp_sum(a0[m]);
      if (p.epi == 1) a1[m] = warp_sum(a1[m]);
    }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) {
        if (m >= p.M) break;
        if (p.epi == 1) ((bf16*)p.y)[(size_t)m * p.ldy + g] = __float2bfloat16(silu(a0[m]) * a1[m]);
        else if (p.epi == 0) ((bf16*)p.y)[(size_t)m * p.ldy + g] = __float2bfloat16(a0[m]);
        else ((float*)p.y)[(size_t)m * p.ldy + g] = a0[m];
      }
    }
  }
}

// ---- routed experts ----
// Routes are sorted by expert: seg_start[e] .. seg_start[e+1] index into route_token / route_weight.
constexpr int kRouteParallelMax = 64;   // up to this many routes in a step, every route gets its own blocks

struct MoeParams {
  const uint8_t* W13;  // [E, 2I, H] raw rows (gate rows then up rows per expert)
  const uint8_t* W2;   // [E, H, I]
  int type13, type2;
  int E, H, I;
  const bf16* x;        // [T, H]
  const int* seg_start; // [E + 1]
  const int* route_token;   // [R]
  const float* route_weight; // [R]
  float* hbuf;          // [R, I] fp32 hidden of every route (already times the route weight)
  float* y;             // [T, H] fp32, accumulated with atomics
  float limit;          // SwiGLU clamp, 0 = off
  int expert_offset;    // first expert id stored in W13 / W2 (expert parallel shard)
  int local_experts;
  float* ybuf;          // [R, H] per-route outputs for the fixed-order reduce; null = atomics into y
};

// Gate/up rows of one expert against MB staged tokens (MB = 1, 2, 4 or 8: a decode step has one token per expert, and
// decoding a weight once per token slot that is not there would be wasted arithmetic).
template <int MB>
__device__ __forceinline__ void moe_w13_rows(const MoeParams& p, const uint8_t* base, size_t rb, const float* xs, int rs, int cnt, int lane,
                                             int warp, uint8_t* stage) {
  for (int j = blockIdx.x * kWarps + warp; j < p.I; j += gridDim.x * kWarps) {
    float g[MB], u[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) { g[m] = 0.f; u[m] = 0.f; }
    dispatch_row<MB>(p.type13, base + (size_t)j * rb, xs, p.H, lane, g, stage);
    dispatch_row<MB>(p.type13, base + (size_t)(p.I + j) * rb, xs, p.H, lane, u, stage);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      float gv = warp_sum(g[m]), uv = warp_sum(u[m]);
      if (p.limit > 0.f) {
        gv = fminf(gv, p.limit);
        uv = fminf(fmaxf(uv, -p.limit), p.limit);
      }
      if (lane == 0 && m < cnt) p.hbuf[(size_t)(rs + m) * p.I + j] = silu(gv) * uv * p.route_weight[rs + m];
    }
  }
}

template <int MB>
__device__ __forceinline__ void moe_w2_rows(const MoeParams& p, const uint8_t* base, size_t rb, const float* hs, int rs, int cnt, int lane,
                                            int warp, uint8_t* stage) {
  for (int n = blockIdx.x * kWarps + warp; n < p.H; n += gridDim.x * kWarps) {
    float a[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) a[m] = 0.f;
    dispatch_row<MB>(p.type2, base + (size_t)n * rb, hs, p.I, lane, a, stage);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const float v = warp_sum(a[m]);
      if (lane == 0 && m < cnt) {
        if (p.ybuf != nullptr) p.ybuf[(size_t)(rs + m) * p.H + n] = v;
        else atomicAdd(p.y + (size_t)p.route_token[rs + m] * p.H + n, v);
      }
    }
  }
}

// grid: (row tiles, local experts). Each block stages up to 8 routed tokens of its expert at a
// time and lets its warps walk gate/up row pairs.
__global__ void __launch_bounds__(kThreads) gguf_moe_w13_kernel(const MoeParams p) {
  extern __shared__ __align__(16) float xs[];  // [8][H]
  const int le = blockIdx.y, e = le + p.expert_offset;
  const int r0 = p.seg_start[e], r1 = p.seg_start[e + 1];
  if (r0 >= r1) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t rb = row_bytes(p.type13, p.H);
  const uint8_t* base = p.W13 + (size_t)le * 2 * p.I * rb;
  for (int rs = r0; rs < r1; rs += 8) {
    const int cnt = min(8, r1 - rs);
    __syncthreads();
    const int mb = cnt <= 1 ? 1 : cnt <= 2 ? 2 : cnt <= 4 ? 4 : 8;
    for (int m = 0; m < mb; ++m)
      for (int k = tid; k < p.H; k += kThreads)
        xs[m * p.H + k] = m < cnt ? __bfloat162float(p.x[(size_t)p.route_token[rs + m] * p.H + k]) : 0.f;
    __syncthreads();
    if (mb == 1) moe_w13_rows<1>(p, base, rb, xs, rs, cnt, lane, warp, nullptr);
    else if (mb == 2) moe_w13_rows<2>(p, base, rb, xs, rs, cnt, lane, warp, nullptr);
    else if (mb == 4) moe_w13_rows<4>(p, base, rb, xs, rs, cnt, lane, warp, nullptr);
    else moe_w13_rows<8>(p, base, rb, xs, rs, cnt, lane, warp, nullptr);
  }
}

__global__ void __launch_bounds__(kThreads) gguf_moe_w2_kernel(const MoeParams p) {
  extern __shared__ __align__(16) float hs[];  // [8][I]
  const int le = blockIdx.y, e = le + p.expert_offset;
  const int r0 = p.seg_start[e], r1 = p.seg_start[e + 1];
  if (r0 >= r1) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t rb = row_bytes(p.type2, p.I);
  const uint8_t* base = p.W2 + (size_t)le * p.H * rb;
  for (int rs = r0; rs < r1; rs += 8) {
    const int cnt = min(8, r1 - rs);
    __syncthreads();
    const int mb = cnt <= 1 ? 1 : cnt <= 2 ? 2 : cnt <= 4 ? 4 : 8;
    for (int m = 0; m < mb; ++m)
      for (int k = tid; k < p.I; k += kThreads) hs[m * p.I + k] = m < cnt ? p.hbuf[(size_t)(rs + m) * p.I + k] : 0.f;
    __syncthreads();
    if (mb == 1) moe_w2_rows<1>(p, base, rb, hs, rs, cnt, lane, warp, nullptr);
    else if (mb == 2) moe_w2_rows<2>(p, base, rb, hs, rs, cnt, lane, warp, nullptr);
    else if (mb == 4) moe_w2_rows<4>(p, base, rb, hs, rs, cnt, lane, warp, nullptr);
    else moe_w2_rows<8>(p, base, rb, hs, rs, cnt, lane, warp, nullptr);
  }
}

// Few routes (decode, speculative verify): grid (row tiles, routes of this rank). Every block serves ONE route, so all
// blocks have work and an expert's rows spread over as many blocks as there are tiles; the expert of a route comes
// from a binary search in seg_start.
__device__ __forceinline__ int expert_of_route(const int* seg_start, int lo_e, int hi_e, int r) {
  while (hi_e - lo_e > 1) {   // invariant: seg_start[lo_e] <= r < seg_start[hi_e]
    const int mid = (lo_e + hi_e) >> 1;
    if (seg_start[mid] <= r) lo_e = mid;
    else hi_e = mid;
  }
  return lo_e;
}

__global__ void __launch_bounds__(kThreads) gguf_moe_w13_route_kernel(const MoeParams p) {
  extern __shared__ __align__(16) float xs[];  // [H], then the warps' stage buffers
  const int lo = p.seg_start[p.expert_offset], hi = p.seg_start[p.expert_offset + p.local_experts];
  const int r = lo + blockIdx.y;
  if (r >= hi) return;
  const int e = expert_of_route(p.seg_start, p.expert_offset, p.expert_offset + p.local_experts, r);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t rb = row_bytes(p.type13, p.H);
  const uint8_t* base = p.W13 + (size_t)(e - p.expert_offset) * 2 * p.I * rb;
  for (int k = tid; k < p.H; k += kThreads) xs[k] = __bfloat162float(p.x[(size_t)p.route_token[r] * p.H + k]);
  __syncthreads();
  moe_w13_rows<1>(p, base, rb, xs, r, 1, lane, warp,
                  reinterpret_cast<uint8_t*>(xs + p.H) + (size_t)warp * stage_bytes_per_warp(p.type13, p.H));
}

__global__ void __launch_bounds__(kThreads) gguf_moe_w2_route_kernel(const MoeParams p) {
  extern __shared__ __align__(16) float hs[];  // [I], then the warps' stage buffers
  const int lo = p.seg_start[p.expert_offset], hi = p.seg_start[p.expert_offset + p.local_experts];
  const int r = lo + blockIdx.y;
  if (r >= hi) return;
  const int e = expert_of_route(p.seg_start, p.expert_offset, p.expert_offset + p.local_experts, r);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t rb = row_bytes(p.type2, p.I);
  const uint8_t* base = p.W2 + (size_t)(e - p.expert_offset) * p.H * rb;
  for (int k = tid; k < p.I; k += kThreads) hs[k] = p.hbuf[(size_t)r * p.I + k];
  __syncthreads();
  moe_w2_rows<1>(p, base, rb, hs, r, 1, lane, warp,
                 reinterpret_cast<uint8_t*>(hs + p.I) + (size_t)warp * stage_bytes_per_warp(p.type2, p.I));
}

// Fixed-order reduce: y[t] += sum over k = 0..topk-1 of the output of route (t, k), skipping routes whose
// expert lives on another rank. route_pos[t * topk + k] is the route's position in the expert-sorted order.
__global__ void moe_reduce_routes_kernel(const float* __restrict__ ybuf, const int* __restrict__ route_pos, const int* __restrict__ seg_start,
                                         int topk, int H, int expert_offset, int local_experts, float* y) {
  const int t = blockIdx.y, n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= H) return;
  const int lo = seg_start[expert_offset], hi = seg_start[expert_offset + local_experts];
  float acc = y[(size_t)t * H + n];
  for (int k = 0; k < topk; ++k) {
    const int pos = route_pos[t * topk + k];
    if (pos >= lo && pos < hi) acc += ybuf[(size_t)pos * H + n];
  }
  y[(size_t)t * H + n] = acc;
}

// The same reduce with the route weight applied here (ybuf holds unweighted expert outputs, e.g. from the grouped GEMM).
__global__ void moe_reduce_routes_weighted_kernel(const float* __restrict__ ybuf, const float* __restrict__ route_weight,
                                                  const int* __restrict__ route_pos, const int* __restrict__ seg_start, int topk, int H,
                                                  int expert_offset, int local_experts, float* y) {
  const int t = blockIdx.y, n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= H) return;
  const int lo = seg_start[expert_offset], hi = seg_start[expert_offset + local_experts];
  float acc = y[(size_t)t * H + n];
  for (int k = 0; k < topk; ++k) {
    const int pos = route_pos[t * topk + k];
    if (pos >= lo && pos < hi) acc = fmaf(route_weight[pos], ybuf[(size_t)pos * H + n], acc);
  }
  y[(size_t)t * H + n] = acc;
}

__global__ void invert_routes_kernel(const int* __restrict__ route_src, int R, int* route_pos) {
  const int pos = blockIdx.x * blockDim.x + threadIdx.x;
  if (pos < R) route_pos[route_src[pos]] = pos;
}

// ---- routing ----
// Router logits: grid (expert groups of 8, token tiles of up to 8); one warp per expert, which reads its weight row
// once for the tile's tokens. A single token spreads over E / 8 blocks instead of streaming the whole router matrix
// through one block.
__global__ void __launch_bounds__(256) router_logits_kernel(const bf16* x, const float* rw, int H, int E, int T, float* logits) {
  extern __shared__ float xs[];  // [tokens of the tile][H]
  const int t0 = blockIdx.y * 8, nt = min(8, T - t0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int m = 0; m < nt; ++m)
    for (int k = tid; k < H; k += 256) xs[m * H + k] = __bfloat162float(x[(size_t)(t0 + m) * H + k]);
  __syncthreads();
  const int e = blockIdx.x * 8 + warp;
  if (e >= E) return;
  float a[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) a[m] = 0.f;
  const float* w = rw + (size_t)e * H;
  if (nt == 1) {
    for (int k = lane; k < H; k += 32) a[0] = fmaf(w[k], xs[k], a[0]);
  } else {
    for (int k = lane; k < H; k += 32) {
      const float wv = w[k];
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (m < nt) a[m] = fmaf(wv, xs[m * H + k], a[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    if (m >= nt) break;
    const float v = warp_sum(a[m]);
    if (lane == 0) logits[(size_t)(t0 + m) * E + e] = v;
  }
}

// One block per token: scores from the logits, top-k with lowest-id tie break.
// score_func 0 softmax, 1 sigmoid, 2 sqrt(softplus); selection on score + bias.
__global__ void __launch_bounds__(256) router_topk_kernel(const float* logits, const float* bias, int E,
                                                          int topk, int score_func, int norm_topk, float route_scale,
                                                          int* ids, float* weights) {
  extern __shared__ float sm[];  // [E] scores, [E] selection keys
  float* sc = sm;
  float* key = sc + E;
  __shared__ float red[40];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < E; e += 256) sc[e] = logits[(size_t)t * E + e];
  __syncthreads();
  if (score_func == 0) {
    float mx = -INFINITY;
    for (int e = tid; e < E; e += 256) mx = fmaxf(mx, sc[e]);
    mx = block_max(mx, red);
    float s = 0.f;
    for (int e = tid; e < E; e += 256) {
      sc[e] = __expf(sc[e] - mx);
      s += sc[e];
    }
    s = block_sum(s, red);
    for (int e = tid; e < E; e += 256) sc[e] /= s;
  } else {
    for (int e = tid; e < E; e += 256) sc[e] = score_func == 1 ? sigmoidf_(sc[e]) : sqrtf(softplusf_(sc[e]));
  }
  __syncthreads();
  // keys stay finite: a NaN or -inf key would never win a comparison below, the pick would keep its initial invalid id
  // and index shared memory with it
  for (int e = tid; e < E; e += 256) {
    const float k = sc[e] + (bias ? bias[e] : 0.f);
    key[e] = k > -3.0e38f ? k : -3.0e38f;
  }
  __syncthreads();
  if (warp == 0) {
    float wsum = 0.f;
    for (int j = 0; j < topk; ++j) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32)
        if (key[e] > bv) { bv = key[e]; bi = e; }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        ids[(size_t)t * topk + j] = bi;
        weights[(size_t)t * topk + j] = sc[bi];
        key[bi] = -INFINITY;
      }
      wsum += sc[bi];
      __syncwarp();
    }
    if (lane < topk) {
      float w = weights[(size_t)t * topk + lane];
      if (norm_topk) w /= (wsum > 0.f ? wsum : 1.f);
      weights[(size_t)t * topk + lane] = w * route_scale;
    }
  }
}

// Group routes by expert (single block; T * topk routes): counts, exclusive scan, fill in
// token order so that the layout is deterministic.
__global__ void __launch_bounds__(256) group_routes_kernel(const int* ids, const float* weights, int T, int topk, int E,
                                                           int* seg_start, int* route_token, float* route_weight,
                                                           int* route_src) {
  extern __shared__ int cnt[];  // [E + 1]
  const int tid = threadIdx.x, R = T * topk;
  for (int e = tid; e <= E; e += 256) cnt[e] = 0;
  __syncthreads();
  for (int r = tid; r < R; r += 256) {
#if PK_DEBUG_BUILD
    if (ids[r] < 0 || ids[r] >= E) {
      PK_DEBUG_RECORD(102, ids[r], E);
      continue;
    }
#endif
    atomicAdd(&cnt[ids[r]], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      cnt[e] = run;
      seg_start[e] = run;
      run += c;
    }
    cnt[E] = run;
    seg_start[E] = run;
  }
  __syncthreads();
  // deterministic fill: expert e's routes in increasing route index
  for (int e = tid; e < E; e += 256) {
    int pos = cnt[e];
    for (int r = 0; r < R; ++r)
      if (ids[r] == e) {
        route_token[pos] = r / topk;
        route_weight[pos] = weights[r];
        if (route_src) route_src[pos] = r;
        ++pos;
      }
  }
}

// Quantised embedding: decode selected rows to bf16 (one warp per 256 weights).
__global__ void __launch_bounds__(256) gguf_dequant_rows_kernel(const uint8_t* W, int type, const int* rows, int nrows,
                                                                int K, int row_offset, int table_rows, bf16* out) {
  // one warp per 256-weight block, walking (row, block) units with a grid stride; a lane's eight weights leave as one
  // 16-byte store
  const int lane = threadIdx.x & 31;
  const int nblk = K >> 8;
  const size_t rb = row_bytes(type, K);
  const long long units = (long long)nrows * nblk;
  for (long long u = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * 8) {
    const int r = (int)(u / nblk), blk = (int)(u - (long long)r * nblk);
    const int src = (rows ? rows[r] : r) - row_offset;
    const bool mine = src >= 0 && src < table_rows;
    float w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = 0.f;
    if (mine) {
      const uint8_t* b = W + (size_t)src * rb + (size_t)blk * block_bytes(type);
      switch (type) {
        case T_IQ2_XXS: decode8<T_IQ2_XXS>(b, lane, w); break;
        case T_Q2_K: decode8<T_Q2_K>(b, lane, w); break;
        case T_IQ1_M: decode8<T_IQ1_M>(b, lane, w); break;
        case T_Q4_K: decode8<T_Q4_K>(b, lane, w); break;
        case T_Q5_K: decode8<T_Q5_K>(b, lane, w); break;
        case T_IQ2_XS: decode8<T_IQ2_XS>(b, lane, w); break;
        case T_IQ3_XXS: decode8<T_IQ3_XXS>(b, lane, w); break;
        case T_IQ4_XS: decode8<T_IQ4_XS>(b, lane, w); break;
        case T_Q6_K: decode8<T_Q6_K>(b, lane, w); break;
        case T_Q8_0: decode8<T_Q8_0>(b, lane, w); break;
        case T_MXFP4: decode8<T_MXFP4>(b, lane, w); break;
        default: decode8<T_BF16>(b, lane, w); break;
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pr = __floats2bfloat162_rn(w[2 * i], w[2 * i + 1]);
      o[i] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * K + (blk << 8) + (lane << 3)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int M>
int launch_linear(const LinearParams& p_in, int sm_count, cudaStream_t stream) {
  LinearParams p = p_in;
  p.stage_bytes = M <= 2 ? stage_bytes_per_warp(p.type, p.K) : 0;
  const size_t smem = (size_t)M * p.K * sizeof(float) + (size_t)kWarps * p.stage_bytes;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gguf_linear_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 184 * 1024) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  const int groups = p.epi == 1 ? p.N / 2 : p.N;
  int blocks = (groups + kWarps - 1) / kWarps;
  blocks = min(blocks, (sm_count > 0 ? sm_count : 148) * 8);
  gguf_linear_kernel<M><<<blocks, kThreads, smem, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

}  // namespace

PK_API int pk_gguf_block_bytes(int type) { return (type >= 0 && type <= T_LAST) ? block_bytes(type) : 0; }

// x bf16 [M, K] (M <= 8, M * K * 4 bytes <= 200 KB), W raw rows, K a multiple of 256.
PK_API int pk_gguf_linear(const void* W, int type, int N, int K, int M, const void* x, const float* gamma, float eps,
                          int epi, void* y, int ldy, int sm_count, cudaStream_t stream) {
  if (type < 0 || type > T_LAST || M < 1 || M > 8 || (K & 255) != 0 || N < 1) return PK_ERR_BAD_ARG;
  if ((size_t)M * K * 4 > 184 * 1024) return PK_ERR_UNSUPPORTED;   // plus the warps' stage buffers
  if (epi == 1 && (N & 1)) return PK_ERR_BAD_ARG;
  LinearParams p{(const uint8_t*)W, type, N, K, M, (const pk::bf16*)x, gamma, eps, epi, y, ldy, 0};
  switch (M) {
    case 1: return launch_linear<1>(p, sm_count, stream);
    case 2: return launch_linear<2>(p, sm_count, stream);
    case 3: case 4: p.M = M; return launch_linear<4>(p, sm_count, stream);
    default: return launch_linear<8>(p, sm_count, stream);
  }
}

// Per-device scratch for the router logits [T, E]; grows on demand (a growth inside a stream capture fails: run one
// step of the same size before capturing, which callers do anyway to warm the kernels up).
static float* router_scratch(size_t floats) {
  static float* buf[64] = {};
  static size_t cap[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cap[dev] < floats) {
    float* nb = nullptr;
    const size_t want = floats < 4096 ? 4096 : floats;
    if (cudaMalloc((void**)&nb, want * sizeof(float)) != cudaSuccess) return nullptr;
    // the old buffer may still be in use by kernels in flight: it is left to the process lifetime (sizes settle quickly)
    buf[dev] = nb;
    cap[dev] = want;
  }
  return buf[dev];
}

PK_API int pk_router_topk(const void* x, const float* router_w, const float* bias, int T, int H, int E, int topk,
                          int score_func, int norm_topk, float route_scale, int* ids, float* weights,
                          cudaStream_t stream) {
  if (T < 1 || topk < 1 || topk > 32 || topk > E) return PK_ERR_BAD_ARG;
  const int tile = T < 8 ? T : 8;
  const size_t smem_x = (size_t)tile * H * sizeof(float);
  if (smem_x > 200 * 1024 || (size_t)2 * E * sizeof(float) > 48 * 1024) return PK_ERR_UNSUPPORTED;
  if (smem_x > 48 * 1024) {
    static PkDeviceOnce once;
    if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
      if (cudaFuncSetAttribute(router_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
        pk_set_last_cuda_error((int)cudaGetLastError());
        return PK_ERR_CUDA;
      }
      once_guard.done();
    }
  }
  float* logits = router_scratch((size_t)T * E);
  if (logits == nullptr) return PK_ERR_CUDA;
  router_logits_kernel<<<dim3((E + 7) / 8, (T + 7) / 8), 256, smem_x, stream>>>((const pk::bf16*)x, router_w, H, E, T, logits);
  PK_CHECK_LAUNCH();
  router_topk_kernel<<<T, 256, (size_t)2 * E * sizeof(float), stream>>>(logits, bias, E, topk, score_func, norm_topk, route_scale, ids,
                                                                        weights);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_group_routes(const int* ids, const float* weights, int T, int topk, int E, int* seg_start, int* route_token,
                           float* route_weight, int* route_src, cudaStream_t stream) {
  if (E + 1 > 12000) return PK_ERR_UNSUPPORTED;
  group_routes_kernel<<<1, 256, (size_t)(E + 1) * sizeof(int), stream>>>(ids, weights, T, topk, E, seg_start, route_token,
                                                                         route_weight, route_src);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Routed experts of one rank: experts [expert_offset, expert_offset + local_experts) live in
// W13 / W2. y (fp32 [T, H]) must be zeroed by the caller; hbuf holds R * I floats.
// y[t] += sum over the token's routes (in route order) of route_weight * ybuf[route]; routes of experts outside
// [expert_offset, expert_offset + local_experts) are skipped. route_pos: int scratch [T * topk].
PK_API int pk_moe_reduce_routes(const float* ybuf, const float* route_weight, const int* route_src, const int* seg_start, int T, int topk, int H,
                                int expert_offset, int local_experts, int* route_pos, float* y, cudaStream_t stream) {
  if (ybuf == nullptr || route_weight == nullptr || route_src == nullptr || seg_start == nullptr || route_pos == nullptr || y == nullptr || T < 1 || topk < 1)
    return PK_ERR_BAD_ARG;
  const int R = T * topk;
  invert_routes_kernel<<<(R + 255) / 256, 256, 0, stream>>>(route_src, R, route_pos);
  PK_CHECK_LAUNCH();
  moe_reduce_routes_weighted_kernel<<<dim3((H + 255) / 256, T), 256, 0, stream>>>(ybuf, route_weight, route_pos, seg_start, topk, H, expert_offset,
                                                                                  local_experts, y);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// route_pos[route_src[pos]] = pos: where route (t, k) sits in the expert-sorted order.
PK_API int pk_invert_routes(const int* route_src, int R, int* route_pos, cudaStream_t stream) {
  if (route_src == nullptr || route_pos == nullptr || R < 1) return PK_ERR_BAD_ARG;
  invert_routes_kernel<<<(R + 255) / 256, 256, 0, stream>>>(route_src, R, route_pos);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

static int moe_forward_impl(const void* W13, const void* W2, int type13, int type2, int E, int H, int I, const void* x,
                            const int* seg_start, const int* route_token, const float* route_weight, float* hbuf, float* y,
                            float limit, int expert_offset, int local_experts, int sm_count, float* ybuf, cudaStream_t stream,
                            int total_routes = 0);

PK_API int pk_gguf_moe_forward(const void* W13, const void* W2, int type13, int type2, int E, int H, int I,
                               const void* x, const int* seg_start, const int* route_token, const float* route_weight,
                               float* hbuf, float* y, float limit, int expert_offset, int local_experts, int sm_count,
                               cudaStream_t stream) {
  return moe_forward_impl(W13, W2, type13, type2, E, H, I, x, seg_start, route_token, route_weight, hbuf, y, limit, expert_offset,
                          local_experts, sm_count, nullptr, stream);
}

// Same result up to rounding, but bitwise reproducible: every route writes its own output row (ybuf, R * H
// floats) and a second kernel adds the rows of each token in route order. route_src comes from pk_group_routes;
// route_pos is R ints of scratch; T tokens with topk routes each.
PK_API int pk_gguf_moe_forward_det(const void* W13, const void* W2, int type13, int type2, int E, int H, int I, const void* x,
                                   const int* seg_start, const int* route_token, const float* route_weight, const int* route_src,
                                   float* hbuf, float* ybuf, int* route_pos, float* y, int T, int topk, float limit,
                                   int expert_offset, int local_experts, int sm_count, cudaStream_t stream) {
  if (route_src == nullptr || ybuf == nullptr || route_pos == nullptr || T < 1 || topk < 1) return PK_ERR_BAD_ARG;
  const int R = T * topk;
  const int rc = moe_forward_impl(W13, W2, type13, type2, E, H, I, x, seg_start, route_token, route_weight, hbuf, y, limit,
                                  expert_offset, local_experts, sm_count, ybuf, stream, R);
  if (rc != PK_OK) return rc;
  invert_routes_kernel<<<(R + 255) / 256, 256, 0, stream>>>(route_src, R, route_pos);
  PK_CHECK_LAUNCH();
  moe_reduce_routes_kernel<<<dim3((H + 255) / 256, T), 256, 0, stream>>>(ybuf, route_pos, seg_start, topk, H, expert_offset,
                                                                         local_experts, y);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

static int moe_forward_impl(const void* W13, const void* W2, int type13, int type2, int E, int H, int I, const void* x,
                            const int* seg_start, const int* route_token, const float* route_weight, float* hbuf, float* y,
                            float limit, int expert_offset, int local_experts, int sm_count, float* ybuf, cudaStream_t stream,
                            int total_routes) {
  if ((H & 255) || (I & 255) || local_experts < 1) return PK_ERR_BAD_ARG;
  if ((size_t)8 * H * 4 > 184 * 1024 || (size_t)8 * I * 4 > 184 * 1024) return PK_ERR_UNSUPPORTED;   // plus the warps' stage buffers
  MoeParams p{(const uint8_t*)W13, (const uint8_t*)W2, type13, type2, E, H, I, (const pk::bf16*)x, seg_start, route_token,
              route_weight, hbuf, y, limit, expert_offset, local_experts, ybuf};
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gguf_moe_w13_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 184 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gguf_moe_w2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 184 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gguf_moe_w13_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 184 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gguf_moe_w2_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 184 * 1024) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  (void)sm_count;
  if (total_routes > 0 && total_routes <= kRouteParallelMax) {
    // one block set per route: at most total_routes of them belong to this rank
    MoeParams q = p;
    const int t13 = (I + kWarps - 1) / kWarps, t2 = (H + kWarps - 1) / kWarps;
    gguf_moe_w13_route_kernel<<<dim3(t13 < 256 ? t13 : 256, total_routes), kThreads,
                                (size_t)H * 4 + (size_t)kWarps * stage_bytes_per_warp(type13, H), stream>>>(q);
    PK_CHECK_LAUNCH();
    gguf_moe_w2_route_kernel<<<dim3(t2 < 256 ? t2 : 256, total_routes), kThreads,
                               (size_t)I * 4 + (size_t)kWarps * stage_bytes_per_warp(type2, I), stream>>>(q);
    PK_CHECK_LAUNCH();
    return PK_OK;
  }
  const int tiles13 = min((I + kWarps - 1) / kWarps, 32), tiles2 = min((H + kWarps - 1) / kWarps, 32);
  gguf_moe_w13_kernel<<<dim3(tiles13, local_experts), kThreads, (size_t)8 * H * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  gguf_moe_w2_kernel<<<dim3(tiles2, local_experts), kThreads, (size_t)8 * I * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// out[r, :] = dequant(W[rows[r] - row_offset, :]) as bf16; rows outside the local table give zeros
// (vocabulary-sharded embedding). rows == null means rows 0..nrows-1.
PK_API int pk_gguf_dequant_rows(const void* W, int type, const int* rows, int nrows, int K, int row_offset,
                                int table_rows, void* out, cudaStream_t stream) {
  if (type < 0 || type > T_LAST || (K & 255) != 0 || nrows < 1) return PK_ERR_BAD_ARG;
  if (((uintptr_t)out & 15) != 0) return PK_ERR_BAD_ARG;
  const long long units = (long long)nrows * (K >> 8);
  const long long want = (units + 7) / 8;
  const int grid = (int)(want < 148LL * 32 ? want : 148LL * 32);
  gguf_dequant_rows_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)W, type, rows, nrows, K, row_offset, table_rows,
                                                    (pk::bf16*)out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// DeepSeek-V4 specific kernels: hyper-connection mixing (with the following RMSNorm fused),
// head preparation (per-head RMS scaling, interleaved RoPE, Hadamard + FP4 fake quantisation),
// KV preparation with FP8 fake quantisation, gated-pooling compressor, lightning-indexer
// scores, sink-softmax sparse attention over window + compressed rows, hash routing.
//
// Roles in the reference: src/csrc/cuda_kernel_impl.cu (hc_split_pre / hc_post, hadamard128,
// fused q/kv prefuse kernels, compressor, c4 indexer, sparse attention variants) and
// cpp_engine/src/cuda_ops.cu. Layouts and fusion boundaries here are this engine's own:
//  * the residual stream is fp32 [M, 4, dim];
//  * window keys live in a ring of `ring` rows (ring >= window + rows per call - 1, so that a
//    multi-row call never overwrites a row that one of its own queries still needs) followed
//    by the compressed entries; attention computes the window rows arithmetically from the
//    position and takes compressed rows either as "all visible" or from a selection list;
//  * the compressor keeps the last 2*ratio (overlap) or ratio per-token projections in a ring
//    indexed by position, so no state is shifted.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "../common/pk_common.cuh"

namespace {
using namespace pk;

constexpr int kHcMax = 4;

// ------------------------------------------------------------------------------------------
// numerics shared by several kernels

__device__ __forceinline__ float pow2_ceil_scale(float amax_over_qmax) {
  // 2^ceil(log2(x)) for x > 0, exact on powers of two
  int e;
  const float m = frexpf(amax_over_qmax, &e);          // x = m * 2^e, m in [0.5, 1)
  return m == 0.5f ? ldexpf(1.f, e - 1) : ldexpf(1.f, e);
}

__device__ __forceinline__ float fp8_round_trip(float v, float s) {
  const float q = fminf(fmaxf(v / s, -448.f), 448.f);
  return e4m3_to_float(float_to_e4m3(q)) * s;
}

// nearest E2M1 level, ties toward zero
__device__ __forceinline__ float fp4_round_trip(float v, float s) {
  const float n = fminf(fmaxf(v / s, -6.f), 6.f), a = fabsf(n);
  const float l = a <= 0.25f ? 0.f : a <= 0.75f ? 0.5f : a <= 1.25f ? 1.f : a <= 1.75f ? 1.5f : a <= 2.5f ? 2.f
                : a <= 3.5f ? 3.f : a <= 5.f ? 4.f : 6.f;
  return (n < 0.f ? -l : l) * s;
}

// In-place orthonormal Walsh-Hadamard transform of 128 floats in shared memory by threads
// 0..127 of the block (all threads of the block must call; `tid` is threadIdx.x).
__device__ __forceinline__ void hadamard128_smem(float* x, int tid) {
  for (int stride = 1; stride < 128; stride <<= 1) {
    float a = 0.f, b = 0.f;
    const bool act = tid < 128 && (tid & stride) == 0;
    if (act) {
      a = x[tid];
      b = x[tid + stride];
    }
    __syncthreads();
    if (act) {
      x[tid] = a + b;
      x[tid + stride] = a - b;
    }
    __syncthreads();
  }
  if (tid < 128) x[tid] *= 0.08838834764831845f;
  __syncthreads();
}

// FP4 fake quantisation of 128 floats in shared memory, blocks of 32 (threads 0..127).
__device__ __forceinline__ void fp4_quant128_smem(float* x, float* scales4, int tid) {
  if (tid < 4) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(x[tid * 32 + i]));
    scales4[tid] = pow2_ceil_scale(fmaxf(amax, 6.f * 1.1754943508222875e-38f) / 6.f);
  }
  __syncthreads();
  if (tid < 128) x[tid] = fp4_round_trip(x[tid], scales4[tid >> 5]);
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
// hc_pre (+ RMSNorm) and hc_head (+ RMSNorm)

struct HcPreParams {
  const float* h;       // [M, hc, dim]
  const float* fn;      // [mix, hc*dim]
  const float* scale;   // [3] (pre mode) or [1] (head mode)
  const float* base;    // [mix]
  const float* gamma;   // [dim] RMSNorm weight applied to the mixed vector (may be null)
  int M, dim, hc, mix, iters, head_mode;
  float hc_eps, norm_eps;
  bf16* x_out;          // [M, dim] normalised mixed vector
  float* x_raw;         // [M, dim] mixed vector before the norm (may be null)
  float* post;          // [M, hc]     (pre mode)
  float* comb;          // [M, hc, hc] (pre mode)
};

constexpr int kHcThreads = 256;
constexpr int kMixMax = 24;

__global__ void __launch_bounds__(kHcThreads) hc_pre_kernel(const HcPreParams p) {
  extern __shared__ float xs[];                      // [dim]
  __shared__ float red[kMixMax + 1][kHcThreads / 32];
  __shared__ float mixv[kMixMax + 1];
  __shared__ float pre[kHcMax];
  __shared__ float scratch[33];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.hc * p.dim;
  const float* h = p.h + (size_t)m * n;

  float acc[kMixMax + 1];
#pragma unroll
  for (int r = 0; r <= kMixMax; ++r) acc[r] = 0.f;
  for (int i = tid * 4; i < n; i += kHcThreads * 4) {
    const float4 v = *reinterpret_cast<const float4*>(h + i);
    acc[kMixMax] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
    for (int r = 0; r < kMixMax; ++r) {
      if (r < p.mix) {
        const float4 f = *reinterpret_cast<const float4*>(p.fn + (size_t)r * n + i);
        acc[r] += f.x * v.x + f.y * v.y + f.z * v.z + f.w * v.w;
      }
    }
  }
#pragma unroll
  for (int r = 0; r <= kMixMax; ++r) {
    const float s = warp_sum(acc[r]);
    if (lane == 0) red[r][warp] = s;
  }
  __syncthreads();
  if (tid <= kMixMax) {
    float s = 0.f;
    for (int w = 0; w < kHcThreads / 32; ++w) s += red[tid][w];
    mixv[tid] = s;
  }
  __syncthreads();
  if (tid == 0) {
    const int hc = p.hc;
    const float r = rsqrtf(mixv[kMixMax] / (float)n + p.norm_eps);
    if (p.head_mode) {
      for (int i = 0; i < hc; ++i) pre[i] = sigmoidf_(mixv[i] * r * p.scale[0] + p.base[i]) + p.hc_eps;
    } else {
      for (int i = 0; i < hc; ++i) {
        pre[i] = sigmoidf_(mixv[i] * r * p.scale[0] + p.base[i]) + p.hc_eps;
        p.post[(size_t)m * hc + i] = 2.f * sigmoidf_(mixv[hc + i] * r * p.scale[1] + p.base[hc + i]);
      }
      float c[kHcMax][kHcMax];
      for (int i = 0; i < hc; ++i) {
        float mx = -INFINITY;
        for (int j = 0; j < hc; ++j) {
          c[i][j] = mixv[2 * hc + i * hc + j] * r * p.scale[2] + p.base[2 * hc + i * hc + j];
          mx = fmaxf(mx, c[i][j]);
        }
        float s = 0.f;
        for (int j = 0; j < hc; ++j) {
          c[i][j] = expf(c[i][j] - mx);
          s += c[i][j];
        }
        for (int j = 0; j < hc; ++j) c[i][j] = c[i][j] / s + p.hc_eps;
      }
      for (int it = 0; it < p.iters; ++it) {
        if (it > 0) {
          for (int i = 0; i < hc; ++i) {
            float s = p.hc_eps;
            for (int j = 0; j < hc; ++j) s += c[i][j];
            for (int j = 0; j < hc; ++j) c[i][j] /= s;
          }
        }
        for (int j = 0; j < hc; ++j) {
          float s = p.hc_eps;
          for (int i = 0; i < hc; ++i) s += c[i][j];
          for (int i = 0; i < hc; ++i) c[i][j] /= s;
        }
      }
      for (int i = 0; i < hc; ++i)
        for (int j = 0; j < hc; ++j) p.comb[((size_t)m * hc + i) * hc + j] = c[i][j];
    }
  }
  __syncthreads();
  float ss = 0.f;
  for (int d = tid; d < p.dim; d += kHcThreads) {
    float x = 0.f;
    for (int i = 0; i < p.hc; ++i) x += pre[i] * h[(size_t)i * p.dim + d];
    xs[d] = x;
    ss += x * x;
    if (p.x_raw) p.x_raw[(size_t)m * p.dim + d] = x;
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)p.dim + p.norm_eps);
  for (int d = tid; d < p.dim; d += kHcThreads) {
    const float g = p.gamma ? p.gamma[d] : 1.f;
    p.x_out[(size_t)m * p.dim + d] = __float2bfloat16(p.gamma ? xs[d] * r * g : xs[d]);
  }
}

// h_out[m][j][d] = post[m][j] * (y[m][d] + y2[m][d]) + sum_i comb[m][i][j] * h[m][i][d]  (in place allowed)
__global__ void hc_post_kernel(const float* __restrict__ y, const float* __restrict__ y2, const float* h, const float* __restrict__ post,
                               const float* __restrict__ comb, int dim, int hc, float* h_out) {
  const int m = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= dim) return;
  float hv[kHcMax];
  for (int i = 0; i < hc; ++i) hv[i] = h[((size_t)m * hc + i) * dim + d];
  float yv = y[(size_t)m * dim + d];
  if (y2) yv += y2[(size_t)m * dim + d];
  for (int j = 0; j < hc; ++j) {
    float o = post[(size_t)m * hc + j] * yv;
    for (int i = 0; i < hc; ++i) o += comb[((size_t)m * hc + i) * hc + j] * hv[i];
    h_out[((size_t)m * hc + j) * dim + d] = o;
  }
}

// ------------------------------------------------------------------------------------------
// head preparation: one block per (row, head)
//   flags bit0: scale by rsqrt(mean(x^2) + eps) (no gamma)   bit1: RoPE on the last rd dims
//         bit2: inverse RoPE                                  bit3: Hadamard-128 + FP4 fake quant (hd == 128)

struct HeadPrepParams {
  bf16* x;              // [M, H, hd] in place
  const int* pos;       // [M]
  const float* cos_t;   // [max_pos, rd/2]
  const float* sin_t;
  int H, hd, rd, flags;
  float eps;
};

__global__ void __launch_bounds__(128) head_prep_kernel(const HeadPrepParams p) {
  extern __shared__ float v[];          // [hd]
  __shared__ float scratch[33];
  __shared__ float sc4[4];
  const int m = blockIdx.x, hh = blockIdx.y, tid = threadIdx.x;
  bf16* x = p.x + ((size_t)m * p.H + hh) * p.hd;
  float ss = 0.f;
  for (int d = tid; d < p.hd; d += 128) {
    const float t = __bfloat162float(x[d]);
    v[d] = t;
    ss += t * t;
  }
  if (p.flags & 1) {
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / (float)p.hd + p.eps);
    for (int d = tid; d < p.hd; d += 128) v[d] *= r;
  }
  __syncthreads();
  if (p.flags & 6) {
    const int half = p.rd / 2, off = p.hd - p.rd;
    const float sgn = (p.flags & 4) ? -1.f : 1.f;
    for (int i = tid; i < half; i += 128) {
      const float c = p.cos_t[(size_t)p.pos[m] * half + i], s = sgn * p.sin_t[(size_t)p.pos[m] * half + i];
      const float a = v[off + 2 * i], b = v[off + 2 * i + 1];
      v[off + 2 * i] = a * c - b * s;
      v[off + 2 * i + 1] = a * s + b * c;
    }
    __syncthreads();
  }
  if (p.flags & 8) {
    hadamard128_smem(v, tid);
    fp4_quant128_smem(v, sc4, tid);
  }
  for (int d = tid; d < p.hd; d += 128) x[d] = __float2bfloat16(v[d]);
}

// ------------------------------------------------------------------------------------------
// KV preparation: RMSNorm(gamma) -> RoPE on last rd -> FP8 fake quant (blocks of 64) of the rest
// -> bf16 row at ring slot pos % ring. One block (128 threads) per row.

struct KvPrepParams {
  const float* kv;      // [M, hd] projection output
  const float* gamma;   // [hd]
  const int* pos;
  const float* cos_t;
  const float* sin_t;
  int hd, rd, ring;
  float eps;
  bf16* dst;            // [ring + ..., hd]
  const int* dst_rows;  // optional: row of dst for each input row (null: pos % ring)
};

__global__ void __launch_bounds__(128) kv_prep_kernel(const KvPrepParams p) {
  extern __shared__ float v[];          // [hd]
  __shared__ float scratch[33];
  __shared__ float bscale[16];
  const int m = blockIdx.x, tid = threadIdx.x;
  const float* src = p.kv + (size_t)m * p.hd;
  float ss = 0.f;
  for (int d = tid; d < p.hd; d += 128) {
    v[d] = src[d];
    ss += v[d] * v[d];
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)p.hd + p.eps);
  for (int d = tid; d < p.hd; d += 128) v[d] = v[d] * r * p.gamma[d];
  __syncthreads();
  const int half = p.rd / 2, off = p.hd - p.rd, pos = p.pos[m];
  for (int i = tid; i < half; i += 128) {
    const float c = p.cos_t[(size_t)pos * half + i], s = p.sin_t[(size_t)pos * half + i];
    const float a = v[off + 2 * i], b = v[off + 2 * i + 1];
    v[off + 2 * i] = a * c - b * s;
    v[off + 2 * i + 1] = a * s + b * c;
  }
  const int nblk = off / 64;
  if (tid < nblk) {
    float amax = 0.f;
    for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[tid * 64 + i]));
    bscale[tid] = pow2_ceil_scale(fmaxf(amax, 1e-4f) / 448.f);
  }
  __syncthreads();
  bf16* dst = p.dst + (size_t)(p.dst_rows ? p.dst_rows[m] : pos % p.ring) * p.hd;
  for (int d = tid; d < p.hd; d += 128) dst[d] = __float2bfloat16(d < off ? fp8_round_trip(v[d], bscale[d >> 6]) : v[d]);
}

// ------------------------------------------------------------------------------------------
// Compressor pooling. One block per completed entry.
//   proj  [M, 2*C] fp32 rows of this call: kv projection (C = coff*cd) then score projection
//   ring  [2][slots][C] fp32: kv and (score + ape) of earlier tokens, slot = position % slots
// Entry c pools tokens [c*ratio, (c+1)*ratio) (second half of the channels when overlapping) and,
// when overlapping, tokens [(c-1)*ratio, c*ratio) with the first half of the channels.

struct CompressParams {
  const float* proj;
  const float* ape;       // [ratio, C]
  float* ring;            // [2, slots, C]
  const float* gamma;     // [cd]
  const float* cos_t;
  const float* sin_t;
  int pos0, M, ratio, cd, overlap, slots, rd, rotate, first_entry;
  float eps;
  bf16* dst;              // [entries, cd]; entry c is written to row c
};

__global__ void __launch_bounds__(128) compress_pool_kernel(const CompressParams p) {
  extern __shared__ float v[];          // [cd]
  __shared__ float scratch[33];
  __shared__ float bscale[16];
  const int c = p.first_entry + blockIdx.x, tid = threadIdx.x;
  const int C = (p.overlap ? 2 : 1) * p.cd;
  const int nslot = (p.overlap ? 2 : 1) * p.ratio;
  const int t_first = c * p.ratio - (p.overlap ? p.ratio : 0);
  for (int d = tid; d < p.cd; d += 128) {
    float mx = -INFINITY;
    for (int s = 0; s < nslot; ++s) {
      const int t = t_first + s;
      if (t < 0) continue;
      const int ch = (p.overlap && s >= p.ratio) ? p.cd + d : d;
      const float sc = t >= p.pos0 ? p.proj[(size_t)(t - p.pos0) * 2 * C + C + ch] + p.ape[(size_t)(t % p.ratio) * C + ch]
                                   : p.ring[((size_t)p.slots + (t % p.slots)) * C + ch];
      mx = fmaxf(mx, sc);
    }
    float num = 0.f, den = 0.f;
    for (int s = 0; s < nslot; ++s) {
      const int t = t_first + s;
      if (t < 0) continue;
      const int ch = (p.overlap && s >= p.ratio) ? p.cd + d : d;
      float sc, kv;
      if (t >= p.pos0) {
        const float* row = p.proj + (size_t)(t - p.pos0) * 2 * C;
        sc = row[C + ch] + p.ape[(size_t)(t % p.ratio) * C + ch];
        kv = row[ch];
      } else {
        sc = p.ring[((size_t)p.slots + (t % p.slots)) * C + ch];
        kv = p.ring[(size_t)(t % p.slots) * C + ch];
      }
      const float e = __expf(sc - mx);
      num += e * kv;
      den += e;
    }
    v[d] = num / den;
  }
  __syncthreads();
  float ss = 0.f;
  for (int d = tid; d < p.cd; d += 128) ss += v[d] * v[d];
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)p.cd + p.eps);
  for (int d = tid; d < p.cd; d += 128) v[d] = v[d] * r * p.gamma[d];
  __syncthreads();
  const int half = p.rd / 2, off = p.cd - p.rd, pos = c * p.ratio;
  for (int i = tid; i < half; i += 128) {
    const float cs = p.cos_t[(size_t)pos * half + i], sn = p.sin_t[(size_t)pos * half + i];
    const float a = v[off + 2 * i], b = v[off + 2 * i + 1];
    v[off + 2 * i] = a * cs - b * sn;
    v[off + 2 * i + 1] = a * sn + b * cs;
  }
  __syncthreads();
  bf16* dst = p.dst + (size_t)c * p.cd;
  if (p.rotate) {                       // cd == 128
    hadamard128_smem(v, tid);
    fp4_quant128_smem(v, bscale, tid);
    for (int d = tid; d < p.cd; d += 128) dst[d] = __float2bfloat16(v[d]);
  } else {
    const int nblk = off / 64;
    if (tid < nblk) {
      float amax = 0.f;
      for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[tid * 64 + i]));
      bscale[tid] = pow2_ceil_scale(fmaxf(amax, 1e-4f) / 448.f);
    }
    __syncthreads();
    for (int d = tid; d < p.cd; d += 128) dst[d] = __float2bfloat16(d < off ? fp8_round_trip(v[d], bscale[d >> 6]) : v[d]);
  }
}

// After pooling: remember the last `slots` tokens of this call. One block per remembered token.
__global__ void compress_ring_kernel(const CompressParams p) {
  const int C = (p.overlap ? 2 : 1) * p.cd;
  const int keep = min(p.M, p.slots);
  const int i = p.M - keep + blockIdx.x, t = p.pos0 + i;
  const float* row = p.proj + (size_t)i * 2 * C;
  for (int ch = threadIdx.x; ch < C; ch += blockDim.x) {
    p.ring[(size_t)(t % p.slots) * C + ch] = row[ch];
    p.ring[((size_t)p.slots + (t % p.slots)) * C + ch] = row[C + ch] + p.ape[(size_t)(t % p.ratio) * C + ch];
  }
}

// ------------------------------------------------------------------------------------------
// Lightning-indexer scores: score[m][c] = sum_h w[m][h] * relu(q[m][h] . k[c]) for c < (pos+1)/ratio,
// -inf for the other c < ld. One thread per entry, q of the row in shared memory.

struct IndexScoreParams {
  const bf16* q;        // [M, ih, 128]
  const bf16* k;        // [n, 128]
  const float* w;       // [M, ldw] head weights (already scaled)
  const int* pos;
  int ih, ratio, ld, ldw;
  float wscale;
  float* score;         // [M, ld]
};

__global__ void __launch_bounds__(128) index_score_kernel(const IndexScoreParams p) {
  extern __shared__ float qs[];         // [ih, 128] then w [ih]
  const int m = blockIdx.y, tid = threadIdx.x;
  float* ws = qs + p.ih * 128;
  for (int i = tid; i < p.ih * 128; i += 128) qs[i] = __bfloat162float(p.q[(size_t)m * p.ih * 128 + i]);
  for (int i = tid; i < p.ih; i += 128) ws[i] = p.w[(size_t)m * p.ldw + i] * p.wscale;
  __syncthreads();
  const int c = blockIdx.x * 128 + tid;
  if (c >= p.ld) return;
  const int nvalid = (p.pos[m] + 1) / p.ratio;
  if (c >= nvalid) {
    p.score[(size_t)m * p.ld + c] = -INFINITY;
    return;
  }
  uint32_t kr[64];
  const uint4* kp = reinterpret_cast<const uint4*>(p.k + (size_t)c * 128);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint4 t = kp[i];
    kr[4 * i] = t.x;
    kr[4 * i + 1] = t.y;
    kr[4 * i + 2] = t.z;
    kr[4 * i + 3] = t.w;
  }
  float total = 0.f;
  for (int h = 0; h < p.ih; ++h) {
    const float* qh = qs + h * 128;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      dot += qh[2 * i] * __uint_as_float(kr[i] << 16);
      dot += qh[2 * i + 1] * __uint_as_float(kr[i] & 0xffff0000u);
    }
    total += ws[h] * fmaxf(dot, 0.f);
  }
  p.score[(size_t)m * p.ld + c] = total;
}

// ------------------------------------------------------------------------------------------
// Sparse attention with a sink logit. K == V: one row of `hd` dims per key.
// Rows of query m (position p): window rows (p - j) % ring for j < min(p + 1, win); compressed rows
// comp_base + c, where c runs over all c < (p + 1) / ratio (mode 1) or over sel[m][0..ksel) with -1 for
// unused entries (mode 2). One warp per head; inverse RoPE of the output fused.

struct SparseAttnParams {
  const bf16* q;        // [M, H, hd]
  const bf16* kv;       // [ring + entries, hd]
  const int* pos;
  const int* rope_pos;  // [M] position used for the inverse RoPE of the output (null: pos)
  const int* sel;       // [M, ksel] (mode 2)
  const float* sink;    // [H]
  const float* cos_t;
  const float* sin_t;
  int H, win, ring, ratio, mode, ksel, rd;
  float scale;
  bf16* out;            // [M, H, hd]
};

// One warp serves G consecutive heads of a query row: the key row is loaded once per warp and used for all G heads.
template <int DPL, int G>   // dims per lane: hd = 32 * DPL
__global__ void __launch_bounds__(256) sparse_attn_kernel(const SparseAttnParams p) {
  constexpr int HD = 32 * DPL;
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hh = (blockIdx.y * (blockDim.x >> 5) + warp) * G;     // first head of this warp
  if (hh >= p.H) return;
  const int pos = p.pos[m];
  float qv[G][DPL], acc[G][DPL], mx[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int hg = min(hh + g, p.H - 1);     // a warp past the last head repeats it and stores nothing
    const bf16* q = p.q + ((size_t)m * p.H + hg) * HD + lane * DPL;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      qv[g][i] = __bfloat162float(q[i]) * p.scale;
      acc[g][i] = 0.f;
    }
    // the sink contributes exp(sink - mx) to the denominator only; without one the running maximum starts at -inf
    mx[g] = p.sink ? p.sink[hg] : -INFINITY;
    l[g] = p.sink ? 1.f : 0.f;
  }
  const int nwin = min(pos + 1, p.win);
  const int ncomp = p.mode == 1 ? (pos + 1) / p.ratio : p.mode == 2 ? p.ksel : 0;
  for (int r = 0; r < nwin + ncomp; ++r) {
    int row;
    if (r < nwin) {
      row = (pos - r) % p.ring;
    } else if (p.mode == 1) {
      row = p.ring + (r - nwin);
    } else {
      const int c = p.sel[(size_t)m * p.ksel + (r - nwin)];
      if (c < 0) continue;
      row = p.ring + c;
    }
    const bf16* k = p.kv + (size_t)row * HD + lane * DPL;
    float kf[DPL], dot[G];
    uint32_t kw[DPL / 2];
    // a lane's DPL * 2 bytes start on a multiple of their own size: 16-byte loads where that size allows
    if constexpr (DPL % 8 == 0) {
#pragma unroll
      for (int v = 0; v < DPL / 8; ++v) {
        const uint4 t = reinterpret_cast<const uint4*>(k)[v];
        kw[4 * v] = t.x; kw[4 * v + 1] = t.y; kw[4 * v + 2] = t.z; kw[4 * v + 3] = t.w;
      }
    } else if constexpr (DPL % 4 == 0) {
#pragma unroll
      for (int v = 0; v < DPL / 4; ++v) {
        const uint2 t = reinterpret_cast<const uint2*>(k)[v];
        kw[2 * v] = t.x; kw[2 * v + 1] = t.y;
      }
    } else {
#pragma unroll
      for (int v = 0; v < DPL / 2; ++v) kw[v] = reinterpret_cast<const uint32_t*>(k)[v];
    }
#pragma unroll
    for (int g = 0; g < G; ++g) dot[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; i += 2) {
      const uint32_t u = kw[i >> 1];
      kf[i] = __uint_as_float(u << 16);
      kf[i + 1] = __uint_as_float(u & 0xffff0000u);
#pragma unroll
      for (int g = 0; g < G; ++g) dot[g] += qv[g][i] * kf[i] + qv[g][i + 1] * kf[i + 1];
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float d = warp_sum(dot[g]);
      // d is the same in every lane, so the branch is uniform: most keys do not raise the maximum
      if (d > mx[g]) {
        const float cs = __expf(mx[g] - d);
        l[g] = l[g] * cs + 1.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * cs + kf[i];
        mx[g] = d;
      } else {
        const float e = __expf(d - mx[g]);
        l[g] += e;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(e, kf[i], acc[g][i]);
      }
    }
  }
  // inverse RoPE on the last rd dims (pairs never straddle lanes: DPL is even)
  const int off = HD - p.rd, half = p.rd / 2;
  const int rp = p.rope_pos ? p.rope_pos[m] : pos;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (hh + g >= p.H) break;
    const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] *= inv;
    if (lane * DPL + DPL > off) {
#pragma unroll
      for (int i = 0; i < DPL; i += 2) {
        const int d = lane * DPL + i;
        if (d >= off) {
          const int pi = (d - off) >> 1;
          const float c = p.cos_t[(size_t)rp * half + pi], s = -p.sin_t[(size_t)rp * half + pi];
          const float a = acc[g][i], b = acc[g][i + 1];
          acc[g][i] = a * c - b * s;
          acc[g][i + 1] = a * s + b * c;
        }
      }
    }
    bf16* o = p.out + ((size_t)m * p.H + hh + g) * HD + lane * DPL;
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = __float2bfloat16(acc[g][i]);
  }
}

// ------------------------------------------------------------------------------------------
// Hash routing: expert ids come from a table; weights are the normalised sqrt(softplus) scores.

__global__ void __launch_bounds__(256) hash_route_kernel(const bf16* __restrict__ x, const float* __restrict__ gate_w, const int* __restrict__ tid2eid,
                                                        const int* __restrict__ tokens, int H, int topk, int score_func, float route_scale,
                                                        int* ids, float* weights) {
  __shared__ float sc[32];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int k = warp; k < topk; k += nw) {
    const int e = tid2eid[(size_t)tokens[t] * topk + k];
    float dot = 0.f;
    for (int i = lane; i < H; i += 32) dot += __bfloat162float(x[(size_t)t * H + i]) * gate_w[(size_t)e * H + i];
    dot = warp_sum(dot);
    if (lane == 0) {
      sc[k] = score_func == 1 ? sigmoidf_(dot) : sqrtf(softplusf_(dot));
      ids[(size_t)t * topk + k] = e;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int k = 0; k < topk; ++k) s += sc[k];
    for (int k = 0; k < topk; ++k) weights[(size_t)t * topk + k] = sc[k] / s * route_scale;
  }
}

}  // namespace

// ==========================================================================================
// C entry points

PK_API int pk_dsv4_hc_pre(const float* h, const float* fn, const float* scale, const float* base, const float* gamma, int M,
                          int dim, int hc, int iters, int head_mode, float hc_eps, float norm_eps, void* x_out, float* x_raw,
                          float* post, float* comb, cudaStream_t stream) {
  const int mix = head_mode ? hc : (2 + hc) * hc;
  if (M < 1 || hc < 1 || hc > kHcMax || mix > kMixMax || (dim & 3) != 0 || dim * 4 > 160 * 1024) return PK_ERR_BAD_ARG;
  if (!head_mode && (post == nullptr || comb == nullptr)) return PK_ERR_BAD_ARG;
  HcPreParams p{h, fn, scale, base, gamma, M, dim, hc, mix, iters, head_mode, hc_eps, norm_eps, (pk::bf16*)x_out, x_raw, post, comb};
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(hc_pre_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  hc_pre_kernel<<<M, kHcThreads, (size_t)dim * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_dsv4_hc_post(const float* y, const float* y2, const float* h, const float* post, const float* comb, int M, int dim,
                           int hc, float* h_out, cudaStream_t stream) {
  if (M < 1 || hc < 1 || hc > kHcMax) return PK_ERR_BAD_ARG;
  hc_post_kernel<<<dim3((dim + 255) / 256, M), 256, 0, stream>>>(y, y2, h, post, comb, dim, hc, h_out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_dsv4_head_prep(void* x, const int* pos, const float* cos_t, const float* sin_t, int M, int H, int hd, int rd,
                             int flags, float eps, cudaStream_t stream) {
  if (M < 1 || H < 1 || hd < rd || (rd & 1) || ((flags & 8) && hd != 128)) return PK_ERR_BAD_ARG;
  HeadPrepParams p{(pk::bf16*)x, pos, cos_t, sin_t, H, hd, rd, flags, eps};
  head_prep_kernel<<<dim3(M, H), 128, (size_t)hd * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_dsv4_kv_prep_rows(const float* kv, const float* gamma, const int* pos, const int* dst_rows, const float* cos_t,
                                const float* sin_t, int M, int hd, int rd, int ring, float eps, void* dst, cudaStream_t stream);

PK_API int pk_dsv4_kv_prep(const float* kv, const float* gamma, const int* pos, const float* cos_t, const float* sin_t, int M,
                           int hd, int rd, int ring, float eps, void* dst, cudaStream_t stream) {
  return pk_dsv4_kv_prep_rows(kv, gamma, pos, nullptr, cos_t, sin_t, M, hd, rd, ring, eps, dst, stream);
}

// dst_rows (may be null) names the destination row of every input row instead of pos % ring.
PK_API int pk_dsv4_kv_prep_rows(const float* kv, const float* gamma, const int* pos, const int* dst_rows, const float* cos_t,
                                const float* sin_t, int M, int hd, int rd, int ring, float eps, void* dst, cudaStream_t stream) {
  if (M < 1 || hd < rd || ((hd - rd) & 63) != 0 || (hd - rd) / 64 > 16 || ring < 1) return PK_ERR_BAD_ARG;
  KvPrepParams p{kv, gamma, pos, cos_t, sin_t, hd, rd, ring, eps, (pk::bf16*)dst, dst_rows};
  kv_prep_kernel<<<M, 128, (size_t)hd * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Rows pos0 .. pos0+M-1. Entries completed by this call are written to dst; the ring then takes the
// last `slots` rows of the call. slots >= 2*ratio (overlap) or ratio; a larger ring keeps rows that a
// later call may still need after the caller rewinds its position (speculative decoding).
PK_API int pk_dsv4_compress(const float* proj, const float* ape, float* ring, const float* gamma, const float* cos_t,
                            const float* sin_t, int pos0, int M, int ratio, int cd, int overlap, int slots, int rd, int rotate,
                            float eps, void* dst, cudaStream_t stream) {
  if (M < 1 || ratio < 1 || cd < rd || (rotate && cd != 128) || (!rotate && (((cd - rd) & 63) != 0 || (cd - rd) / 64 > 16)))
    return PK_ERR_BAD_ARG;
  if (slots < (overlap ? 2 : 1) * ratio) return PK_ERR_BAD_ARG;
  // entries c whose completing position (c+1)*ratio - 1 lies in [pos0, pos0 + M)
  const int c_first = pos0 / ratio;
  const int c_last = (pos0 + M) / ratio - 1;
  CompressParams p{proj, ape, ring, gamma, cos_t, sin_t, pos0, M, ratio, cd, overlap, slots, rd, rotate, c_first, eps, (pk::bf16*)dst};
  if (c_last >= c_first) {
    compress_pool_kernel<<<c_last - c_first + 1, 128, (size_t)cd * 4, stream>>>(p);
    PK_CHECK_LAUNCH();
  }
  compress_ring_kernel<<<min(M, slots), 128, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_dsv4_index_score(const void* q, const void* k, const float* w, const int* pos, int M, int ih, int ratio, int ld,
                               int ldw, float wscale, float* score, cudaStream_t stream) {
  if (M < 1 || ih < 1 || ld < 1 || (size_t)ih * 129 * 4 > 96 * 1024) return PK_ERR_BAD_ARG;
  IndexScoreParams p{(const pk::bf16*)q, (const pk::bf16*)k, w, pos, ih, ratio, ld, ldw, wscale, score};
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(index_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  index_score_kernel<<<dim3((ld + 127) / 128, M), 128, (size_t)ih * 129 * 4, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// rope_pos (may be null) gives the positions for the inverse RoPE when they differ from the positions that define the
// window (draft blocks: every draft query sees the committed window but sits at its own position).
PK_API int pk_dsv4_sparse_attn_ex(const void* q, const void* kv, const int* pos, const int* rope_pos, const int* sel, const float* sink,
                                  const float* cos_t, const float* sin_t, int M, int H, int hd, int win, int ring, int ratio,
                                  int mode, int ksel, int rd, float scale, void* out, cudaStream_t stream);

PK_API int pk_dsv4_sparse_attn(const void* q, const void* kv, const int* pos, const int* sel, const float* sink,
                               const float* cos_t, const float* sin_t, int M, int H, int hd, int win, int ring, int ratio,
                               int mode, int ksel, int rd, float scale, void* out, cudaStream_t stream) {
  return pk_dsv4_sparse_attn_ex(q, kv, pos, nullptr, sel, sink, cos_t, sin_t, M, H, hd, win, ring, ratio, mode, ksel, rd, scale, out, stream);
}

PK_API int pk_dsv4_sparse_attn_ex(const void* q, const void* kv, const int* pos, const int* rope_pos, const int* sel, const float* sink,
                                  const float* cos_t, const float* sin_t, int M, int H, int hd, int win, int ring, int ratio,
                                  int mode, int ksel, int rd, float scale, void* out, cudaStream_t stream) {
  // win == 0 (no window rows, entries start at row `ring`) serves latent attention over a plain position-indexed cache:
  // mode 1 with ratio 1 is dense causal attention, mode 2 attends the selected rows; sink may be null then
  if (M < 1 || H < 1 || win < 0 || ring < win || (win == 0 && mode == 0) || (mode == 2 && sel == nullptr) || (mode == 1 && ratio < 1)) return PK_ERR_BAD_ARG;
  if (sink == nullptr && win > 0) return PK_ERR_BAD_ARG;
  if (((uintptr_t)kv & 15) != 0 || ((uintptr_t)q & 3) != 0) return PK_ERR_BAD_ARG;     // key rows are read with 16-byte loads
  SparseAttnParams p{(const pk::bf16*)q, (const pk::bf16*)kv, pos, rope_pos, sel, sink, cos_t, sin_t, H, win, ring, ratio, mode, ksel, rd,
                     scale, (pk::bf16*)out};
  // Heads per warp (the key row is read once for all of them): measured at 64 rows x 64 heads x 640 keys of 512,
  // one head per warp 380 us, two 427 us, four 647 us (the registers of the extra accumulators cost more residency
  // than the shared loads save once the row is read with 16-byte loads), so one is the default;
  // POCKET_SPARSE_ATTN_G = 2 or 4 selects the others.
  static const int forced_g = [] {
    const char* e = getenv("POCKET_SPARSE_ATTN_G");
    return e ? atoi(e) : 0;
  }();
  int G = 1;
  if ((forced_g == 1 || forced_g == 2 || forced_g == 4) && H % forced_g == 0) G = forced_g;
  const int warps_needed = H / G;
  const int wpb = warps_needed >= 4 ? 4 : warps_needed;
  const dim3 grid(M, (warps_needed + wpb - 1) / wpb);
#define PK_SPARSE_ATTN_LAUNCH(GG)                                                                                  \
  do {                                                                                                             \
    if (hd == 512) sparse_attn_kernel<16, GG><<<grid, wpb * 32, 0, stream>>>(p);                                   \
    else if (hd == 128) sparse_attn_kernel<4, GG><<<grid, wpb * 32, 0, stream>>>(p);                               \
    else if (hd == 576) sparse_attn_kernel<18, GG><<<grid, wpb * 32, 0, stream>>>(p); /* MLA latent 512 + rope 64 */ \
    else if (hd == 320) sparse_attn_kernel<10, GG><<<grid, wpb * 32, 0, stream>>>(p); /* latent 256 + rope 64 */    \
    else return PK_ERR_UNSUPPORTED;                                                                                \
  } while (0)
  if (G == 4) PK_SPARSE_ATTN_LAUNCH(4);
  else if (G == 2) PK_SPARSE_ATTN_LAUNCH(2);
  else PK_SPARSE_ATTN_LAUNCH(1);
#undef PK_SPARSE_ATTN_LAUNCH
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_dsv4_hash_route(const void* x, const float* gate_w, const int* tid2eid, const int* tokens, int T, int H, int topk,
                              int score_func, float route_scale, int* ids, float* weights, cudaStream_t stream) {
  if (T < 1 || topk < 1 || topk > 32 || score_func == 0) return PK_ERR_BAD_ARG;
  hash_route_kernel<<<T, 256, 0, stream>>>((const pk::bf16*)x, gate_w, tid2eid, tokens, H, topk, score_func,
                                           route_scale, ids, weights);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

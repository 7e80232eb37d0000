// Weight-streaming small-batch linear for decode and speculative verify (1..8 rows).
//
// y[m, n] = sum_k x[m, k] * W[n, k]    with W either FP8 E4M3 carrying one fp32 scale per
// 128x128 block (the Safetensors FP8 layout: w = e4m3(code) * scale_inv[n/128, k/128]) or
// plain bf16 rows appended after the FP8 rows (router / gate projections, lm_head).
//
// The kernel is bandwidth bound, so everything around the product is fused into it:
//   prologue  x = resid + sum_r parts[r]      (the reduce side of a push-based all-reduce:
//                                              every rank's partial already sits in local
//                                              memory; the block waits on the ranks' flags)
//             x = rmsnorm(x) * (1 + gamma) or * gamma
//   epilogue  store bf16 / fp32, SiLU(gate) * up, or push the fp32 partial rows into every
//             peer's slot buffer and publish a flag (the scatter side of the all-reduce).
//
// Arithmetic: the activations are staged in shared memory as fp16 scaled by a power of two
// so that |x| <= 1; FP8 codes unpack to fp16 pairs with one instruction, products are
// accumulated four at a time with packed fp16 FMAs (|sum| <= 4 * 448) and then folded into
// fp32 with the block scale. This keeps the instruction count per weight byte low enough
// for the loads, not the ALUs, to set the pace.
//
// Behavioural counterpart in the reference: cpp_engine/cuda/qwen_half_ops.cu:89-374
// (fp8_matvec_f16*, fp8_matmul_f16_small_batch, fp8_swiglu_*), which are separate SIMT
// kernels with an LUT decode and NCCL all-reduces between them.
#include <cstdlib>

#include "../common/pk_comm.cuh"
#include "../common/pk_common.cuh"
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSmemBytes = 108 * 1024;  // staged fp16 activations + one fp32 scratch row

struct MatvecParams {
  const uint8_t* W;      // [N, K] e4m3
  const float* scale;    // [ceil(N/128), ceil(K/128)]
  const bf16* Wb;        // [Nb, K] bf16 rows that follow the fp8 rows (may be null)
  int N, Nb, K;
  int M;                 // rows of x
  // prologue
  const bf16* x_in;      // [M, K] or null
  const float* parts;    // [nparts, M, K] fp32 or null
  int nparts;
  bf16* hidden_out;      // [M, K]: x before the norm, written by block 0 (may be null)
  const float* gamma;    // [K] or null
  int norm_mode;         // 1: *(1+gamma), 2: *gamma
  int flat_path;         // 1: blocks own whole row pairs and their warps split the block's k-iterations evenly
  int self_prefetch;     // flat path: L2-prefetch the rest of each warp's first stretch before the staging
  unsigned long long* dbg;  // optional phase timestamps (see pk_matvec_set_debug); null in normal use
  float eps;
  PkWait wait;
  // epilogue
  int epi;               // 0 bf16 y[M, Nout], 1 swiglu -> bf16 y[M, N/2], 2 fp32 y[M, Nout], 3 push
  bf16* y_bf16;
  float* y_f32;
  int ldy;               // row stride of y (elements)
  PkPush push;
  int kc;                // staged chunk length (multiple of 512)
  int single_chunk;
  // ring variant: byte offsets inside the dynamic shared memory
  int use_scratch;       // 0: no norm and no partial sums, the activations are staged straight from x_in
  int acc_off, ring_off, bar_off, scale_off;
};

// Position (in halves) of element k inside a staged row. Within each run of 512 elements the
// two 16-byte pieces of a lane's 16 values sit 256 halves apart, so a warp's LDS.128 touches
// 32 consecutive 16-byte words (no bank conflicts).
__device__ __forceinline__ int staged_index(int k) {
  const int blk = k >> 9, r = k & 511;
  return (blk << 9) + (((r >> 3) & 1) << 8) + ((r >> 4) << 3) + (r & 7);
}

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t v16) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v16, __NV_E4M3);
  return *reinterpret_cast<__half2*>(&h);
}

// 16 fp8 codes times 16 staged activations -> fp32 partial (unscaled).
__device__ __forceinline__ float dot16_fp8(const uint4& w, const uint4& x0, const uint4& x1) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  const uint32_t xx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __half2 lo = e4m3x2_to_half2(ww[j] & 0xffffu);
    const __half2 hi = e4m3x2_to_half2(ww[j] >> 16);
    a0 = __hfma2(lo, *reinterpret_cast<const __half2*>(&xx[2 * j]), a0);
    a1 = __hfma2(hi, *reinterpret_cast<const __half2*>(&xx[2 * j + 1]), a1);
  }
  const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
  return (f0.x + f0.y) + (f1.x + f1.y);
}

__device__ __forceinline__ float dot16_bf16(const uint4& w0, const uint4& w1, const uint4& x0, const uint4& x1) {
  const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  const uint32_t xx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 xv = __half22float2(*reinterpret_cast<const __half2*>(&xx[j]));
    acc = fmaf(__uint_as_float(ww[j] << 16), xv.x, acc);
    acc = fmaf(__uint_as_float(ww[j] & 0xffff0000u), xv.y, acc);
  }
  return acc;
}

// A batch of four k-iterations for a row pair: eight 16-byte loads in flight per lane.
struct Fp8Batch {
  uint4 a[4], b[4];
  float sa[4], sb[4];
};

__device__ __forceinline__ void load_fp8_batch(Fp8Batch& bt, const uint8_t* w0p, const uint8_t* w1p,
                                               const float* s0p, const float* s1p, int it0, int klen, int lane) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int ka = ((it0 + u) << 9) + (lane << 4);
    const bool ok = ka < klen;
    bt.a[u] = ok ? ld_stream_u4(w0p + ka) : make_uint4(0, 0, 0, 0);
    bt.b[u] = ok ? ld_stream_u4(w1p + ka) : make_uint4(0, 0, 0, 0);
    bt.sa[u] = ok ? __ldg(s0p + (ka >> 7)) : 0.f;
    bt.sb[u] = ok ? __ldg(s1p + (ka >> 7)) : 0.f;
  }
}

template <int M>
__device__ __forceinline__ void consume_fp8_batch(const Fp8Batch& bt, const __half* xs, int kc, int it0, int iters,
                                                  int lane, float (&acc0)[M], float (&acc1)[M]) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    // The staged chunk ends at iteration `iters`; nothing beyond it may be read.
    if (it0 + u >= iters) break;
    const int base = ((it0 + u) << 9) + (lane << 3);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 x0 = *reinterpret_cast<const uint4*>(xs + m * kc + base);
      const uint4 x1 = *reinterpret_cast<const uint4*>(xs + m * kc + base + 256);
      acc0[m] = fmaf(dot16_fp8(bt.a[u], x0, x1), bt.sa[u], acc0[m]);
      acc1[m] = fmaf(dot16_fp8(bt.b[u], x0, x1), bt.sb[u], acc1[m]);
    }
  }
}

// Raw (pre-norm) value of eight consecutive elements of row m: x_in + sum of parts.
__device__ __forceinline__ void load8(const MatvecParams& p, int M, int m, int k, float (&v)[8]) {
  uint4 xv = make_uint4(0, 0, 0, 0);
  if (p.x_in) xv = __ldg(reinterpret_cast<const uint4*>(p.x_in + (size_t)m * p.K + k));
  const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
  for (int r = 0; r < p.nparts; ++r) {
    const float4* pp = reinterpret_cast<const float4*>(p.parts + ((size_t)r * M + m) * p.K + k);
    const float4 a = pp[0], b = pp[1];
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
    v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
}

// Round to the bf16 residual stream; optionally store it; returns the rounded values.
__device__ __forceinline__ void round_store8(const MatvecParams& p, int m, int k, float (&v)[8], bool store) {
  uint32_t packed[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    packed[j] = *reinterpret_cast<const uint32_t*>(&h2);
    v[2 * j] = __uint_as_float(packed[j] << 16);
    v[2 * j + 1] = __uint_as_float(packed[j] & 0xffff0000u);
  }
  if (store)
    *reinterpret_cast<uint4*>(p.hidden_out + (size_t)m * p.K + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

__device__ __forceinline__ void gamma8(const MatvecParams& p, int k, float (&v)[8]) {
  if (p.gamma == nullptr) return;
  const float one = p.norm_mode == 1 ? 1.f : 0.f;
  const float4 a = __ldg(reinterpret_cast<const float4*>(p.gamma + k));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p.gamma + k + 4));
  v[0] *= one + a.x; v[1] *= one + a.y; v[2] *= one + a.z; v[3] *= one + a.w;
  v[4] *= one + b.x; v[5] *= one + b.y; v[6] *= one + b.z; v[7] *= one + b.w;
}

// Two block-wide reductions at once: sum of a, max of b.
__device__ __forceinline__ void block_sum_max(float& a, float& b, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_max(b);
  __syncthreads();
  if (lane == 0) {
    red[warp] = a;
    red[16 + warp] = b;
  }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    ta += red[w];
    tb = fmaxf(tb, red[16 + w]);
  }
  a = ta;
  b = tb;
}

// Final staged value: normalise, round to bf16 (what an unfused pipeline would have stored),
// scale into [-1, 1] and write fp16 at the permuted position.
__device__ __forceinline__ void stage8(__half* xs_row, int k_in_chunk, const float (&t)[8], float rs, float cinv,
                                       bool round_bf16) {
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float a = t[2 * j] * rs, b = t[2 * j + 1] * rs;
    if (round_bf16) {
      a = __bfloat162float(__float2bfloat16(a));
      b = __bfloat162float(__float2bfloat16(b));
    }
    const __half2 h = __floats2half2_rn(a * cinv, b * cinv);
    out[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(xs_row + staged_index(k_in_chunk)) = make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ float pow2_at_least(float a) {
  // smallest power of two >= a (a > 0), as a float
  int e;
  const float m = frexpf(a, &e);  // a = m * 2^e, m in [0.5, 1)
  return ldexpf(1.f, m == 0.5f ? e - 1 : e);
}

template <int M>
__global__ void __launch_bounds__(kThreads, 2) matvec_kernel(const MatvecParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);                         // [M][kc]
  float* scratch = reinterpret_cast<float*>(smem_raw + (size_t)M * p.kc * 2);  // [K] (single chunk only)
  __shared__ float red[40];
  __shared__ float s_rs[8], s_c[8];  // per row: rstd (or 1) and the power-of-two range scale

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, kc = p.kc;
  const bool swiglu = p.epi == 1;
  if (p.dbg != nullptr && tid == 0) atomicMin(p.dbg + 0, global_timer_ns());
  const int half_n = p.N >> 1;
  // Row pairs: a warp owns two output rows at a time (gate_j and up_j for SwiGLU, else
  // rows 2g and 2g+1), so that every staged activation is read once per two weight rows.
  const int total_rows = p.N + p.Nb;
  const int n_groups = swiglu ? half_n : (total_rows + 1) >> 1;
  const int warps_total = gridDim.x * kWarps;
  const int gwarp = blockIdx.x * kWarps + warp;
  const int kb_count = (K + 127) >> 7;
  const bool round_x = p.gamma != nullptr;

  // Weights do not depend on the activations: issue the first batch of this warp's first
  // row pair before the prologue so that the HBM latency overlaps the norm.
  Fp8Batch bt;
  bool have_pre = false;
  // Flat path: the block owns row pairs [g_lo, g_hi); their k-iterations, laid end to end, are cut
  // into one contiguous range per warp, so every warp streams the same number of bytes whatever the
  // row count. A warp adds the partial sums of each row pair it touches into shared memory.
  const int iters_all = (K + 511) >> 9;
  const int g_lo = (int)(((long long)blockIdx.x * n_groups) / gridDim.x);
  const int g_hi = (int)(((long long)(blockIdx.x + 1) * n_groups) / gridDim.x);
  const int flat_total = (g_hi - g_lo) * iters_all;
  const int flat_begin = (int)(((long long)warp * flat_total) / kWarps);
  const int flat_end = (int)(((long long)(warp + 1) * flat_total) / kWarps);
  if (p.flat_path) {
    if (flat_begin < flat_end) {
      const int gl = flat_begin / iters_all, it = flat_begin - gl * iters_all, g0 = g_lo + gl;
      const int it_stop = min(iters_all, it + (flat_end - flat_begin));
      const int r0 = swiglu ? g0 : 2 * g0;
      if (r0 < p.N) {
        const int r1c = swiglu ? g0 + half_n : (2 * g0 + 1 < p.N ? 2 * g0 + 1 : r0);
        load_fp8_batch(bt, p.W + (size_t)r0 * K, p.W + (size_t)r1c * K, p.scale + (size_t)(r0 >> 7) * kb_count,
                       p.scale + (size_t)(r1c >> 7) * kb_count, it, min(K, it_stop << 9), lane);
        have_pre = true;
        // Ask L2 for the rest of this warp's first stretch (up to 16 KB per row) so that HBM keeps streaming while
        // the block stages the activations.
        if (p.self_prefetch && lane == 0) {
          const unsigned k_from = (unsigned)min(K, (it + 4) << 9), k_to = (unsigned)min(K, it_stop << 9);
          if (k_to > k_from) {
            const unsigned n = min(k_to - k_from, 16384u) & ~15u;
            if (n) {
              asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.W + (size_t)r0 * K + k_from), "r"(n) : "memory");
              asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.W + (size_t)r1c * K + k_from), "r"(n) : "memory");
            }
          }
        }
      }
    }
  } else {
    const int g0 = gwarp;
    const int r0 = swiglu ? g0 : 2 * g0;
    if (g0 < n_groups && r0 < p.N) {
      const int r1c = swiglu ? g0 + half_n : (2 * g0 + 1 < p.N ? 2 * g0 + 1 : r0);
      load_fp8_batch(bt, p.W + (size_t)r0 * K, p.W + (size_t)r1c * K, p.scale + (size_t)(r0 >> 7) * kb_count,
                     p.scale + (size_t)(r1c >> 7) * kb_count, 0, min(kc, K), lane);
      have_pre = true;
    }
  }

  // Programmatic dependent launch (when enabled): this grid may have been scheduled while the
  // previous kernel of the stream was still draining. Everything above touched weights only;
  // activations, partial sums and every output are behind this point.
  pdl_wait();
  pdl_trigger();
  if (p.parts != nullptr && p.wait.flag != nullptr) {
    if (tid == 0) wait_all_ranks(p.wait);
    __syncthreads();
  }

  const int nchunks8 = K >> 3;
  const bool write_hidden = p.hidden_out != nullptr && blockIdx.x == 0;
  if (p.single_chunk) {
    // One pass over global memory: t = bf16(x + parts) * (1 + gamma) into the fp32 scratch
    // row with the sum of squares and the largest magnitude, then a shared-memory pass that
    // normalises, scales and converts.
    for (int m = 0; m < M; ++m) {
      float ss = 0.f, amax = 0.f;
      for (int c0 = tid; c0 < nchunks8; c0 += kThreads * 4) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * kThreads;
          if (c < nchunks8) load8(p, M, m, c * 8, v[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * kThreads;
          if (c >= nchunks8) continue;
          if (p.parts != nullptr || write_hidden) round_store8(p, m, c * 8, v[u], write_hidden);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[u][j] * v[u][j];
          gamma8(p, c * 8, v[u]);
#pragma unroll
          for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[u][j]));
          *reinterpret_cast<float4*>(scratch + c * 8) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
          *reinterpret_cast<float4*>(scratch + c * 8 + 4) = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
        }
      }
      block_sum_max(ss, amax, red);
      const float rs = p.gamma != nullptr ? rsqrtf(ss / (float)K + p.eps) : 1.f;
      const float c = pow2_at_least(fmaxf(amax * rs, 1e-30f));
      if (tid == 0) s_c[m] = c;
      const float cinv = 1.f / c;
      __half* row = xs + m * kc;
      for (int c8 = tid; c8 < (kc >> 3); c8 += kThreads) {
        float t[8];
        if (c8 < nchunks8) {
          const float4 a = *reinterpret_cast<const float4*>(scratch + c8 * 8);
          const float4 b = *reinterpret_cast<const float4*>(scratch + c8 * 8 + 4);
          t[0] = a.x; t[1] = a.y; t[2] = a.z; t[3] = a.w; t[4] = b.x; t[5] = b.y; t[6] = b.z; t[7] = b.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) t[j] = 0.f;
        }
        stage8(row, c8 * 8, t, rs, cinv, round_x);
      }
      __syncthreads();  // the scratch row is reused by the next m
    }
  } else {
    // The row does not fit: statistics first (one extra pass over L2-resident data).
    for (int m = 0; m < M; ++m) {
      float ss = 0.f, amax = 0.f;
      for (int c = tid; c < nchunks8; c += kThreads) {
        float v[8];
        load8(p, M, m, c * 8, v);
        if (p.parts != nullptr) round_store8(p, m, c * 8, v, false);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
        gamma8(p, c * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      }
      block_sum_max(ss, amax, red);
      const float rs = p.gamma != nullptr ? rsqrtf(ss / (float)K + p.eps) : 1.f;
      if (tid == 0) {
        s_rs[m] = rs;
        s_c[m] = pow2_at_least(fmaxf(amax * rs, 1e-30f));
      }
    }
    __syncthreads();
  }

  if (p.dbg != nullptr && tid == 0) {
    atomicMin(p.dbg + 1, global_timer_ns());
    atomicMax(p.dbg + 2, global_timer_ns());
  }
  if (p.flat_path) {
    float* s_acc = scratch;                         // [row pairs of the block][2][M]; the scratch row is free now
    const int ngb = g_hi - g_lo;
    __shared__ int s_edge_g[kWarps][2];
    __shared__ float s_edge_v[kWarps][2][2 * M];
    for (int i = tid; i < ngb * 2 * M; i += kThreads) s_acc[i] = 0.f;
    if (tid < kWarps * 2) s_edge_g[tid >> 1][tid & 1] = -1;
    __syncthreads();
    int pos = flat_begin;
    while (pos < flat_end) {
      const int gl = pos / iters_all, it = pos - gl * iters_all, g = g_lo + gl;
      const int it_stop = min(iters_all, it + (flat_end - pos));
      const int klim = min(K, it_stop << 9);
      const int r0 = swiglu ? g : 2 * g;
      const int r1 = swiglu ? g + half_n : 2 * g + 1;
      float a0[M], a1[M];
#pragma unroll
      for (int m = 0; m < M; ++m) a0[m] = a1[m] = 0.f;
      if (r0 < p.N) {
        const int r1c = r1 < p.N ? r1 : r0;
        const uint8_t* w0p = p.W + (size_t)r0 * K;
        const uint8_t* w1p = p.W + (size_t)r1c * K;
        const float* s0p = p.scale + (size_t)(r0 >> 7) * kb_count;
        const float* s1p = p.scale + (size_t)(r1c >> 7) * kb_count;
        bool loaded = have_pre && pos == flat_begin;
#pragma unroll 1
        for (int it0 = it; it0 < it_stop; it0 += 4) {
          if (!loaded) load_fp8_batch(bt, w0p, w1p, s0p, s1p, it0, klim, lane);
          loaded = false;
          consume_fp8_batch<M>(bt, xs, kc, it0, it_stop, lane, a0, a1);
        }
      } else {
        const int r1c = r1 < total_rows ? r1 : r0;
        const bf16* w0p = p.Wb + (size_t)(r0 - p.N) * K;
        const bf16* w1p = p.Wb + (size_t)(r1c - p.N) * K;
#pragma unroll 2
        for (int i2 = it; i2 < it_stop; ++i2) {
          const int ka = (i2 << 9) + (lane << 4);
          if (ka < K) {
            const uint4 w00 = __ldg(reinterpret_cast<const uint4*>(w0p + ka));
            const uint4 w01 = __ldg(reinterpret_cast<const uint4*>(w0p + ka + 8));
            const uint4 w10 = __ldg(reinterpret_cast<const uint4*>(w1p + ka));
            const uint4 w11 = __ldg(reinterpret_cast<const uint4*>(w1p + ka + 8));
            const int base = (i2 << 9) + (lane << 3);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const uint4 x0 = *reinterpret_cast<const uint4*>(xs + m * kc + base);
              const uint4 x1 = *reinterpret_cast<const uint4*>(xs + m * kc + base + 256);
              a0[m] += dot16_bf16(w00, w01, x0, x1);
              a1[m] += dot16_bf16(w10, w11, x0, x1);
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        a0[m] = warp_sum(a0[m]);
        a1[m] = warp_sum(a1[m]);
      }
      if (lane == 0) {
        // A row pair wholly inside this warp's range has one writer. Only the first and the last
        // segment of a range can be partial; they go to this warp's two edge slots and are added in
        // warp order below, so the result does not depend on timing.
        const bool whole = it == 0 && it_stop == iters_all;
        const int e = pos == flat_begin ? 0 : 1;
        float* dst0 = whole ? s_acc + (gl * 2) * M : &s_edge_v[warp][e][0];
        float* dst1 = whole ? s_acc + (gl * 2 + 1) * M : &s_edge_v[warp][e][M];
        if (!whole) s_edge_g[warp][e] = gl;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          dst0[m] = a0[m];
          dst1[m] = a1[m];
        }
      }
      pos += it_stop - it;
    }
    if (p.dbg != nullptr && lane == 0) {
      atomicMin(p.dbg + 3, global_timer_ns());
      atomicMax(p.dbg + 4, global_timer_ns());
    }
    __syncthreads();
    for (int idx = tid; idx < ngb * M; idx += kThreads) {
      const int gl = idx / M, m = idx - gl * M, g = g_lo + gl;
      float v0 = s_acc[(gl * 2) * M + m], v1 = s_acc[(gl * 2 + 1) * M + m];
#pragma unroll
      for (int w = 0; w < kWarps; ++w)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          if (s_edge_g[w][e] == gl) {
            v0 += s_edge_v[w][e][m];
            v1 += s_edge_v[w][e][M + m];
          }
      v0 *= s_c[m];
      v1 *= s_c[m];
      if (swiglu) {
        p.y_bf16[(size_t)m * p.ldy + g] = __float2bfloat16(silu(v0) * v1);
      } else {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int n = 2 * g + r;
          if (n >= total_rows) continue;
          const float v = r == 0 ? v0 : v1;
          if (p.epi == 0) {
            p.y_bf16[(size_t)m * p.ldy + n] = __float2bfloat16(v);
          } else if (p.epi == 2) {
            p.y_f32[(size_t)m * p.ldy + n] = v;
          } else {
            const size_t off = ((size_t)p.push.rank * M + m) * p.ldy + n;
            for (int pr = 0; pr < p.push.world; ++pr) p.push.dst[pr][off] = v;
          }
        }
      }
    }
    if (p.epi == 3) publish_when_grid_done(p.push);
    return;
  }
  float acc[2][M];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kc) {
    const int klen = min(kc, K - k0);
    if (!p.single_chunk) {
      if (k0 > 0) __syncthreads();
      for (int m = 0; m < M; ++m) {
        const float rs = s_rs[m], cinv = 1.f / s_c[m];
        for (int c8 = tid; c8 < (kc >> 3); c8 += kThreads) {
          float t[8];
          if (c8 * 8 < klen) {
            load8(p, M, m, k0 + c8 * 8, t);
            if (p.parts != nullptr || write_hidden) round_store8(p, m, k0 + c8 * 8, t, write_hidden);
            gamma8(p, k0 + c8 * 8, t);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = 0.f;
          }
          stage8(xs + m * kc, c8 * 8, t, rs, cinv, round_x);
        }
      }
      __syncthreads();
    }

    // ---- stream the weight rows ----
    for (int g = gwarp; g < n_groups; g += warps_total) {
      int row[2];
      if (swiglu) {
        row[0] = g;
        row[1] = g + half_n;
      } else {
        row[0] = 2 * g;
        row[1] = 2 * g + 1;
      }
      const int iters = (klen + 511) >> 9;
      if (row[0] < p.N) {
        // Both rows are FP8 (N is even).
        const bool has1 = row[1] < p.N;
        const uint8_t* w0p = p.W + (size_t)row[0] * K + k0;
        const uint8_t* w1p = p.W + (size_t)(has1 ? row[1] : row[0]) * K + k0;
        const float* s0p = p.scale + (size_t)(row[0] >> 7) * kb_count + (k0 >> 7);
        const float* s1p = p.scale + (size_t)((has1 ? row[1] : row[0]) >> 7) * kb_count + (k0 >> 7);
        bool loaded = have_pre && k0 == 0 && g == gwarp;
#pragma unroll 1
        for (int it0 = 0; it0 < iters; it0 += 4) {
          if (!loaded) load_fp8_batch(bt, w0p, w1p, s0p, s1p, it0, klen, lane);
          loaded = false;
          consume_fp8_batch<M>(bt, xs, kc, it0, iters, lane, acc[0], acc[1]);
        }
      } else {
        const bool has1 = row[1] < total_rows;
        const bf16* w0p = p.Wb + (size_t)(row[0] - p.N) * K + k0;
        const bf16* w1p = p.Wb + (size_t)((has1 ? row[1] : row[0]) - p.N) * K + k0;
#pragma unroll 2
        for (int it = 0; it < iters; ++it) {
          const int ka = (it << 9) + (lane << 4);
          if (ka < klen) {
            const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(w0p + ka));
            const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(w0p + ka + 8));
            const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(w1p + ka));
            const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(w1p + ka + 8));
            const int base = (it << 9) + (lane << 3);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const uint4 x0 = *reinterpret_cast<const uint4*>(xs + m * kc + base);
              const uint4 x1 = *reinterpret_cast<const uint4*>(xs + m * kc + base + 256);
              acc[0][m] += dot16_bf16(a0, a1, x0, x1);
              acc[1][m] += dot16_bf16(b0, b1, x0, x1);
            }
          }
        }
      }

      // ---- flush this group when its last chunk is done ----
      if (k0 + kc >= K) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]) * s_c[m];
        if (lane == 0) {
          if (swiglu) {
#pragma unroll
            for (int m = 0; m < M; ++m)
              p.y_bf16[(size_t)m * p.ldy + g] = __float2bfloat16(silu(acc[0][m]) * acc[1][m]);
          } else {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const int n = row[r];
              if (n >= total_rows) continue;
#pragma unroll
              for (int m = 0; m < M; ++m) {
                const float v = acc[r][m];
                if (p.epi == 0) {
                  p.y_bf16[(size_t)m * p.ldy + n] = __float2bfloat16(v);
                } else if (p.epi == 2) {
                  p.y_f32[(size_t)m * p.ldy + n] = v;
                } else {
                  // Push: slot layout [world][M][ldy]; this rank's rows go to every peer.
                  const size_t off = ((size_t)p.push.rank * M + m) * p.ldy + n;
                  for (int pr = 0; pr < p.push.world; ++pr) p.push.dst[pr][off] = v;
                }
              }
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
      }
    }
  }

  if (p.dbg != nullptr && lane == 0) {
    atomicMin(p.dbg + 3, global_timer_ns());
    atomicMax(p.dbg + 4, global_timer_ns());
  }
  if (p.epi == 3) publish_when_grid_done(p.push);
}

template <int M>
int launch_m(MatvecParams& p, int groups, int sm_count, cudaStream_t stream) {
  // Single chunk when M fp16 rows plus one fp32 scratch row fit; else chunks of fp16 only.
  const int kround = (p.K + 511) & ~511;
  size_t smem;
  if ((size_t)M * kround * 2 + (size_t)p.K * 4 <= (size_t)kSmemBytes) {
    p.kc = kround;
    p.single_chunk = 1;
    smem = (size_t)M * kround * 2 + (size_t)p.K * 4;
  } else {
    p.kc = ((kSmemBytes / (2 * M)) >> 9) << 9;
    p.single_chunk = 0;
    smem = (size_t)M * p.kc * 2;
  }
  int blocks = (groups + kWarps - 1) / kWarps;
  p.flat_path = 0;
  if (p.single_chunk) {
    const int cap = (sm_count > 0 ? sm_count : 148) * 2;
    const int fb = groups < cap ? groups : cap;
    const int per_block = (groups + fb - 1) / fb;
    if ((size_t)per_block * 2 * M <= (size_t)p.K) {   // the block's accumulators reuse the scratch row
      p.flat_path = 1;
      blocks = fb;
    } else if (blocks > cap) {
      blocks = cap;
    }
  }  // chunked: exactly one group per warp (one accumulator set per warp)
  if (blocks < 1) blocks = 1;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(matvec_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  PK_LAUNCH_PDL(matvec_kernel<M>, dim3(blocks), dim3(kThreads), smem, stream, p);
  return PK_OK;
}

// ------------------------------------------------------------------------------------------
// Ring variant of the flat path, for FP8 rows and one or two activation rows (decode). Each warp streams its
// weight bytes through a private shared-memory ring filled by bulk asynchronous copies (cp.async.bulk completing on
// an mbarrier), so that no registers are tied up by loads in flight and the amount in flight is set by the ring size:
// 8 KB per warp, 128 KB per SM. The first ring-full is requested before the wait on the previous kernel and before the
// activations are staged, which keeps HBM busy across the kernel boundary; afterwards the warp's lane 0 refills a slot
// as soon as the warp has read it. Weight scales of the block's (at most four) 128-row blocks sit in shared memory.
// bf16 rows that follow the FP8 rows are loaded directly, as in the other paths.

#ifndef PK_RING_BLOCKS
#define PK_RING_BLOCKS 3
#endif
constexpr int kRingBlocksPerSm = PK_RING_BLOCKS;       // resident blocks per SM the ring variant is sized for
constexpr int kRingSlots = kRingBlocksPerSm >= 3 ? 2 : 4;   // per warp
constexpr int kSlotIters = kRingBlocksPerSm >= 4 ? 1 : 2;   // k-iterations (512 weights) per slot and row
constexpr int kRowSlotBytes = kSlotIters * 512;
constexpr int kSlotBytes = 2 * kRowSlotBytes;         // a row pair
constexpr int kRingBytes = kWarps * kRingSlots * kSlotBytes;
constexpr int kRingSmemLimit = kRingBlocksPerSm >= 4 ? 55 * 1024 : kRingBlocksPerSm == 3 ? 74 * 1024 : 112 * 1024;
constexpr int kRingMaxPairsPerBlock = 64;             // keeps a block's rows inside two 128-row scale blocks per side

__device__ uint32_t g_matvec_ring_status = 0;         // first mbarrier wait that ran out (0 = none)

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   sm100::smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(sm100::smem_u32(bar))
               : "memory");
}

template <int M>
__global__ void __launch_bounds__(kThreads, kRingBlocksPerSm) matvec_ring_kernel(const MatvecParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);                            // [M][kc]
  float* scratch = reinterpret_cast<float*>(smem_raw + (size_t)M * p.kc * 2);  // [K] when use_scratch
  float* s_acc = reinterpret_cast<float*>(smem_raw + p.acc_off);               // [row pairs of the block][2][M]
  float* s_scale = reinterpret_cast<float*>(smem_raw + p.scale_off);           // [2 sides][2 row blocks][kb_count]
  __shared__ float red[40];
  __shared__ float s_c[8];
  __shared__ uint32_t s_abort;
  __shared__ int s_edge_g[kWarps][2];
  __shared__ float s_edge_v[kWarps][2][2 * M];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* ring = smem_raw + p.ring_off + (size_t)warp * kRingSlots * kSlotBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + p.bar_off) + warp * kRingSlots;
  const int K = p.K, kc = p.kc;
  const bool swiglu = p.epi == 1;
  const int half_n = p.N >> 1;
  const int total_rows = p.N + p.Nb;
  const int n_groups = swiglu ? half_n : (total_rows + 1) >> 1;
  const int kb_count = (K + 127) >> 7;
  const bool round_x = p.gamma != nullptr;
  const int iters_all = (K + 511) >> 9;
  const int g_lo = (int)(((long long)blockIdx.x * n_groups) / gridDim.x);
  const int g_hi = (int)(((long long)(blockIdx.x + 1) * n_groups) / gridDim.x);
  const int flat_total = (g_hi - g_lo) * iters_all;
  const int flat_begin = (int)(((long long)warp * flat_total) / kWarps);
  const int flat_end = (int)(((long long)(warp + 1) * flat_total) / kWarps);
  auto row0_of = [&](int g) { return swiglu ? g : 2 * g; };
  auto row1_of = [&](int g) { return swiglu ? g + half_n : (2 * g + 1 < p.N ? 2 * g + 1 : 2 * g); };   // FP8 pairs only
  const int rbA = row0_of(g_lo) >> 7, rbB = row1_of(g_lo) >> 7;

  if (tid == 0) s_abort = 0u;
  if (lane == 0) {
#pragma unroll
    for (int s2 = 0; s2 < kRingSlots; ++s2) sm100::mbar_init(&bars[s2], 1);
    sm100::mbar_fence_init();
  }
  __syncwarp();

  // Producer cursor: the next slot to request, in the same order in which the warp will read.
  int ppos = flat_begin, pk = 0;
  auto issue_next = [&]() {
    while (ppos < flat_end) {
      const int gl = ppos / iters_all, it = ppos - gl * iters_all;
      const int seg_stop = min(iters_all, it + (flat_end - ppos));
      const int n_it = min(kSlotIters, seg_stop - it);
      const int g = g_lo + gl, r0 = row0_of(g);
      ppos += n_it;
      if (r0 >= p.N) continue;   // bf16 rows do not go through the ring
      if (lane == 0) {
        const int ka = it << 9;
        const uint32_t bytes = (uint32_t)min(n_it << 9, K - ka);
        const int slot = pk % kRingSlots;
        uint8_t* dst = ring + slot * kSlotBytes;
        sm100::mbar_arrive_expect_tx(&bars[slot], 2 * bytes);
        bulk_load(dst, p.W + (size_t)r0 * K + ka, bytes, &bars[slot]);
        bulk_load(dst + kRowSlotBytes, p.W + (size_t)row1_of(g) * K + ka, bytes, &bars[slot]);
      }
      ++pk;
      return;
    }
  };
#pragma unroll 1
  for (int s2 = 0; s2 < kRingSlots; ++s2) issue_next();

  // Scales of the block's row blocks (weights only, so still ahead of the dependency wait).
  if (row0_of(g_lo) < p.N) {
    const int n_rb = (p.N + 127) >> 7;
    for (int idx = tid; idx < 4 * kb_count; idx += kThreads) {
      const int q = idx / kb_count, kb = idx - q * kb_count;
      const int rb = ((q >> 1) ? rbB : rbA) + (q & 1);
      s_scale[idx] = rb < n_rb ? __ldg(p.scale + (size_t)rb * kb_count + kb) : 0.f;
    }
  }

  pdl_wait();
  pdl_trigger();
  if (p.parts != nullptr && p.wait.flag != nullptr) {
    if (tid == 0) wait_all_ranks(p.wait);
    __syncthreads();
  }

  // ---- stage the activations ----
  const int nchunks8 = K >> 3;
  const bool write_hidden = p.hidden_out != nullptr && blockIdx.x == 0;
  for (int m = 0; m < M; ++m) {
    float ss = 0.f, amax = 0.f;
    __half* row = xs + m * kc;
    if (p.use_scratch) {
      for (int c0 = tid; c0 < nchunks8; c0 += kThreads * 4) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * kThreads;
          if (c < nchunks8) load8(p, M, m, c * 8, v[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * kThreads;
          if (c >= nchunks8) continue;
          if (p.parts != nullptr || write_hidden) round_store8(p, m, c * 8, v[u], write_hidden);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[u][j] * v[u][j];
          gamma8(p, c * 8, v[u]);
#pragma unroll
          for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[u][j]));
          *reinterpret_cast<float4*>(scratch + c * 8) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
          *reinterpret_cast<float4*>(scratch + c * 8 + 4) = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
        }
      }
    } else {
      // plain bf16 input, no norm: the range scale needs the largest magnitude only
      for (int c = tid; c < nchunks8; c += kThreads) {
        float v[8];
        load8(p, M, m, c * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      }
    }
    block_sum_max(ss, amax, red);
    const float rs = p.gamma != nullptr ? rsqrtf(ss / (float)K + p.eps) : 1.f;
    const float c = pow2_at_least(fmaxf(amax * rs, 1e-30f));
    if (tid == 0) s_c[m] = c;
    const float cinv = 1.f / c;
    for (int c8 = tid; c8 < (kc >> 3); c8 += kThreads) {
      float t[8];
      if (c8 < nchunks8) {
        if (p.use_scratch) {
          const float4 a = *reinterpret_cast<const float4*>(scratch + c8 * 8);
          const float4 b = *reinterpret_cast<const float4*>(scratch + c8 * 8 + 4);
          t[0] = a.x; t[1] = a.y; t[2] = a.z; t[3] = a.w; t[4] = b.x; t[5] = b.y; t[6] = b.z; t[7] = b.w;
        } else {
          load8(p, M, m, c8 * 8, t);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = 0.f;
      }
      stage8(row, c8 * 8, t, rs, cinv, round_x);
    }
    __syncthreads();  // the scratch row is reused by the next m; the staged rows become visible
  }

  const int ngb = g_hi - g_lo;
  for (int i = tid; i < ngb * 2 * M; i += kThreads) s_acc[i] = 0.f;
  if (tid < kWarps * 2) s_edge_g[tid >> 1][tid & 1] = -1;
  __syncthreads();

  // ---- stream ----
  int ck = 0;   // FP8 slots read so far
  int pos = flat_begin;
  while (pos < flat_end) {
    const int gl = pos / iters_all, it = pos - gl * iters_all, g = g_lo + gl;
    const int it_stop = min(iters_all, it + (flat_end - pos));
    const int r0 = row0_of(g);
    float a0[M], a1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) a0[m] = a1[m] = 0.f;
    if (r0 < p.N) {
      const float* sc0 = s_scale + ((r0 >> 7) - rbA) * kb_count;
      const float* sc1 = s_scale + (2 + (row1_of(g) >> 7) - rbB) * kb_count;
#pragma unroll 1
      for (int it0 = it; it0 < it_stop; it0 += kSlotIters) {
        const int n_it = min(kSlotIters, it_stop - it0);
        const int slot = ck % kRingSlots;
        if (!sm100::mbar_wait(&bars[slot], (uint32_t)((ck / kRingSlots) & 1), &s_abort, &g_matvec_ring_status, 31u)) break;
        const uint8_t* sp = ring + slot * kSlotBytes + (lane << 4);
#pragma unroll
        for (int u = 0; u < kSlotIters; ++u) {
          if (u >= n_it) break;
          const int ka = ((it0 + u) << 9) + (lane << 4);
          if (ka < K) {
            const uint4 wa = *reinterpret_cast<const uint4*>(sp + (u << 9));
            const uint4 wb = *reinterpret_cast<const uint4*>(sp + kRowSlotBytes + (u << 9));
            const float sa = sc0[ka >> 7], sb = sc1[ka >> 7];
            const int base = ((it0 + u) << 9) + (lane << 3);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const uint4 x0 = *reinterpret_cast<const uint4*>(xs + m * kc + base);
              const uint4 x1 = *reinterpret_cast<const uint4*>(xs + m * kc + base + 256);
              a0[m] = fmaf(dot16_fp8(wa, x0, x1), sa, a0[m]);
              a1[m] = fmaf(dot16_fp8(wb, x0, x1), sb, a1[m]);
            }
          }
        }
        ++ck;
        __syncwarp();     // every lane has read the slot: it can be refilled
        issue_next();
      }
    } else {
      const int r1 = 2 * g + 1;
      const int r1c = r1 < total_rows ? r1 : r0;
      const bf16* w0p = p.Wb + (size_t)(r0 - p.N) * K;
      const bf16* w1p = p.Wb + (size_t)(r1c - p.N) * K;
#pragma unroll 2
      for (int i2 = it; i2 < it_stop; ++i2) {
        const int ka = (i2 << 9) + (lane << 4);
        if (ka < K) {
          const uint4 w00 = __ldg(reinterpret_cast<const uint4*>(w0p + ka));
          const uint4 w01 = __ldg(reinterpret_cast<const uint4*>(w0p + ka + 8));
          const uint4 w10 = __ldg(reinterpret_cast<const uint4*>(w1p + ka));
          const uint4 w11 = __ldg(reinterpret_cast<const uint4*>(w1p + ka + 8));
          const int base = (i2 << 9) + (lane << 3);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint4 x0 = *reinterpret_cast<const uint4*>(xs + m * kc + base);
            const uint4 x1 = *reinterpret_cast<const uint4*>(xs + m * kc + base + 256);
            a0[m] += dot16_bf16(w00, w01, x0, x1);
            a1[m] += dot16_bf16(w10, w11, x0, x1);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      a0[m] = warp_sum(a0[m]);
      a1[m] = warp_sum(a1[m]);
    }
    if (lane == 0) {
      // One writer for a row pair that lies wholly inside this warp's range; the partial first and last segments go
      // to the warp's two edge slots and are added in warp order below (the result does not depend on timing).
      const bool whole = it == 0 && it_stop == iters_all;
      const int e = pos == flat_begin ? 0 : 1;
      float* dst0 = whole ? s_acc + (gl * 2) * M : &s_edge_v[warp][e][0];
      float* dst1 = whole ? s_acc + (gl * 2 + 1) * M : &s_edge_v[warp][e][M];
      if (!whole) s_edge_g[warp][e] = gl;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        dst0[m] = a0[m];
        dst1[m] = a1[m];
      }
    }
    pos += it_stop - it;
  }
  __syncthreads();
  for (int idx = tid; idx < ngb * M; idx += kThreads) {
    const int gl = idx / M, m = idx - gl * M, g = g_lo + gl;
    float v0 = s_acc[(gl * 2) * M + m], v1 = s_acc[(gl * 2 + 1) * M + m];
#pragma unroll
    for (int w = 0; w < kWarps; ++w)
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (s_edge_g[w][e] == gl) {
          v0 += s_edge_v[w][e][m];
          v1 += s_edge_v[w][e][M + m];
        }
    v0 *= s_c[m];
    v1 *= s_c[m];
    if (swiglu) {
      p.y_bf16[(size_t)m * p.ldy + g] = __float2bfloat16(silu(v0) * v1);
    } else {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int n = 2 * g + r;
        if (n >= total_rows) continue;
        const float v = r == 0 ? v0 : v1;
        if (p.epi == 0) {
          p.y_bf16[(size_t)m * p.ldy + n] = __float2bfloat16(v);
        } else if (p.epi == 2) {
          p.y_f32[(size_t)m * p.ldy + n] = v;
        } else {
          const size_t off = ((size_t)p.push.rank * M + m) * p.ldy + n;
          for (int pr = 0; pr < p.push.world; ++pr) p.push.dst[pr][off] = v;
        }
      }
    }
  }
  if (p.epi == 3) publish_when_grid_done(p.push);
}

// Ring variant when it applies: FP8 rows present, one or two activation rows, few enough row pairs per block for the
// scale staging, and everything fits beside a second resident block. Returns -1 when the caller should use the
// register-streaming kernel.
template <int M>
int launch_ring(MatvecParams& p, int groups, int sm_count, cudaStream_t stream) {
  if (p.N <= 0 || (((uintptr_t)p.W) & 15) != 0) return -1;
  const int cap = (sm_count > 0 ? sm_count : 148) * kRingBlocksPerSm;
  const int blocks = groups < cap ? groups : cap;
  const int per_block = (groups + blocks - 1) / blocks;
  if (per_block > kRingMaxPairsPerBlock) return -1;
  const int kround = (p.K + 511) & ~511;
  const int kb_count = (p.K + 127) >> 7;
  p.kc = kround;
  p.single_chunk = 1;
  p.flat_path = 1;
  p.use_scratch = (p.gamma != nullptr || p.parts != nullptr || p.hidden_out != nullptr) ? 1 : 0;
  size_t off = (size_t)M * kround * 2 + (p.use_scratch ? (size_t)p.K * 4 : 0);
  off = (off + 127) & ~(size_t)127;
  p.acc_off = (int)off;
  off += (size_t)kRingMaxPairsPerBlock * 2 * M * sizeof(float);
  off = (off + 127) & ~(size_t)127;
  p.ring_off = (int)off;
  off += kRingBytes;
  p.bar_off = (int)off;
  off += (size_t)kWarps * kRingSlots * sizeof(uint64_t);
  p.scale_off = (int)off;
  off += (size_t)4 * kb_count * sizeof(float);
  if (off > (size_t)kRingSmemLimit) return -1;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(matvec_ring_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmemLimit) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  PK_LAUNCH_PDL(matvec_ring_kernel<M>, dim3(blocks), dim3(kThreads), off, stream, p);
  return PK_OK;
}

unsigned long long* g_matvec_dbg = nullptr;
}  // namespace

// Bulk L2 prefetch of a warp's first stretch of weights at kernel start is opt-in (POCKET_L2_PREFETCH=1).
static bool l2_prefetch_enabled() {
  const char* on = getenv("POCKET_L2_PREFETCH");
  return on != nullptr && on[0] == '1';
}

// The ring variant is on by default; POCKET_MATVEC_RING=0 keeps every shape on the register-streaming kernel.
static bool ring_enabled() {
  const char* v = getenv("POCKET_MATVEC_RING");
  return v == nullptr || v[0] != '0';
}

// First bounded wait of the ring variant that ran out since the last call (0 = none); clears the word.
PK_API unsigned pk_matvec_ring_status() {
  unsigned v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_matvec_ring_status, sizeof v) != cudaSuccess) return 0xffffffffu;
  if (v != 0) cudaMemcpyToSymbol(g_matvec_ring_status, &zero, sizeof zero);
  return v;
}

PK_API int pk_matvec(const void* W, const float* scale, const void* Wb, int N, int Nb, int K, int M,
                     const void* x_in, const float* parts, int nparts, void* hidden_out,
                     const float* gamma, int norm_mode, float eps, const PkWait* wait, int epi,
                     void* y, int ldy, const PkPush* push, int sm_count, cudaStream_t stream) {
  if (M < 1 || M > 8 || K <= 0 || (K & 15) != 0 || N < 0 || Nb < 0 || (N + Nb) == 0) return PK_ERR_BAD_ARG;
  if (epi == 1 && ((N & 1) != 0 || Nb != 0)) return PK_ERR_BAD_ARG;
  if (Nb > 0 && (N & 1) != 0) return PK_ERR_BAD_ARG;  // a row pair never mixes dtypes
  if (hidden_out != nullptr && hidden_out == x_in) return PK_ERR_BAD_ARG;  // other blocks still read x_in
  if (x_in == nullptr && (parts == nullptr || nparts <= 0)) return PK_ERR_BAD_ARG;
  if (epi == 3 && push == nullptr) return PK_ERR_BAD_ARG;
  if (((uintptr_t)x_in & 15) != 0 || ((uintptr_t)parts & 15) != 0 || ((uintptr_t)gamma & 15) != 0) return PK_ERR_BAD_ARG;
  MatvecParams p{};
  p.W = (const uint8_t*)W;
  p.scale = scale;
  p.Wb = (const pk::bf16*)Wb;
  p.N = N;
  p.Nb = Nb;
  p.K = K;
  p.M = M;
  p.x_in = (const pk::bf16*)x_in;
  p.parts = parts;
  p.nparts = parts ? nparts : 0;
  p.hidden_out = (pk::bf16*)hidden_out;
  p.gamma = gamma;
  p.norm_mode = norm_mode;
  p.dbg = g_matvec_dbg;
  p.self_prefetch = l2_prefetch_enabled() && (K & 15) == 0 && (((uintptr_t)W) & 15) == 0;
  p.eps = eps;
  if (wait) p.wait = *wait;
  p.epi = epi;
  p.y_bf16 = (pk::bf16*)y;
  p.y_f32 = (float*)y;
  p.ldy = ldy;
  if (push) p.push = *push;

  const int groups = epi == 1 ? N / 2 : (N + Nb + 1) / 2;
  if (M <= 2 && ring_enabled()) {
    const int rc = M == 1 ? launch_ring<1>(p, groups, sm_count, stream) : launch_ring<2>(p, groups, sm_count, stream);
    if (rc >= 0) return rc;
  }
  switch (M) {
    case 1: return launch_m<1>(p, groups, sm_count, stream);
    case 2: return launch_m<2>(p, groups, sm_count, stream);
    case 3: return launch_m<3>(p, groups, sm_count, stream);
    case 4: return launch_m<4>(p, groups, sm_count, stream);
    case 5: return launch_m<5>(p, groups, sm_count, stream);
    case 6: return launch_m<6>(p, groups, sm_count, stream);
    case 7: return launch_m<7>(p, groups, sm_count, stream);
    default: return launch_m<8>(p, groups, sm_count, stream);
  }
}

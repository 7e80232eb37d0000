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
// Behavioural counterpart in the reference: cpp_engine/cuda/qwen_half_ops.cu:89-374
// (fp8_matvec_f16*, fp8_matmul_f16_small_batch, fp8_swiglu_*), which are separate SIMT
// kernels with an LUT decode and NCCL all-reduces between them.
#include "../common/pk_comm.cuh"
#include "../common/pk_common.cuh"

namespace {

using namespace pk;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSmemFloats = 18 * 1024;  // 72 KB of staged activations per block

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
  float eps;
  PkWait wait;
  // epilogue
  int epi;               // 0 bf16 y[M, Nout], 1 swiglu -> bf16 y[M, N/2], 2 fp32 y[M, Nout], 3 push
  bf16* y_bf16;
  float* y_f32;
  int ldy;               // row stride of y (elements)
  PkPush push;
};

// Position of element k of a row inside the staged chunk. Within each run of 512
// elements the four float4 of a lane's 16 values are spread 128 floats apart so that a
// warp's LDS.128 touches 32 consecutive float4 (no bank conflicts).
__device__ __forceinline__ int staged_index(int k) {
  const int blk = k >> 9, r = k & 511;
  return (blk << 9) + (((r >> 2) & 3) << 7) + ((r >> 4) << 2) + (r & 3);
}

template <int M>
__device__ __forceinline__ void fma16_fp8(const uint4& w, const float* xs, int base, int kc_stride,
                                          float (&part)[M]) {
  // 16 fp8 codes -> 16 floats, times x rows.
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = e4m3x2_to_float2((uint16_t)(ww[j] & 0xffffu));
    const float2 b = e4m3x2_to_float2((uint16_t)(ww[j] >> 16));
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + m * kc_stride + base + (j << 7));
      part[m] = fmaf(a.x, xv.x, part[m]);
      part[m] = fmaf(a.y, xv.y, part[m]);
      part[m] = fmaf(b.x, xv.z, part[m]);
      part[m] = fmaf(b.y, xv.w, part[m]);
    }
  }
}

template <int M>
__device__ __forceinline__ void fma16_bf16(const uint4& w0, const uint4& w1, const float* xs, int base,
                                           int kc_stride, float (&part)[M]) {
  const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a0 = __uint_as_float(ww[2 * j] << 16), a1 = __uint_as_float(ww[2 * j] & 0xffff0000u);
    const float a2 = __uint_as_float(ww[2 * j + 1] << 16), a3 = __uint_as_float(ww[2 * j + 1] & 0xffff0000u);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const float4 xv = *reinterpret_cast<const float4*>(xs + m * kc_stride + base + (j << 7));
      part[m] = fmaf(a0, xv.x, part[m]);
      part[m] = fmaf(a1, xv.y, part[m]);
      part[m] = fmaf(a2, xv.z, part[m]);
      part[m] = fmaf(a3, xv.w, part[m]);
    }
  }
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
__device__ __forceinline__ void consume_fp8_batch(const Fp8Batch& bt, const float* xs, int kc, int it0, int iters,
                                                  int lane, float (&acc0)[M], float (&acc1)[M]) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    // The staged chunk ends at iteration `iters`; nothing beyond it may be read.
    if (it0 + u >= iters) break;
    float pa[M], pb[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { pa[m] = 0.f; pb[m] = 0.f; }
    fma16_fp8<M>(bt.a[u], xs, ((it0 + u) << 9) + (lane << 2), kc, pa);
    fma16_fp8<M>(bt.b[u], xs, ((it0 + u) << 9) + (lane << 2), kc, pb);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      acc0[m] = fmaf(pa[m], bt.sa[u], acc0[m]);
      acc1[m] = fmaf(pb[m], bt.sb[u], acc1[m]);
    }
  }
}

template <int M>
__global__ void __launch_bounds__(kThreads, 2) matvec_kernel(const MatvecParams p) {
  extern __shared__ __align__(16) float xs[];  // [M][kc] staged activations (permuted)
  __shared__ float red[40];
  __shared__ float rstd[8];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K;
  const int kc = min(((kSmemFloats / M) >> 9) << 9, (K + 511) & ~511);  // chunk length, multiple of 512
  const bool swiglu = p.epi == 1;
  const int half_n = p.N >> 1;
  // Row pairs: a warp owns two output rows at a time (gate_j and up_j for SwiGLU, else
  // rows 2g and 2g+1), so that every staged activation is read once per two weight rows.
  const int total_rows = p.N + p.Nb;
  const int n_groups = swiglu ? half_n : (total_rows + 1) >> 1;
  const int warps_total = gridDim.x * kWarps;
  const int gwarp = blockIdx.x * kWarps + warp;

  const int kb_count = (K + 127) >> 7;
  // Weights do not depend on the activations: issue the first batch of this warp's first
  // row pair before the prologue so that the HBM latency overlaps the norm.
  Fp8Batch bt;
  bool have_pre = false;
  {
    const int g0 = gwarp;
    const int r0 = swiglu ? g0 : 2 * g0;
    if (g0 < n_groups && r0 < p.N) {
      const int r1c = swiglu ? g0 + half_n : (2 * g0 + 1 < p.N ? 2 * g0 + 1 : r0);
      load_fp8_batch(bt, p.W + (size_t)r0 * K, p.W + (size_t)r1c * K, p.scale + (size_t)(r0 >> 7) * kb_count,
                     p.scale + (size_t)(r1c >> 7) * kb_count, 0, min(kc, K), lane);
      have_pre = true;
    }
  }

  // ---- wait for the producers of `parts`, then the per-row statistics ----
  if (p.parts != nullptr && p.wait.flag != nullptr) {
    if (tid == 0) wait_all_ranks(p.wait);
    __syncthreads();
  }
  const bool single_chunk = K <= kc;
  if (p.gamma != nullptr && !single_chunk) {
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int k = tid; k < K; k += kThreads) {
        float v = p.x_in ? __bfloat162float(p.x_in[(size_t)m * K + k]) : 0.f;
        for (int r = 0; r < p.nparts; ++r) v += p.parts[((size_t)r * M + m) * K + k];
        // The residual stream is kept in bf16; normalise what a later reader will see.
        v = __bfloat162float(__float2bfloat16(v));
        ss += v * v;
      }
      ss = block_sum(ss, red);
      if (tid == 0) rstd[m] = rsqrtf(ss / (float)K + p.eps);
    }
    __syncthreads();
  }

  float acc[2][M];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kc) {
    const int klen = min(kc, K - k0);
    // ---- stage the chunk ----
    if (k0 > 0) __syncthreads();
    if (single_chunk) {
      // One pass over global memory: stage the raw rows and their sums of squares, then
      // normalise in shared memory.
      for (int m = 0; m < M; ++m) {
        float ss = 0.f;
        // Zero the padding of the last 512-element run (read by lanes past K, times zero weights).
        for (int k = K + tid; k < kc; k += kThreads) xs[m * kc + staged_index(k)] = 0.f;
        // Eight elements per thread and step, four steps in flight, so that the loads of
        // the whole row overlap instead of forming one latency chain per element.
        const int nchunks = K >> 3;
        for (int c0 = tid; c0 < nchunks; c0 += kThreads * 4) {
          float v[4][8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * kThreads;
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (c < nchunks && p.x_in) xv = __ldg(reinterpret_cast<const uint4*>(p.x_in + (size_t)m * K + c * 8));
            const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[u][2 * j] = __uint_as_float(w[j] << 16);
              v[u][2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
          }
          for (int r = 0; r < p.nparts; ++r) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = c0 + u * kThreads;
              if (c < nchunks) {
                const float4* pp = reinterpret_cast<const float4*>(p.parts + ((size_t)r * M + m) * K + c * 8);
                const float4 a = pp[0], b = pp[1];
                v[u][0] += a.x; v[u][1] += a.y; v[u][2] += a.z; v[u][3] += a.w;
                v[u][4] += b.x; v[u][5] += b.y; v[u][6] += b.z; v[u][7] += b.w;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * kThreads;
            if (c >= nchunks) continue;
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[u][2 * j], v[u][2 * j + 1]);
              packed[j] = *reinterpret_cast<const uint32_t*>(&h2);
              if (p.parts != nullptr) {
                v[u][2 * j] = __uint_as_float(packed[j] << 16);
                v[u][2 * j + 1] = __uint_as_float(packed[j] & 0xffff0000u);
              }
            }
            if (p.hidden_out != nullptr && blockIdx.x == 0)
              *reinterpret_cast<uint4*>(p.hidden_out + (size_t)m * K + c * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            // elements 8c..8c+7 live in two float4 of the permuted layout
            const int si = m * kc + staged_index(c * 8);
            *reinterpret_cast<float4*>(xs + si) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
            *reinterpret_cast<float4*>(xs + si + 128) = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[u][j] * v[u][j];
          }
        }
        if (p.gamma != nullptr) {
          ss = block_sum(ss, red);
          const float rs = rsqrtf(ss / (float)K + p.eps);
          const float one = p.norm_mode == 1 ? 1.f : 0.f;
          const int nq = K >> 2;
          for (int c0 = tid; c0 < nq; c0 += kThreads * 4) {
            float4 gv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = c0 + u * kThreads;
              gv[u] = c < nq ? __ldg(reinterpret_cast<const float4*>(p.gamma) + c) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = c0 + u * kThreads;
              if (c >= nq) continue;
              float4* xp = reinterpret_cast<float4*>(xs + m * kc + staged_index(c * 4));
              float4 xv = *xp;
              // Activations are bf16 everywhere else; round here too so that the fused and
              // unfused paths see the same operand.
              xv.x = __bfloat162float(__float2bfloat16(xv.x * rs * (one + gv[u].x)));
              xv.y = __bfloat162float(__float2bfloat16(xv.y * rs * (one + gv[u].y)));
              xv.z = __bfloat162float(__float2bfloat16(xv.z * rs * (one + gv[u].z)));
              xv.w = __bfloat162float(__float2bfloat16(xv.w * rs * (one + gv[u].w)));
              *xp = xv;
            }
          }
        }
      }
    } else {
      for (int m = 0; m < M; ++m) {
        for (int k = tid; k < kc; k += kThreads) {
          float v = 0.f;
          if (k < klen) {
            const size_t gi = (size_t)m * K + k0 + k;
            v = p.x_in ? __bfloat162float(p.x_in[gi]) : 0.f;
            for (int r = 0; r < p.nparts; ++r) v += p.parts[((size_t)r * M + m) * K + k0 + k];
            const bf16 hv = __float2bfloat16(v);
            if (p.hidden_out != nullptr && blockIdx.x == 0) p.hidden_out[gi] = hv;
            if (p.parts != nullptr) v = __bfloat162float(hv);
            if (p.gamma != nullptr) {
              const float g = p.gamma[k0 + k];
              v = __bfloat162float(__float2bfloat16(v * rstd[m] * (p.norm_mode == 1 ? 1.f + g : g)));
            }
          }
          xs[m * kc + staged_index(k)] = v;
        }
      }
    }
    __syncthreads();

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
            fma16_bf16<M>(a0, a1, xs, (it << 9) + (lane << 2), kc, acc[0]);
            fma16_bf16<M>(b0, b1, xs, (it << 9) + (lane << 2), kc, acc[1]);
          }
        }
      }

      // ---- flush this group when its last chunk is done ----
      if (k0 + kc >= K) {
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
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

  if (p.epi == 3) publish_when_grid_done(p.push);
}

template <int M>
int launch_m(const MatvecParams& p, int blocks, cudaStream_t stream) {
  const int kc = min(((kSmemFloats / M) >> 9) << 9, (p.K + 511) & ~511);
  const size_t smem = (size_t)M * kc * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(matvec_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kSmemFloats * (int)sizeof(float)) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    configured = true;
  }
  matvec_kernel<M><<<blocks, kThreads, smem, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

}  // namespace

// A chunked K loop keeps one accumulator set per warp, so a warp may own only one row
// group when K does not fit one chunk. The launcher sizes the grid accordingly.
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
  p.eps = eps;
  if (wait) p.wait = *wait;
  p.epi = epi;
  p.y_bf16 = (pk::bf16*)y;
  p.y_f32 = (float*)y;
  p.ldy = ldy;
  if (push) p.push = *push;

  const int groups = epi == 1 ? N / 2 : (N + Nb + 1) / 2;
  const int kc = (((kSmemFloats / M) >> 9) << 9);
  const bool chunked = K > kc;
  int blocks;
  if (chunked) {
    blocks = (groups + kWarps - 1) / kWarps;  // exactly one group per warp
  } else {
    const int per_sm = 2;
    blocks = (groups + kWarps - 1) / kWarps;
    const int cap = (sm_count > 0 ? sm_count : 148) * per_sm;
    if (blocks > cap) blocks = cap;
  }
  if (blocks < 1) blocks = 1;
  switch (M) {
    case 1: return launch_m<1>(p, blocks, stream);
    case 2: return launch_m<2>(p, blocks, stream);
    case 3: return launch_m<3>(p, blocks, stream);
    case 4: return launch_m<4>(p, blocks, stream);
    case 5: return launch_m<5>(p, blocks, stream);
    case 6: return launch_m<6>(p, blocks, stream);
    case 7: return launch_m<7>(p, blocks, stream);
    default: return launch_m<8>(p, blocks, stream);
  }
}

// Chunked Gated DeltaNet scan for prefill (chunk = 64 tokens).
//
// The recurrence  S_t = e^{g_t} S_{t-1} + k_t (x) delta_t,  delta_t = beta_t (v_t - (e^{g_t} S_{t-1})^T k_t)
// is serial in t; inside a chunk it is rewritten (WY / UT transform) so that only one
// state update per chunk stays serial. With G_i the running sum of g inside the chunk,
//   A_ij = beta_i e^{G_i - G_j} (k_i . k_j)  (j < i),       (I + A) Delta = beta (V - e^{G} K S_0)
//   U = (I + A)^{-1} (beta V),  W = (I + A)^{-1} (beta e^{G} K),   Delta = U - W S_0
//   O = e^{G} Q S_0 + P Delta,  P_ij = e^{G_i - G_j} (q_i . k_j)  (j <= i)
//   S_C = e^{G_C} S_0 + (e^{G_C - G} K)^T Delta
// Everything that does not touch S (conv + SiLU, norms, gates, A, U, W, P) runs in
// parallel over (head, chunk); the state pass runs over (head, quarter of the value dim).
// The reference engine has only the token-serial form for prefill
// (cpp_engine/cuda/qwen_half_ops.cu:858-930, one 128-float state column per thread).
//
// All matrix products here are fp32 SIMT; they are the next candidates for tcgen05 tiles.
#include <cstdlib>
#include "../common/pk_common.cuh"

namespace {

using namespace pk;

constexpr int CH = 64;   // chunk length
constexpr int D = 128;   // key and value head dim
constexpr int KS = 129;  // padded row stride of K / Q tiles in shared memory

// ---------------------------------------------------------------------------------------
// prep: conv + SiLU, L2 norms, gates, for every token in parallel

struct PrepParams {
  const bf16* proj;  // [T, ld]: q(KD) | k(KD) | v(VD) | z(VD) | a(Hv) | b(Hv)
  int ld, T, Tpad, Hk, Hv;
  const float* conv_w;      // [C, 4]
  const float* conv_state;  // [C, 3] inputs at times -3, -2, -1
  const float* A_log;
  const float* dt_bias;
  float* qn;    // [Tpad, Hk, 128] l2-normalised, times 1/sqrt(128)
  float* kn;    // [Tpad, Hk, 128]
  float* v;     // [Tpad, Hv, 128]
  float* g;     // [Tpad, Hv] log decay
  float* beta;  // [Tpad, Hv]
};

// Inputs of channels ch and ch + 1 (ch even) at time t: the projection row, or the remembered tail for t < 0.
__device__ __forceinline__ float2 conv_input2(const PrepParams& p, int t, int ch) {
  if (t >= 0) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.proj + (size_t)t * p.ld + ch));
  return make_float2(p.conv_state[(size_t)ch * 3 + (3 + t)], p.conv_state[(size_t)(ch + 1) * 3 + (3 + t)]);
}

// One block per (token, key head): 64 threads per 128-channel segment (q, k, then the head's value heads), two
// adjacent channels per thread.
__global__ void __launch_bounds__(256) deltanet_prep_kernel(const PrepParams p) {
  const int t = blockIdx.x, hk = blockIdx.y;
  const int rep = p.Hv / p.Hk;
  const int seg = threadIdx.x >> 6, d = (threadIdx.x & 63) * 2;  // seg 0: q, 1: k, 2+: value heads
  const int KD = p.Hk * D, VD = p.Hv * D;
  __shared__ float s_sum[4][2];
  const int h = hk * rep + (seg - 2);
  float y0 = 0.f, y1 = 0.f;
  if (t < p.T) {
    const int ch = seg == 0 ? hk * D + d : seg == 1 ? KD + hk * D + d : 2 * KD + h * D + d;
    const float4 w0 = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch * 4);
    const float4 w1 = *reinterpret_cast<const float4*>(p.conv_w + (size_t)(ch + 1) * 4);
    const float2 a = conv_input2(p, t - 3, ch), b = conv_input2(p, t - 2, ch), c = conv_input2(p, t - 1, ch), e = conv_input2(p, t, ch);
    y0 = w0.x * a.x + w0.y * b.x + w0.z * c.x + w0.w * e.x;
    y1 = w1.x * a.y + w1.y * b.y + w1.z * c.y + w1.w * e.y;
    y0 = __bfloat162float(__float2bfloat16(silu(y0)));
    y1 = __bfloat162float(__float2bfloat16(silu(y1)));
  }
  const float ss = warp_sum(y0 * y0 + y1 * y1);
  if ((threadIdx.x & 31) == 0) s_sum[seg][(threadIdx.x >> 5) & 1] = ss;
  __syncthreads();
  if (seg < 2) {
    const float tot = s_sum[seg][0] + s_sum[seg][1];
    const float n = rsqrtf(tot + 1e-6f) * (seg == 0 ? rsqrtf((float)D) : 1.f);
    float* dst = (seg == 0 ? p.qn : p.kn) + ((size_t)t * p.Hk + hk) * D + d;
    *reinterpret_cast<float2*>(dst) = make_float2(y0 * n, y1 * n);
  } else {
    *reinterpret_cast<float2*>(p.v + ((size_t)t * p.Hv + h) * D + d) = make_float2(y0, y1);
    if (d == 0) {
      float gg = 0.f, bb = 0.f;
      if (t < p.T) {
        const bf16* row = p.proj + (size_t)t * p.ld;
        const float a = __bfloat162float(row[2 * KD + 2 * VD + h]);
        const float b = __bfloat162float(row[2 * KD + 2 * VD + p.Hv + h]);
        gg = -__expf(p.A_log[h]) * softplusf_(a + p.dt_bias[h]);
        bb = sigmoidf_(b);
      }
      p.g[(size_t)t * p.Hv + h] = gg;
      p.beta[(size_t)t * p.Hv + h] = bb;
    }
  }
}

// New conv tail = inputs of the last three tokens. Runs after prep (which reads the old tail).
__global__ void deltanet_tail_kernel(const bf16* proj, int ld, int T, int channels, float* conv_state) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= channels) return;
  float nv[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int t = T - 3 + j;
    nv[j] = t >= 0 ? __bfloat162float(proj[(size_t)t * ld + ch]) : conv_state[(size_t)ch * 3 + (3 + t)];
  }
#pragma unroll
  for (int j = 0; j < 3; ++j) conv_state[(size_t)ch * 3 + j] = nv[j];
}

// ---------------------------------------------------------------------------------------
// per (chunk, value head): G, A, U, W, P

struct ChunkParams {
  const float* qn; const float* kn; const float* v; const float* g; const float* beta;
  int Hk, Hv, Tpad;
  float* U;   // [Hv, Tpad, 128]
  float* W;   // [Hv, Tpad, 128]
  float* P;   // [Hv, Tpad/64, 64, 64]
  float* G;   // [Hv, Tpad] running log decay inside the chunk
};

__global__ void __launch_bounds__(256) deltanet_chunk_kernel(const ChunkParams p) {
  extern __shared__ float smem[];
  float* Ks = smem;                  // [64][129]
  float* Qs = Ks + CH * KS;          // [64][129]
  float* As = Qs + CH * KS;          // [64][64]
  float* Gs = As + CH * CH;          // [64]
  float* Bs = Gs + CH;               // [64]
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int hk = h / (p.Hv / p.Hk);
  const int t0 = c * CH;

  for (int i = tid; i < CH * D; i += 256) {
    const int r = i >> 7, d = i & 127;
    Ks[r * KS + d] = p.kn[((size_t)(t0 + r) * p.Hk + hk) * D + d];
    Qs[r * KS + d] = p.qn[((size_t)(t0 + r) * p.Hk + hk) * D + d];
  }
  if (tid < 32) {
    // inclusive scan of g over the 64 tokens (two per lane)
    const float g0 = p.g[(size_t)(t0 + 2 * tid) * p.Hv + h], g1 = p.g[(size_t)(t0 + 2 * tid + 1) * p.Hv + h];
    float s = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, s, o);
      if (tid >= o) s += n;
    }
    Gs[2 * tid + 1] = s;
    Gs[2 * tid] = s - g1;
    Bs[2 * tid] = p.beta[(size_t)(t0 + 2 * tid) * p.Hv + h];
    Bs[2 * tid + 1] = p.beta[(size_t)(t0 + 2 * tid + 1) * p.Hv + h];
  }
  __syncthreads();
  if (tid < CH) p.G[(size_t)h * p.Tpad + t0 + tid] = Gs[tid];

  // A and P: thread owns column j and rows i = ig + 4n
  {
    const int j = tid & 63, ig = tid >> 6;
    float accA[16], accP[16];
#pragma unroll
    for (int n = 0; n < 16; ++n) { accA[n] = 0.f; accP[n] = 0.f; }
    for (int k = 0; k < D; ++k) {
      const float kj = Ks[j * KS + k];
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int i = ig + 4 * n;
        accA[n] = fmaf(Ks[i * KS + k], kj, accA[n]);
        accP[n] = fmaf(Qs[i * KS + k], kj, accP[n]);
      }
    }
    float* Pout = p.P + (((size_t)h * (p.Tpad / CH) + c) * CH) * CH;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const int i = ig + 4 * n;
      const float e = __expf(Gs[i] - Gs[j]);
      As[i * CH + j] = j < i ? Bs[i] * e * accA[n] : 0.f;
      Pout[i * CH + j] = j <= i ? e * accP[n] : 0.f;
    }
  }
  __syncthreads();

  // Forward substitution, one right-hand-side column per thread: columns 0..127 are
  // beta*V (-> U), columns 128..255 are beta*e^G*K (-> W).
  {
    const int col = tid & 127;
    const bool isW = tid >= 128;
    float X[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float b;
      if (isW) b = Bs[i] * __expf(Gs[i]) * Ks[i * KS + col];
      else b = Bs[i] * p.v[((size_t)(t0 + i) * p.Hv + h) * D + col];
      float acc = b;
#pragma unroll
      for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
        const float4 a = *reinterpret_cast<const float4*>(As + i * CH + j4 * 4);
        // entries at or right of the diagonal are stored as zero
        if (j4 * 4 + 0 < i) acc = fmaf(-a.x, X[j4 * 4 + 0], acc);
        if (j4 * 4 + 1 < i) acc = fmaf(-a.y, X[j4 * 4 + 1], acc);
        if (j4 * 4 + 2 < i) acc = fmaf(-a.z, X[j4 * 4 + 2], acc);
        if (j4 * 4 + 3 < i) acc = fmaf(-a.w, X[j4 * 4 + 3], acc);
      }
      X[i] = acc;
      float* dst = (isW ? p.W : p.U) + ((size_t)h * p.Tpad + t0 + i) * D + col;
      *dst = acc;
    }
  }
}

// ---------------------------------------------------------------------------------------
// state pass: serial over chunks, parallel over (value head, 32-column slice of the state)

struct StateParams {
  const float* qn; const float* kn; const float* U; const float* W; const float* P; const float* G;
  int Hk, Hv, Tpad, nchunks;
  float* state;  // [Hv, 128, 128]
  float* O;      // [Tpad, Hv, 128]
};

constexpr int SL = 32;   // state columns per block
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ST threads per block: with 512 (16 warps) warp w owns 4 chunk rows and 8 state rows, with 256 it owns 8 and 16.
// One block per SM (137 KB of shared memory). The three operand tiles of a chunk (W, q, k: 32 KB each) and P arrive by
// cp.async straight into the buffer that the matching phase of the PREVIOUS chunk has just finished with, so every load
// has two phases of arithmetic to land in: W(c+1) is issued after the Delta phase of chunk c, q and P after the output
// phase, k after the state phase. Three groups are always in flight in that order, so "all but the two newest groups
// have landed" is the right wait before every phase. q and k stay unscaled in shared memory: e^{G_i} multiplies the
// q.S sums, e^{G_C - G_j} multiplies Delta_j on the way into the state update.
// Before: loads, then arithmetic, per chunk (20 us per chunk step, a third of it exposed load latency).
template <int ST>
__global__ void __launch_bounds__(ST) deltanet_state_kernel(const StateParams p) {
  constexpr int RW = CH / (ST / 32);   // chunk rows per warp
  constexpr int SW = D / (ST / 32);    // state rows per warp
  extern __shared__ __align__(16) float smem[];
  float* Ws = smem;               // [64][128]
  float* Qs = Ws + CH * D;        // [64][128]  q_i (unscaled)
  float* Ks = Qs + CH * D;        // [64][128]  k_i (unscaled)
  float* Ps = Ks + CH * D;        // [64][64]
  float* Ds = Ps + CH * CH;       // [64][32]   Delta
  float* Ss = Ds + CH * SL;       // [128][32]  state slice
  float* Gs = Ss + D * SL;        // [64]
  float* Eq = Gs + CH;            // [64] e^{G_i}
  float* Ek = Eq + CH;            // [64] e^{G_C - G_i}
  const int h = blockIdx.x, sl = blockIdx.y, tid = threadIdx.x;
  const int hk = h / (p.Hv / p.Hk);
  const int tx = tid & 31, ty = tid >> 5;
  float* sp = p.state + (size_t)h * D * D + sl * SL;

  auto issue_w = [&](int c) {
    if (c < p.nchunks) {
      const float* src = p.W + ((size_t)h * p.Tpad + (size_t)c * CH) * D;
      for (int i = tid; i < CH * D / 4; i += ST) cp_async16(Ws + i * 4, src + i * 4);
    }
    cp_async_commit();
  };
  auto issue_qp = [&](int c) {
    if (c < p.nchunks) {
      for (int i = tid; i < CH * D / 4; i += ST) {
        const int r = i >> 5, d4 = (i & 31) * 4;
        cp_async16(Qs + r * D + d4, p.qn + ((size_t)(c * CH + r) * p.Hk + hk) * D + d4);
      }
      const float* src = p.P + (((size_t)h * p.nchunks + c) * CH) * CH;
      for (int i = tid; i < CH * CH / 4; i += ST) cp_async16(Ps + i * 4, src + i * 4);
    }
    cp_async_commit();
  };
  auto issue_k = [&](int c) {
    if (c < p.nchunks) {
      for (int i = tid; i < CH * D / 4; i += ST) {
        const int r = i >> 5, d4 = (i & 31) * 4;
        cp_async16(Ks + r * D + d4, p.kn + ((size_t)(c * CH + r) * p.Hk + hk) * D + d4);
      }
    }
    cp_async_commit();
  };

  issue_w(0);
  issue_qp(0);
  issue_k(0);
  for (int i = tid; i < D * SL; i += ST) Ss[i] = sp[(size_t)(i >> 5) * D + (i & 31)];
  float gnext = tid < CH ? p.G[(size_t)h * p.Tpad + tid] : 0.f;

  for (int c = 0; c < p.nchunks; ++c) {
    const int t0 = c * CH;
    if (tid < CH) Gs[tid] = gnext;
    if (tid < CH && c + 1 < p.nchunks) gnext = p.G[(size_t)h * p.Tpad + t0 + CH + tid];
    float acc[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) acc[r] = p.U[((size_t)h * p.Tpad + t0 + ty * RW + r) * D + sl * SL + tx];
    __syncthreads();
    const float gC = Gs[CH - 1];
    if (tid < CH) {
      Eq[tid] = __expf(Gs[tid]);
      Ek[tid] = __expf(gC - Gs[tid]);
    }
    cp_async_wait<2>();   // W of this chunk
    __syncthreads();

    // Delta = U - W S, rows ty*RW .. ty*RW+RW-1
    for (int k = 0; k < D; k += 4) {
      const float s0 = Ss[(k + 0) * SL + tx], s1 = Ss[(k + 1) * SL + tx], s2 = Ss[(k + 2) * SL + tx],
                  s3 = Ss[(k + 3) * SL + tx];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float4 w = *reinterpret_cast<const float4*>(Ws + (ty * RW + r) * D + k);
        acc[r] -= w.x * s0 + w.y * s1 + w.z * s2 + w.w * s3;
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) Ds[(ty * RW + r) * SL + tx] = acc[r];
    __syncthreads();
    issue_w(c + 1);       // Ws is free
    cp_async_wait<2>();   // q and P of this chunk
    __syncthreads();

    // O = e^{G} (q S) + P Delta
#pragma unroll
    for (int r = 0; r < RW; ++r) acc[r] = 0.f;
    for (int k = 0; k < D; k += 4) {
      const float s0 = Ss[(k + 0) * SL + tx], s1 = Ss[(k + 1) * SL + tx], s2 = Ss[(k + 2) * SL + tx],
                  s3 = Ss[(k + 3) * SL + tx];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float4 w = *reinterpret_cast<const float4*>(Qs + (ty * RW + r) * D + k);
        acc[r] += w.x * s0 + w.y * s1 + w.z * s2 + w.w * s3;
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) acc[r] *= Eq[ty * RW + r];
    for (int j = 0; j < CH; j += 4) {
      const float d0 = Ds[(j + 0) * SL + tx], d1 = Ds[(j + 1) * SL + tx], d2 = Ds[(j + 2) * SL + tx],
                  d3 = Ds[(j + 3) * SL + tx];
#pragma unroll
      for (int r = 0; r < RW; ++r) {
        const float4 w = *reinterpret_cast<const float4*>(Ps + (ty * RW + r) * CH + j);
        acc[r] += w.x * d0 + w.y * d1 + w.z * d2 + w.w * d3;
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r)
      p.O[((size_t)(t0 + ty * RW + r) * p.Hv + h) * D + sl * SL + tx] = acc[r];
    __syncthreads();
    issue_qp(c + 1);      // Qs and Ps are free
    cp_async_wait<2>();   // k of this chunk
    __syncthreads();

    // S <- e^{G_C} S + k^T (e^{G_C - G} Delta), rows ty*SW .. ty*SW+SW-1
    float sn[SW];
    const float eC = __expf(gC);
#pragma unroll
    for (int r = 0; r < SW; ++r) sn[r] = eC * Ss[(ty * SW + r) * SL + tx];
    for (int j = 0; j < CH; ++j) {
      const float dj = Ds[j * SL + tx] * Ek[j];
#pragma unroll
      for (int r4 = 0; r4 < SW / 4; ++r4) {
        const float4 k = *reinterpret_cast<const float4*>(Ks + j * D + ty * SW + r4 * 4);
        sn[r4 * 4 + 0] = fmaf(k.x, dj, sn[r4 * 4 + 0]);
        sn[r4 * 4 + 1] = fmaf(k.y, dj, sn[r4 * 4 + 1]);
        sn[r4 * 4 + 2] = fmaf(k.z, dj, sn[r4 * 4 + 2]);
        sn[r4 * 4 + 3] = fmaf(k.w, dj, sn[r4 * 4 + 3]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < SW; ++r) Ss[(ty * SW + r) * SL + tx] = sn[r];
    issue_k(c + 1);       // Ks is free
    __syncthreads();
  }
  cp_async_wait<0>();
  for (int i = tid; i < D * SL; i += ST) sp[(size_t)(i >> 5) * D + (i & 31)] = Ss[i];
}

// ---------------------------------------------------------------------------------------
// gated RMSNorm of the scan output

// One warp per (token, value head), four channels per lane.
__global__ void __launch_bounds__(256) deltanet_out_kernel(const float* O, const bf16* proj, int ld, int Hk, int Hv, int T,
                                                           const float* norm_w, float eps, bf16* out) {
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= T * Hv) return;
  const int t = unit / Hv, h = unit - t * Hv, d = (threadIdx.x & 31) * 4;
  const float4 o = *reinterpret_cast<const float4*>(O + ((size_t)t * Hv + h) * D + d);
  const float ss = warp_sum(o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w);
  const int KD = Hk * D, VD = Hv * D;
  const uint2 zr = *reinterpret_cast<const uint2*>(proj + (size_t)t * ld + 2 * KD + VD + h * D + d);
  const float z0 = __uint_as_float(zr.x << 16), z1 = __uint_as_float(zr.x & 0xffff0000u), z2 = __uint_as_float(zr.y << 16),
              z3 = __uint_as_float(zr.y & 0xffff0000u);
  const float4 w = *reinterpret_cast<const float4*>(norm_w + d);
  const float r = rsqrtf(ss / (float)D + eps);
  __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * r * w.x * silu(z0), o.y * r * w.y * silu(z1));
  __nv_bfloat162 hi = __floats2bfloat162_rn(o.z * r * w.z * silu(z2), o.w * r * w.w * silu(z3));
  uint2 packed;
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + (size_t)t * VD + h * D + d) = packed;
}

}  // namespace

// Workspace floats needed for T tokens (Tpad = T rounded up to 64).
PK_API size_t pk_deltanet_chunk_workspace(int T, int key_heads, int value_heads) {
  const size_t Tpad = (size_t)((T + CH - 1) / CH) * CH;
  return Tpad * key_heads * D * 2      // qn, kn
         + Tpad * value_heads * D * 4  // v, U, W, O
         + Tpad * value_heads * 3      // g, beta, G
         + (size_t)value_heads * Tpad * CH;  // P
}

// Same contract as pk_deltanet_seq (state and conv_state advance by T tokens), but the
// work is chunk-parallel. `ws` holds pk_deltanet_chunk_workspace(T, ...) floats.
PK_API int pk_deltanet_chunked(const void* proj, int ld, int T, int key_heads, int value_heads, int key_dim,
                               int value_dim, const float* conv_w, float* conv_state, const float* A_log,
                               const float* dt_bias, const float* norm_w, float eps, float* state, void* out,
                               float* ws, cudaStream_t stream) {
  if (key_dim != D || value_dim != D) return PK_ERR_UNSUPPORTED;
  if (T < 1 || key_heads < 1 || value_heads % key_heads != 0 || ((uintptr_t)ws & 15) != 0) return PK_ERR_BAD_ARG;   // cp.async of 16 bytes
  if ((ld & 3) != 0 || ((uintptr_t)proj & 7) != 0 || ((uintptr_t)out & 7) != 0 || ((uintptr_t)norm_w & 15) != 0) return PK_ERR_BAD_ARG;   // 8-byte row accesses
  const int rep = value_heads / key_heads;
  if (rep > 2) return PK_ERR_UNSUPPORTED;
  const int nchunks = (T + CH - 1) / CH, Tpad = nchunks * CH;
  float* qn = ws;
  float* kn = qn + (size_t)Tpad * key_heads * D;
  float* v = kn + (size_t)Tpad * key_heads * D;
  float* U = v + (size_t)Tpad * value_heads * D;
  float* W = U + (size_t)Tpad * value_heads * D;
  float* O = W + (size_t)Tpad * value_heads * D;
  float* g = O + (size_t)Tpad * value_heads * D;
  float* beta = g + (size_t)Tpad * value_heads;
  float* G = beta + (size_t)Tpad * value_heads;
  float* P = G + (size_t)Tpad * value_heads;

  PrepParams pp{(const pk::bf16*)proj, ld, T, Tpad, key_heads, value_heads, conv_w, conv_state, A_log, dt_bias,
                qn, kn, v, g, beta};
  deltanet_prep_kernel<<<dim3(Tpad, key_heads), 64 * (2 + rep), 0, stream>>>(pp);
  PK_CHECK_LAUNCH();
  const int channels = (2 * key_heads + value_heads) * D;
  deltanet_tail_kernel<<<(channels + 255) / 256, 256, 0, stream>>>((const pk::bf16*)proj, ld, T, channels, conv_state);
  PK_CHECK_LAUNCH();

  static PkDeviceOnce once;
  const size_t smem_chunk = (size_t)(2 * CH * KS + CH * CH + 2 * CH) * sizeof(float);
  const size_t smem_state = (size_t)(3 * CH * D + CH * CH + CH * SL + D * SL + 3 * CH) * sizeof(float);
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(deltanet_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_chunk) != cudaSuccess ||
        cudaFuncSetAttribute(deltanet_state_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_state) != cudaSuccess ||
        cudaFuncSetAttribute(deltanet_state_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_state) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  ChunkParams cp{qn, kn, v, g, beta, key_heads, value_heads, Tpad, U, W, P, G};
  deltanet_chunk_kernel<<<dim3(nchunks, value_heads), 256, smem_chunk, stream>>>(cp);
  PK_CHECK_LAUNCH();
  StateParams sp{qn, kn, U, W, P, G, key_heads, value_heads, Tpad, nchunks, state, O};
  static const int state_threads = [] {
    const char* e = getenv("POCKET_DELTANET_STATE_THREADS");
    return e && atoi(e) == 256 ? 256 : 512;
  }();
  if (state_threads == 256) deltanet_state_kernel<256><<<dim3(value_heads, D / SL), 256, smem_state, stream>>>(sp);
  else deltanet_state_kernel<512><<<dim3(value_heads, D / SL), 512, smem_state, stream>>>(sp);
  PK_CHECK_LAUNCH();
  deltanet_out_kernel<<<(T * value_heads + 7) / 8, 256, 0, stream>>>(O, (const pk::bf16*)proj, ld, key_heads, value_heads, T,
                                                                     norm_w, eps, (pk::bf16*)out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// GQA attention for decode and speculative verify: fused per-head RMSNorm + partial RoPE
// + KV append, split-context flash decode, and the merge that also applies the output
// gate. Behavioural counterpart in the reference: cpp_engine/cuda/qwen_half_ops.cu:932-1158
// (partial_rope, append_kv, gqa_scores / softmax / gqa_values as separate passes) and
// cpp_engine/cuda/qwen_gqa_optimized.cu:253-376 (split + merge for long contexts only).
//
// Positions are read from device memory so that one captured CUDA graph serves every
// decode step; the split count is a launch constant and empty splits return at once.
#include "../common/pk_common.cuh"

namespace {

using namespace pk;

constexpr int kD = 128;  // head dim

struct QkParams {
  const bf16* proj;   // [M, ld]: per q head [q(D) | gate(D)], then k heads, then v heads
  int ld;
  int M, Hq, Hkv;
  const int* pos;     // [M]
  const float* q_gamma;  // [D]
  const float* k_gamma;  // [D]
  float eps;
  int rotary_dim;
  float theta;
  bf16* q_out;        // [M, Hq, D]
  bf16* kcache;       // [Hkv, ctx_cap, D] bf16, or E4M3 codes (one byte per channel) when kv_fp8
  bf16* vcache;
  int ctx_cap;
  // FP8 KV cache (reference: cpp_engine/cuda/qwen_half_ops.cu:1010-1055, append_kv_fp8_kernel): every row of a head is
  // stored as E4M3 codes with one fp32 scale per 64 channels, scale = amax / 448 (1 when the group is all zero).
  int kv_fp8;
  float* kscale;      // [Hkv, ctx_cap, D / 64]
  float* vscale;
};

__global__ void __launch_bounds__(kD) qk_norm_rope_append_kernel(const QkParams p) {
  pk::pdl_wait();
  pk::pdl_trigger();
  const int m = blockIdx.x, hh = blockIdx.y, d = threadIdx.x;
  __shared__ float red[40];
  __shared__ float sy[kD];
  const bool is_q = hh < p.Hq;
  const int hk = hh - p.Hq;
  const bf16* row = p.proj + (size_t)m * p.ld;
  const int off = is_q ? hh * 2 * kD : p.Hq * 2 * kD + hk * kD;
  const float x = __bfloat162float(row[off + d]);
  const float ss = block_sum(x * x, red);
  const float g = is_q ? p.q_gamma[d] : p.k_gamma[d];
  float y = x * rsqrtf(ss / (float)kD + p.eps) * (1.f + g);
  y = __bfloat162float(__float2bfloat16(y));
  sy[d] = y;
  __syncthreads();
  const int pos = p.pos[m];
  if (!is_q && d == 0 && (pos < 0 || pos >= p.ctx_cap)) PK_DEBUG_RECORD(101, pos, p.ctx_cap);   // the row is not written (below)
  const int hr = p.rotary_dim >> 1;
  if (d < p.rotary_dim) {
    const int i = d < hr ? d : d - hr;
    const double inv_freq = pow((double)p.theta, -2.0 * (double)i / (double)p.rotary_dim);
    double sn, cs;
    sincos((double)pos * inv_freq, &sn, &cs);
    const float other = d < hr ? sy[d + hr] : sy[d - hr];
    y = d < hr ? y * (float)cs - other * (float)sn : y * (float)cs + other * (float)sn;
  }
  if (is_q) {
    p.q_out[((size_t)m * p.Hq + hh) * kD + d] = __float2bfloat16(y);
  } else if (p.kv_fp8) {
    // block-uniform branch (k heads): quantise the bf16-rounded key and the value per 64 channels
    const float kvv = __bfloat162float(__float2bfloat16(y));
    const float vv = __bfloat162float(row[p.Hq * 2 * kD + p.Hkv * kD + hk * kD + d]);
    const float ka = warp_max(fabsf(kvv)), va = warp_max(fabsf(vv));
    __syncthreads();   // `red` was used by the norm
    if ((d & 31) == 0) {
      red[d >> 5] = ka;
      red[4 + (d >> 5)] = va;
    }
    __syncthreads();
    const int half = d >> 6;
    const float kmax = fmaxf(red[2 * half], red[2 * half + 1]), vmax = fmaxf(red[4 + 2 * half], red[4 + 2 * half + 1]);
    const float ks = kmax > 0.f ? kmax / 448.f : 1.f, vs = vmax > 0.f ? vmax / 448.f : 1.f;
    if (pos >= 0 && pos < p.ctx_cap) {
      const size_t ri = (size_t)hk * p.ctx_cap + pos;
      reinterpret_cast<uint8_t*>(p.kcache)[ri * kD + d] = float_to_e4m3(kvv / ks);
      reinterpret_cast<uint8_t*>(p.vcache)[ri * kD + d] = float_to_e4m3(vv / vs);
      if ((d & 63) == 0) {
        p.kscale[ri * 2 + half] = ks;
        p.vscale[ri * 2 + half] = vs;
      }
    }
  } else if (pos >= 0 && pos < p.ctx_cap) {
    const size_t ci = ((size_t)hk * p.ctx_cap + pos) * kD + d;
    p.kcache[ci] = __float2bfloat16(y);
    p.vcache[ci] = row[p.Hq * 2 * kD + p.Hkv * kD + hk * kD + d];
  }
}

struct DecodeParams {
  const bf16* q;       // [M, Hq, D]
  const bf16* kcache;  // [Hkv, ctx_cap, D]
  const bf16* vcache;
  const int* pos;      // [M]: row m attends keys 0..pos[m]
  int M, Hq, Hkv, ctx_cap;
  float scale;
  int nsplit;
  int window;          // 0 = full; else keys in (pos-window, pos] plus the first `sink` keys
  int sink;
  float* ws;           // [M, Hq, nsplit, D + 2]
  int kv_fp8;          // caches hold E4M3 codes with one fp32 scale per 64 channels
  const float* kscale; // [Hkv, ctx_cap, 2]
  const float* vscale;
};

// Eight consecutive channels of one cached row as floats. bf16: one 16-byte load; fp8: one 8-byte load and the scale of
// the 64-channel group the lane's channels belong to.
__device__ __forceinline__ void load_kv8(const void* base, const float* scale, size_t row, int l16, bool fp8, float (&f)[8]) {
  if (!fp8) {
    const uint4 r = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(base) + row * kD + l16 * 8);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = __uint_as_float(w[j] << 16);
      f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  } else {
    const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(base) + row * kD + l16 * 8);
    const float sc = scale[row * 2 + (l16 >> 3)];
    const uint32_t w[2] = {r.x, r.y};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float2 a = e4m3x2_to_float2((uint16_t)(w[j] & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(w[j] >> 16));
      f[4 * j] = a.x * sc;
      f[4 * j + 1] = a.y * sc;
      f[4 * j + 2] = b.x * sc;
      f[4 * j + 3] = b.y * sc;
    }
  }
}

template <int G>
__global__ void __launch_bounds__(128) gqa_decode_split_kernel(const DecodeParams p) {
  pk::pdl_wait();
  pk::pdl_trigger();
  const int hk = blockIdx.x, split = blockIdx.y, m = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int l16 = lane & 15, khalf = lane >> 4;
  const int len = min(p.pos[m] + 1, p.ctx_cap);
  int per = (len + p.nsplit - 1) / p.nsplit;
  per = (per + 7) & ~7;
  const int start = split * per, end = min(len, start + per);
  const int win_lo = p.window > 0 ? max(0, len - p.window) : 0;

  float qv[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p.q + ((size_t)m * p.Hq + hk * G + g) * kD + l16 * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      qv[g][2 * j] = __uint_as_float(w[j] << 16) * p.scale;
      qv[g][2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u) * p.scale;
    }
  }
  float mx[G], sum[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    mx[g] = -INFINITY;
    sum[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
  }

  const size_t head_row0 = (size_t)hk * p.ctx_cap;
  const bool fp8 = p.kv_fp8 != 0;
  for (int t0 = start + warp * 2; t0 < end; t0 += 8) {
    const int t = t0 + khalf;
    const bool valid = t < end && (p.window == 0 || t >= win_lo || t < p.sink);
    float kf[8], vf[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) kf[j] = vf[j] = 0.f;
    if (valid) {
      load_kv8(p.kcache, p.kscale, head_row0 + t, l16, fp8, kf);
      load_kv8(p.vcache, p.vscale, head_row0 + t, l16, fp8, vf);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s = fmaf(qv[g][j], kf[j], s);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (valid) {
        const float nm = fmaxf(mx[g], s);
        const float c = __expf(mx[g] - nm), e = __expf(s - nm);
        sum[g] = sum[g] * c + e;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(e, vf[j], acc[g][j] * c);
        mx[g] = nm;
      }
    }
  }

  // merge the two key halves of each warp, then the four warps
  __shared__ float s_m[4][G], s_l[4][G], s_acc[4][G][kD];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float om = __shfl_xor_sync(0xffffffffu, mx[g], 16);
    const float ol = __shfl_xor_sync(0xffffffffu, sum[g], 16);
    const float nm = fmaxf(mx[g], om);
    const float c0 = mx[g] == -INFINITY ? 0.f : __expf(mx[g] - nm);
    const float c1 = om == -INFINITY ? 0.f : __expf(om - nm);
    sum[g] = sum[g] * c0 + ol * c1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float oa = __shfl_xor_sync(0xffffffffu, acc[g][j], 16);
      acc[g][j] = acc[g][j] * c0 + oa * c1;
    }
    mx[g] = nm;
    if (khalf == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s_acc[warp][g][l16 * 8 + j] = acc[g][j];
      if (l16 == 0) {
        s_m[warp][g] = mx[g];
        s_l[warp][g] = sum[g];
      }
    }
  }
  __syncthreads();
  const int d = threadIdx.x;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float nm = fmaxf(fmaxf(s_m[0][g], s_m[1][g]), fmaxf(s_m[2][g], s_m[3][g]));
    float l = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = s_m[w][g] == -INFINITY ? 0.f : __expf(s_m[w][g] - nm);
      l += s_l[w][g] * c;
      a += s_acc[w][g][d] * c;
    }
    float* o = p.ws + (((size_t)m * p.Hq + hk * G + g) * p.nsplit + split) * (kD + 2);
    o[d] = a;
    if (d == 0) {
      o[kD] = nm;
      o[kD + 1] = l;
    }
  }
}

struct MergeParams {
  const float* ws;   // [M, Hq, nsplit, D + 2]
  int nsplit, Hq;
  const bf16* proj;  // gate source ([M, ld], gate of head h at h*2D + D), may be null
  int ld;
  bf16* out;         // [M, Hq*D]
};

__global__ void __launch_bounds__(kD) gqa_merge_kernel(const MergeParams p) {
  pk::pdl_wait();
  pk::pdl_trigger();
  const int m = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* w = p.ws + ((size_t)m * p.Hq + h) * p.nsplit * (kD + 2);
  float nm = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) nm = fmaxf(nm, w[s * (kD + 2) + kD]);
  float l = 0.f, a = 0.f;
  for (int s = 0; s < p.nsplit; ++s) {
    const float ms = w[s * (kD + 2) + kD];
    const float c = ms == -INFINITY ? 0.f : __expf(ms - nm);
    l += w[s * (kD + 2) + kD + 1] * c;
    a += w[s * (kD + 2) + d] * c;
  }
  float o = l > 0.f ? a / l : 0.f;
  if (p.proj != nullptr) {
    const float gate = __bfloat162float(p.proj[(size_t)m * p.ld + h * 2 * kD + kD + d]);
    o *= sigmoidf_(gate);
  }
  p.out[((size_t)m * p.Hq + h) * kD + d] = __float2bfloat16(o);
}

// Whole-vector variant (MiniMax-M2): the RMS statistic runs over all heads of q (or k) together with one gamma per
// element, the rotation is the half-split form on the first rope_dim dims of every head with angles from tables
// [ctx, rope_dim / 2], and k / v go to position pos[t] of caches [Hkv, ctx_cap, 128]. Inputs are the bf16 projections.
struct FullQkParams {
  const bf16* q;   // [T, Hq * D], row stride ldq
  const bf16* k;   // [T, Hkv * D], row stride ldk
  const bf16* v;   // [T, Hkv * D], row stride ldv
  int ldq, ldk, ldv;
  int Hq, Hkv;
  const int* pos;
  const float* q_gamma;
  const float* k_gamma;
  float eps;
  int rope_dim;
  const float* cos_t;
  const float* sin_t;
  bf16* q_out;     // [T, Hq, D]
  bf16* kcache;
  bf16* vcache;
  int ctx_cap;
};

__global__ void __launch_bounds__(256) full_qk_norm_rope_append_kernel(const FullQkParams p) {
  __shared__ float red[40];
  const int t = blockIdx.x, is_k = blockIdx.y, tid = threadIdx.x;
  const int H = is_k ? p.Hkv : p.Hq, n = H * kD;
  const bf16* x = is_k ? p.k + (size_t)t * p.ldk : p.q + (size_t)t * p.ldq;
  const float* gamma = is_k ? p.k_gamma : p.q_gamma;
  float ss = 0.f;
  for (int i = tid; i < n; i += 256) {
    const float v = __bfloat162float(x[i]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / (float)n + p.eps);
  const int pos = p.pos[t], half = p.rope_dim >> 1;
  const bool in_cache = pos >= 0 && pos < p.ctx_cap;
  if (!in_cache && threadIdx.x == 0) PK_DEBUG_RECORD(101, pos, p.ctx_cap);
  for (int i = tid; i < n; i += 256) {
    const int head = i >> 7, d = i & (kD - 1);
    float y = __bfloat162float(x[i]) * rs * gamma[i];
    if (d < p.rope_dim) {
      const int j = d < half ? d : d - half, o = d < half ? i + half : i - half;
      const float yo = __bfloat162float(x[o]) * rs * gamma[o];
      const float cs = p.cos_t[(size_t)pos * half + j], sn = p.sin_t[(size_t)pos * half + j];
      y = d < half ? y * cs - yo * sn : y * cs + yo * sn;
    }
    if (!is_k) {
      p.q_out[((size_t)t * p.Hq + head) * kD + d] = __float2bfloat16(y);
    } else if (in_cache) {
      const size_t ci = ((size_t)head * p.ctx_cap + pos) * kD + d;
      p.kcache[ci] = __float2bfloat16(y);
      p.vcache[ci] = p.v[(size_t)t * p.ldv + i];
    }
  }
}

}  // namespace

PK_API int pk_full_qk_norm_rope_append(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, int T, int Hq, int Hkv,
                                       int head_dim, const int* pos,
                                       const float* q_gamma, const float* k_gamma, float eps, int rope_dim, const float* cos_t,
                                       const float* sin_t, void* q_out, void* kcache, void* vcache, int ctx_cap, cudaStream_t stream) {
  if (head_dim != kD) return PK_ERR_UNSUPPORTED;
  if (T < 1 || rope_dim < 0 || rope_dim > kD || (rope_dim & 1)) return PK_ERR_BAD_ARG;
  FullQkParams p{(const pk::bf16*)q, (const pk::bf16*)k, (const pk::bf16*)v, ldq, ldk, ldv, Hq, Hkv, pos, q_gamma, k_gamma, eps, rope_dim, cos_t, sin_t,
                 (pk::bf16*)q_out, (pk::bf16*)kcache, (pk::bf16*)vcache, ctx_cap};
  full_qk_norm_rope_append_kernel<<<dim3(T, 2), 256, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

namespace {
}  // namespace

// kscale / vscale non-null: FP8 KV cache (kcache / vcache hold one E4M3 code per channel, the scales one fp32 per 64
// channels: [Hkv, ctx_cap, 2]); null: bf16 caches.
PK_API int pk_qk_norm_rope_append_kv(const void* proj, int ld, int M, int Hq, int Hkv, int head_dim,
                                     const int* pos, const float* q_gamma, const float* k_gamma, float eps,
                                     int rotary_dim, float theta, void* q_out, void* kcache, void* vcache, float* kscale,
                                     float* vscale, int ctx_cap, cudaStream_t stream) {
  if (head_dim != kD) return PK_ERR_UNSUPPORTED;
  if (M < 1 || rotary_dim < 0 || rotary_dim > kD || (rotary_dim & 1) || (kscale == nullptr) != (vscale == nullptr)) return PK_ERR_BAD_ARG;
  QkParams p{(const pk::bf16*)proj, ld, M, Hq, Hkv, pos, q_gamma, k_gamma, eps, rotary_dim, theta,
             (pk::bf16*)q_out, (pk::bf16*)kcache, (pk::bf16*)vcache, ctx_cap, kscale != nullptr ? 1 : 0, kscale, vscale};
  PK_LAUNCH_PDL(qk_norm_rope_append_kernel, dim3(M, Hq + Hkv), dim3(kD), 0, stream, p);
  return PK_OK;
}

PK_API int pk_qk_norm_rope_append(const void* proj, int ld, int M, int Hq, int Hkv, int head_dim,
                                  const int* pos, const float* q_gamma, const float* k_gamma, float eps,
                                  int rotary_dim, float theta, void* q_out, void* kcache, void* vcache,
                                  int ctx_cap, cudaStream_t stream) {
  return pk_qk_norm_rope_append_kv(proj, ld, M, Hq, Hkv, head_dim, pos, q_gamma, k_gamma, eps, rotary_dim, theta, q_out, kcache, vcache,
                                   nullptr, nullptr, ctx_cap, stream);
}

PK_API int pk_gqa_decode_kv(const void* q, const void* kcache, const void* vcache, const float* kscale, const float* vscale,
                            const int* pos, int M, int Hq, int Hkv, int head_dim, int ctx_cap, float scale, int nsplit,
                            int window, int sink, float* ws, const void* gate_proj, int ld, void* out, cudaStream_t stream);

PK_API int pk_gqa_decode(const void* q, const void* kcache, const void* vcache, const int* pos, int M,
                         int Hq, int Hkv, int head_dim, int ctx_cap, float scale, int nsplit, int window,
                         int sink, float* ws, const void* gate_proj, int ld, void* out,
                         cudaStream_t stream) {
  return pk_gqa_decode_kv(q, kcache, vcache, nullptr, nullptr, pos, M, Hq, Hkv, head_dim, ctx_cap, scale, nsplit, window, sink, ws,
                          gate_proj, ld, out, stream);
}

// ws must hold M * Hq * nsplit * (head_dim + 2) floats. kscale / vscale non-null: FP8 KV cache (see the append).
PK_API int pk_gqa_decode_kv(const void* q, const void* kcache, const void* vcache, const float* kscale, const float* vscale,
                            const int* pos, int M, int Hq, int Hkv, int head_dim, int ctx_cap, float scale, int nsplit,
                            int window, int sink, float* ws, const void* gate_proj, int ld, void* out, cudaStream_t stream) {
  if (head_dim != kD) return PK_ERR_UNSUPPORTED;
  if (M < 1 || nsplit < 1 || Hkv < 1 || Hq < Hkv || ctx_cap < 1) return PK_ERR_BAD_ARG;   // before any division by Hkv
  if (Hq % Hkv != 0) return PK_ERR_BAD_ARG;
  if ((kscale == nullptr) != (vscale == nullptr)) return PK_ERR_BAD_ARG;
  DecodeParams p{(const pk::bf16*)q, (const pk::bf16*)kcache, (const pk::bf16*)vcache, pos, M, Hq, Hkv,
                 ctx_cap, scale, nsplit, window, sink, ws, kscale != nullptr ? 1 : 0, kscale, vscale};
  const dim3 grid(Hkv, nsplit, M);
  switch (Hq / Hkv) {
    case 1: PK_LAUNCH_PDL(gqa_decode_split_kernel<1>, grid, dim3(128), 0, stream, p); break;
    case 2: PK_LAUNCH_PDL(gqa_decode_split_kernel<2>, grid, dim3(128), 0, stream, p); break;
    case 3: PK_LAUNCH_PDL(gqa_decode_split_kernel<3>, grid, dim3(128), 0, stream, p); break;
    case 4: PK_LAUNCH_PDL(gqa_decode_split_kernel<4>, grid, dim3(128), 0, stream, p); break;
    case 5: PK_LAUNCH_PDL(gqa_decode_split_kernel<5>, grid, dim3(128), 0, stream, p); break;
    case 6: PK_LAUNCH_PDL(gqa_decode_split_kernel<6>, grid, dim3(128), 0, stream, p); break;
    case 8: PK_LAUNCH_PDL(gqa_decode_split_kernel<8>, grid, dim3(128), 0, stream, p); break;
    default: return PK_ERR_UNSUPPORTED;
  }
  PK_CHECK_LAUNCH();
  MergeParams mp{ws, nsplit, Hq, (const pk::bf16*)gate_proj, ld, (pk::bf16*)out};
  PK_LAUNCH_PDL(gqa_merge_kernel, dim3(M, Hq), dim3(kD), 0, stream, mp);
  return PK_OK;
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant: the split partials live in a fixed array inside the library
// image instead of a caller-provided workspace. Contract in pk_gqa_decode_static.h.
#include <cstdio>
#include <mutex>

#include "pk_gqa_decode_static.h"

namespace {
static __device__ __align__(256) float g_gqa_static_ws[PK_GQA_STATIC_WS_FLOATS];

constexpr int kMaxStaticDevices = 64;
float* g_gqa_static_ptr[kMaxStaticDevices] = {};   // device address of the array, per device
std::mutex g_gqa_static_mu;
thread_local char g_gqa_static_msg[192] = "";
}  // namespace

PK_API const char* pk_gqa_decode_static_error(void) { return g_gqa_static_msg; }

PK_API int pk_gqa_decode_static(const void* q, const void* kcache, const void* vcache, const int* pos, int M,
                                int Hq, int Hkv, int head_dim, int ctx_cap, float scale, int nsplit,
                                int window, int sink, const void* gate_proj, int ld, void* out,
                                cudaStream_t stream) {
  g_gqa_static_msg[0] = 0;
  if (M < 1 || Hq < 1 || nsplit < 1 || head_dim < 1) {
    snprintf(g_gqa_static_msg, sizeof g_gqa_static_msg, "pk_gqa_decode_static: M, Hq, nsplit and head_dim must be positive");
    return PK_ERR_BAD_ARG;
  }
  if (Hkv < 1 || Hq < Hkv || Hq % Hkv != 0 || ctx_cap < 1) {
    snprintf(g_gqa_static_msg, sizeof g_gqa_static_msg,
             "pk_gqa_decode_static: Hkv must be positive and divide Hq, ctx_cap must be positive (Hq %d, Hkv %d, ctx_cap %d)", Hq, Hkv,
             ctx_cap);
    return PK_ERR_BAD_ARG;
  }
  const unsigned long long need = (unsigned long long)M * Hq * nsplit * (head_dim + 2);
  if (need > (unsigned long long)PK_GQA_STATIC_WS_FLOATS) {
    snprintf(g_gqa_static_msg, sizeof g_gqa_static_msg,
             "pk_gqa_decode_static: M*Hq*nsplit*(head_dim+2) = %llu floats exceeds the fixed scratch of %d floats; "
             "use pk_gqa_decode with your own workspace",
             need, (int)PK_GQA_STATIC_WS_FLOATS);
    return PK_ERR_BAD_ARG;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    pk_set_last_cuda_error((int)e);
    return PK_ERR_CUDA;
  }
  if (dev < 0 || dev >= kMaxStaticDevices) {
    snprintf(g_gqa_static_msg, sizeof g_gqa_static_msg, "pk_gqa_decode_static: device ordinal %d is not supported", dev);
    return PK_ERR_UNSUPPORTED;
  }
  float* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_gqa_static_mu);
    ws = g_gqa_static_ptr[dev];
    if (ws == nullptr) {   // first call on this device: resolve the array's device address
      e = cudaGetSymbolAddress((void**)&ws, g_gqa_static_ws);
      if (e != cudaSuccess || ws == nullptr) {
        pk_set_last_cuda_error((int)e);
        snprintf(g_gqa_static_msg, sizeof g_gqa_static_msg, "pk_gqa_decode_static: cudaGetSymbolAddress failed (%s)",
                 cudaGetErrorString(e));
        return PK_ERR_CUDA;
      }
      g_gqa_static_ptr[dev] = ws;
    }
  }
  return pk_gqa_decode(q, kcache, vcache, pos, M, Hq, Hkv, head_dim, ctx_cap, scale, nsplit, window, sink, ws,
                       gate_proj, ld, out, stream);
}

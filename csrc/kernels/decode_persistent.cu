// Persistent single-token decode kernel (contract and rationale in pk_decode_persistent.h).
//
// Layout of one block (512 threads = 16 warps = 4 groups of 128 threads, one block per SM):
//   * every warp owns a 4-slot ring in shared memory (a slot = 1 KB of each of two weight rows); lane 0 keeps it
//     full with cp.async.bulk copies that complete on per-slot mbarriers. The producer cursor walks the token's
//     segment list (5 per layer + lm_head) independently of the consumer, so weights of the next phases are in
//     flight while the block stages activations or waits at a barrier.
//   * a segment's row pairs are split evenly over blocks, and a block's (pair, 1 KB chunk) items evenly over its
//     warps ("flat" partition); partial sums of pairs shared by warps are added in warp order (deterministic).
//   * activations are staged as fp16 in [-1, 1] (power-of-two range scale), FP8 codes are unpacked to fp16 pairs
//     and accumulated with packed fp16 FMAs four at a time, then folded into fp32 with the 128x128 block scale:
//     the arithmetic of the per-projection kernels in matvec.cu.
//   * the non-linear phases run on groups of 128 threads: Gated DeltaNet step on (value head, 8 state columns)
//     units, GQA attention on (kv head, context split) units, the split merge on q heads.
#include <cstdio>

#include "../common/pk_comm.cuh"
#include "../common/pk_common.cuh"
#include "../common/pk_sm100.cuh"
#include "pk_decode_persistent.h"

namespace {

using namespace pk;

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kGroups = kThreads / 128;
// Bulk copies are issued at a bounded rate per SM (measured on B200: 1 KB copies top out at 4.2 TB/s over the whole
// chip whatever the ring depth, 2 KB copies reach 5.7-5.9 TB/s with two slots per warp), so a slot holds 2 KB per row.
constexpr int kSlots = 2;
constexpr int kRowSlot = 2048;             // bytes of one row in a slot
constexpr int kAhead = 0;                  // L2 window behind the ring, in items per warp; 0 = off (measured slower, see ring_window)
constexpr int kSlotBytes = 2 * kRowSlot;   // a row pair
constexpr int kD = 128;                    // head dim of attention and DeltaNet
constexpr int kSmemMax = 227 * 1024;

struct Plan {
  int off_scratch;   // fp32 row used by the norm prologues (after the staged fp16 row at offset 0)
  int off_acc;       // per-block accumulators [pairs][2]
  int off_ring;
  int off_bar;
  int group_floats;  // per-group scratch of the attention / DeltaNet phases (inside the region at offset 0)
  int total;
};

struct Seg {
  const uint8_t* w;
  const float* scale;
  int N, K, elem, swiglu;
  int half_n, g_lo, g_hi, cpr, rowbytes, begin, end;
};

// Where a warp is in its fixed walk over the token's weights: segment, flat item index inside it, and the segment's geometry.
struct Cursor {
  int seg;             // segment the cursor is in (-1 before the first)
  int pos, end;        // flat item index of this warp inside that segment
  int cpr, glo, half, N, rowbytes, swiglu;
  const uint8_t* w;
  bool done;
};

struct Ring {
  uint8_t* base;
  uint64_t* bars;
  uint32_t pk, ck;     // slots requested / slots consumed
  uint32_t qk;         // items the L2 prefetch cursor has passed (>= pk)
  Cursor f;            // fill cursor: next item to copy into the ring
  Cursor q;            // prefetch cursor: runs kAhead items ahead of the fill cursor and pulls their bytes into L2
  bool done;
};

struct Ctx {
  unsigned long long base;
  int mark;
  uint32_t bar_idx;
  uint32_t epoch;
  uint64_t budget_ns;
};

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float ldcg_bf16(const bf16* p) {
  return bf16_bits_to_float(__ldcg(reinterpret_cast<const unsigned short*>(p)));
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16(v)); }

__device__ __forceinline__ void group_bar(int grp) {
  asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(128) : "memory");
}

// Sum over the 128 threads of a group. `red4` holds 4 floats of that group.
__device__ __forceinline__ float group_sum(float v, float* red4, int grp, int t) {
  v = warp_sum(v);
  group_bar(grp);
  if ((t & 31) == 0) red4[t >> 5] = v;
  group_bar(grp);
  return (red4[0] + red4[1]) + (red4[2] + red4[3]);
}

__device__ __forceinline__ int staged_index(int k) {
  const int blk = k >> 9, r = k & 511;
  return (blk << 9) + (((r >> 3) & 1) << 8) + ((r >> 4) << 3) + (r & 7);
}

__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t v16) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v16, __NV_E4M3);
  return *reinterpret_cast<__half2*>(&h);
}

// 16 fp8 codes times 16 staged activations -> fp32 partial (unscaled). The conversion instruction and the packed
// fp16 FMAs set the pace of the whole kernel (it is bound by instruction issue, not by HBM). Decoding half of the
// codes with integer operations instead (the byte moved to the top of a 16-bit lane and shifted right by one is the
// fp16 encoding of value * 2^-8) was measured and lost: 9.8 against 9.2 ms per token on the 27B shape.
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

__device__ __forceinline__ float pow2_at_least(float a) {
  int e;
  const float m = frexpf(a, &e);
  return ldexpf(1.f, m == 0.5f ? e - 1 : e);
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   sm100::smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(sm100::smem_u32(bar))
               : "memory");
}

// Phase trace (block 0, thread 0): ids 1 norm staging, 8 plain staging, 9 head-norm staging, 10..14 the five
// projections of a layer, 20 lm_head, 3 grid barrier, 4 site barrier, 5 DeltaNet step, 6 attention splits, 7 merge.
__device__ __forceinline__ void mark(const PkDecParams& p, Ctx& c, int id) {
  if (p.dbg != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && c.mark < p.dbg_cap) {
    p.dbg[2 * c.mark] = (unsigned long long)id;
    p.dbg[2 * c.mark + 1] = global_timer_ns();
    ++c.mark;
  }
}

// ---------------------------------------------------------------------------------------------------------
// segments

__device__ __forceinline__ bool load_seg(const PkDecParams& p, int seg, int warp, Seg& s) {
  const int last = 5 * p.n_layers;
  if (seg > last) return false;
  if (seg == last) {
    s.w = (const uint8_t*)p.lm_head.w;
    s.scale = p.lm_head.scale;
    s.N = p.lm_head.N;
    s.K = p.lm_head.K;
    s.elem = p.lm_head.elem;
  } else {
    const PkDecLinear* l = &p.layers[seg / 5].lin[seg % 5];
    s.w = (const uint8_t*)l->w;
    s.scale = l->scale;
    s.N = l->N;
    s.K = l->K;
    s.elem = l->elem;
  }
  s.swiglu = (seg != last && seg % 5 == 3) ? 1 : 0;
  s.half_n = s.N >> 1;
  const int n_groups = s.swiglu ? s.half_n : (s.N + 1) >> 1;
  s.g_lo = (int)(((long long)blockIdx.x * n_groups) / gridDim.x);
  s.g_hi = (int)(((long long)(blockIdx.x + 1) * n_groups) / gridDim.x);
  s.rowbytes = s.K * s.elem;
  s.cpr = (s.rowbytes + kRowSlot - 1) / kRowSlot;
  const int flat_total = (s.g_hi - s.g_lo) * s.cpr;
  s.begin = (int)(((long long)warp * flat_total) / kWarps);
  s.end = (int)(((long long)(warp + 1) * flat_total) / kWarps);
  return true;
}

// Requests copies until the ring is full or the token's last segment is exhausted. Warp-uniform; lane 0 issues.
// Moves the cursor to its next item (loading the next segment's geometry when the current one is finished); false at the end.
__device__ __forceinline__ bool cursor_ready(const PkDecParams& p, Cursor& c, int warp) {
  while (!c.done && c.pos >= c.end) {
    Seg s;
    ++c.seg;
    if (!load_seg(p, c.seg, warp, s)) {
      c.done = true;
      break;
    }
    c.pos = s.begin;
    c.end = s.end;
    c.cpr = s.cpr;
    c.glo = s.g_lo;
    c.half = s.half_n;
    c.N = s.N;
    c.rowbytes = s.rowbytes;
    c.swiglu = s.swiglu;
    c.w = s.w;
  }
  return !c.done;
}

// The two row pieces of the cursor's item: addresses and byte count.
__device__ __forceinline__ void cursor_item(const Cursor& c, const uint8_t*& a0, const uint8_t*& a1, uint32_t& bytes) {
  const int gl = c.pos / c.cpr, ch = c.pos - gl * c.cpr;
  const int g = c.glo + gl;
  const int r0 = c.swiglu ? g : 2 * g;
  const int r1 = c.swiglu ? g + c.half : (2 * g + 1 < c.N ? 2 * g + 1 : 2 * g);
  const int kb0 = ch * kRowSlot;
  bytes = (uint32_t)min(kRowSlot, c.rowbytes - kb0);
  a0 = c.w + (size_t)r0 * c.rowbytes + kb0;
  a1 = c.w + (size_t)r1 * c.rowbytes + kb0;
}

__device__ __forceinline__ void l2_prefetch(const void* gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem), "r"(bytes) : "memory");
}

// Keeps the warp's ring full. The ring (128 KB per SM) drains in about 3 us, a phase boundary takes 5-10: ring_window()
// below uses the rest of the boundary.
__device__ __forceinline__ void ring_fill(const PkDecParams& p, Ring& r, int warp, int lane) {
  while (r.pk - r.ck < (uint32_t)kSlots && cursor_ready(p, r.f, warp)) {
    if (lane == 0) {
      const uint8_t *a0, *a1;
      uint32_t bytes;
      cursor_item(r.f, a0, a1, bytes);
      const int slot = (int)(r.pk % kSlots);
      uint8_t* dst = r.base + slot * kSlotBytes;
      sm100::mbar_arrive_expect_tx(&r.bars[slot], 2 * bytes);
      bulk_load(dst, a0, bytes, &r.bars[slot]);
      bulk_load(dst + kRowSlot, a1, bytes, &r.bars[slot]);
    }
    ++r.pk;
    ++r.f.pos;
  }
  r.done = r.f.done;
}

// Experiment kept behind kAhead: when the warp is about to wait at a phase boundary (grid barrier, other ranks' words) the next
// kAhead items behind the ring are pulled into L2 (`cp.async.bulk.prefetch.L2`), on the idea that HBM idles for most of a
// 5-10 us boundary once the 128 KB ring per SM is full. Measured on the 27B shape, one GPU, ms per token: off 6.73; four
// items per warp (38 MB per chip) at boundaries only 7.61; the same window kept up during streaming 7.75. Every byte is
// then requested twice and the per-SM request rate is what bounds the ring, so the window costs more than the idle time.
__device__ __forceinline__ void ring_window(const PkDecParams& p, Ring& r, int warp, int lane) {
  if (kAhead <= 0) return;
  if (r.qk < r.pk) {
    r.q = r.f;
    r.qk = r.pk;
  }
  while (r.qk < r.pk + (uint32_t)kAhead && cursor_ready(p, r.q, warp)) {
    if (lane == 0) {
      const uint8_t *a0, *a1;
      uint32_t bytes;
      cursor_item(r.q, a0, a1, bytes);
      l2_prefetch(a0, bytes);
      l2_prefetch(a1, bytes);
    }
    ++r.qk;
    ++r.q.pos;
  }
}

// ---------------------------------------------------------------------------------------------------------
// barriers

struct Shared {
  float red[64];
  float s_c;
  volatile uint32_t abort;
  int edge_g[kWarps][2];
  float edge_v[kWarps][2][2];
  float cand_v[kWarps];
  int cand_i[kWarps];
  float rope_cs[64], rope_sn[64];   // rotation of this token's position (rotary_dim <= 128)
};

__device__ __forceinline__ bool wait_failed(const PkDecParams& p, const Ctx& c, uint64_t t0, uint32_t& iter) {
  if ((++iter & 63u) != 0u) return false;
  if (*((volatile uint32_t*)p.status) != 0u) return true;
  return global_timer_ns() - t0 > c.budget_ns;
}

// Grid barrier. Returns false when the step has been given up.
__device__ __forceinline__ bool bar_grid(const PkDecParams& p, Ctx& c, Shared& sh) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long target = c.base + (unsigned long long)(c.bar_idx + 1u) * gridDim.x;
    __threadfence();
    atomicAdd(p.bar_count, 1ull);
    const uint64_t t0 = global_timer_ns();
    uint32_t iter = 0;
    while (ld_acquire_gpu_u64(p.bar_count) < target) {
      if (wait_failed(p, c, t0, iter)) {
        atomicCAS(p.status, 0u, PK_DEC_ERR_GRID_BARRIER);
        sh.abort = 1u;
        break;
      }
    }
  }
  __syncthreads();
  ++c.bar_idx;
  return sh.abort == 0u;
}

// ---------------------------------------------------------------------------------------------------------
// activation staging (all 512 threads)

__device__ __forceinline__ void block_sum_max(float& a, float& b, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_sum(a);
  b = warp_max(b);
  __syncthreads();
  if (lane == 0) {
    red[warp] = a;
    red[32 + warp] = b;
  }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    ta += red[w];
    tb = fmaxf(tb, red[32 + w]);
  }
  a = ta;
  b = tb;
}

__device__ __forceinline__ void unpack8(const uint4& xv, float (&v)[8]) {
  const uint32_t w[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
  }
}

// Eight consecutive activations (k a multiple of 8) -> fp16 at the staged position.
__device__ __forceinline__ void stage8(__half* xs, int k, const float (&t)[8], float cinv) {
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __half2 h = __floats2half2_rn(t[2 * j] * cinv, t[2 * j + 1] * cinv);
    out[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(xs + staged_index(k)) = make_uint4(out[0], out[1], out[2], out[3]);
}

// Loads four {value, sequence} words (two 16-byte volatile loads that bypass L1) until all four carry `seq`.
// Returns false when the budget ran out.
__device__ __forceinline__ bool ll_load4(const uint2* src, uint32_t seq, float (&v)[4], const PkDecParams& p, const Ctx& c,
                                         uint64_t t0) {
  uint32_t iter = 0;
  while (true) {
    uint4 a, b;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(src) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(src + 2) : "memory");
    if (a.y == seq && a.w == seq && b.y == seq && b.w == seq) {
      v[0] = __uint_as_float(a.x);
      v[1] = __uint_as_float(a.z);
      v[2] = __uint_as_float(b.x);
      v[3] = __uint_as_float(b.z);
      return true;
    }
    if (wait_failed(p, c, t0, iter)) return false;
  }
}

// x = bf16(x_in + sum_r parts[r]); optional store of x (block 0); y = bf16(rmsnorm(x) * (1 + gamma)); stage y.
// `parts` are this rank's {value, sequence} slots of site `site`; the loads wait for every word they add.
// Returns false when a wait ran out (status word set).
__device__ __forceinline__ bool stage_norm(const PkDecParams& p, const Ctx& c, Shared& sh, __half* xs, float* scratch,
                                           const bf16* x_in, const uint2* parts, int nparts, int site, bf16* hidden_out,
                                           const float* gamma, bf16* norm_out) {
  const int K = p.hidden, tid = threadIdx.x, nch = K >> 3;
  const bool wr = hidden_out != nullptr && blockIdx.x == 0;
  const uint32_t seq = c.epoch * p.sites_per_epoch + (uint32_t)site + 1u;
  const uint64_t t0 = nparts > 0 ? global_timer_ns() : 0ull;
  float ss = 0.f, amax = 0.f;
  bool good = true;
  // Optional two stages: with W slots a block reads W x hidden words per site (320 KB at W = 8, 47 MB over the grid).
  // Here every block adds the W partials and the residual for ITS slice of the columns only, publishes the rounded sums as
  // {value, sequence} words in this GPU's own buffer, and then every block polls those hidden words. Same bits as the
  // one-stage sum. Measured slower at W = 8 (4.83 against 4.58 ms per token), so the engine leaves it off.
  const bool two_stage = nparts > 0 && p.two_stage != 0 && p.red[site & 1] != nullptr;
  if (two_stage) {
    uint2* red = p.red[site & 1];
    const int c_lo = (int)(((long long)blockIdx.x * nch) / gridDim.x), c_hi = (int)(((long long)(blockIdx.x + 1) * nch) / gridDim.x);
    for (int c8 = c_lo + tid; c8 < c_hi && good; c8 += kThreads) {
      const int k = c8 * 8;
      float v[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(x_in + k)), v);
      for (int r = 0; r < nparts && good; ++r) {
        float lo[4], hi[4];
        good = ll_load4(parts + (size_t)r * K + k, seq, lo, p, c, t0) && ll_load4(parts + (size_t)r * K + k + 4, seq, hi, p, c, t0);
        if (good) {
          v[0] += lo[0]; v[1] += lo[1]; v[2] += lo[2]; v[3] += lo[3];
          v[4] += hi[0]; v[5] += hi[1]; v[6] += hi[2]; v[7] += hi[3];
        }
      }
      if (!good) break;
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        packed[j] = *reinterpret_cast<const uint32_t*>(&h2);
      }
      if (hidden_out != nullptr) *reinterpret_cast<uint4*>(hidden_out + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the bf16-rounded sums as fp32 bit patterns, two words per 16-byte store
        asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(red + k + 2 * j), "r"(packed[j] << 16), "r"(seq), "r"(packed[j] & 0xffff0000u), "r"(seq)
                     : "memory");
      }
    }
  }
  for (int c8 = tid; c8 < nch; c8 += kThreads) {
    const int k = c8 * 8;
    float v[8];
    if (two_stage) {
      float lo[4], hi[4];
      const uint2* red = p.red[site & 1];
      const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + k));
      const float4 gb = __ldg(reinterpret_cast<const float4*>(gamma + k + 4));
      good = good && ll_load4(red + k, seq, lo, p, c, t0) && ll_load4(red + k + 4, seq, hi, p, c, t0);
      if (!good) break;
      v[0] = lo[0]; v[1] = lo[1]; v[2] = lo[2]; v[3] = lo[3];
      v[4] = hi[0]; v[5] = hi[1]; v[6] = hi[2]; v[7] = hi[3];
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
      v[0] *= 1.f + ga.x; v[1] *= 1.f + ga.y; v[2] *= 1.f + ga.z; v[3] *= 1.f + ga.w;
      v[4] *= 1.f + gb.x; v[5] *= 1.f + gb.y; v[6] *= 1.f + gb.z; v[7] *= 1.f + gb.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      *reinterpret_cast<float4*>(scratch + k) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(scratch + k + 4) = make_float4(v[4], v[5], v[6], v[7]);
      continue;
    }
    // everything that does not depend on the pushed rows is requested before the first poll
    const uint4 xraw = __ldcg(reinterpret_cast<const uint4*>(x_in + k));
    const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma + k));
    const float4 gb = __ldg(reinterpret_cast<const float4*>(gamma + k + 4));
    unpack8(xraw, v);
    for (int r = 0; r < nparts && good; ++r) {
      float lo[4], hi[4];
      good = ll_load4(parts + (size_t)r * K + k, seq, lo, p, c, t0) && ll_load4(parts + (size_t)r * K + k + 4, seq, hi, p, c, t0);
      if (good) {
        v[0] += lo[0]; v[1] += lo[1]; v[2] += lo[2]; v[3] += lo[3];
        v[4] += hi[0]; v[5] += hi[1]; v[6] += hi[2]; v[7] += hi[3];
      }
    }
    if (nparts > 0) {
      uint32_t packed[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        packed[j] = *reinterpret_cast<const uint32_t*>(&h2);
        v[2 * j] = __uint_as_float(packed[j] << 16);
        v[2 * j + 1] = __uint_as_float(packed[j] & 0xffff0000u);
      }
      if (wr) *reinterpret_cast<uint4*>(hidden_out + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    v[0] *= 1.f + ga.x; v[1] *= 1.f + ga.y; v[2] *= 1.f + ga.z; v[3] *= 1.f + ga.w;
    v[4] *= 1.f + gb.x; v[5] *= 1.f + gb.y; v[6] *= 1.f + gb.z; v[7] *= 1.f + gb.w;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    *reinterpret_cast<float4*>(scratch + k) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(scratch + k + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
  if (!good) {
    atomicCAS(p.status, 0u, PK_COMM_TIMEOUT);
    sh.abort = 1u;
  }
  block_sum_max(ss, amax, sh.red);
  if (sh.abort != 0u) return false;
  const float rs = rsqrtf(ss / (float)K + p.eps);
  const float cc = pow2_at_least(fmaxf(amax * rs, 1e-30f));
  if (tid == 0) sh.s_c = cc;
  const float cinv = 1.f / cc;
  const bool wn = norm_out != nullptr && blockIdx.x == 0;
  for (int c8 = tid; c8 < nch; c8 += kThreads) {
    const int k = c8 * 8;
    const float4 a = *reinterpret_cast<const float4*>(scratch + k);
    const float4 b = *reinterpret_cast<const float4*>(scratch + k + 4);
    float t[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 h2 = __floats2bfloat162_rn(t[2 * j] * rs, t[2 * j + 1] * rs);
      packed[j] = *reinterpret_cast<const uint32_t*>(&h2);
      t[2 * j] = __uint_as_float(packed[j] << 16);
      t[2 * j + 1] = __uint_as_float(packed[j] & 0xffff0000u);
    }
    if (wn) *reinterpret_cast<uint4*>(norm_out + k) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    stage8(xs, k, t, cinv);
  }
  __syncthreads();
  return true;
}

// Stage a bf16 vector produced earlier in this launch (no norm). The raw values stay in registers between the
// magnitude pass and the conversion pass (up to 5 x 8 per thread); longer vectors are read twice.
__device__ __forceinline__ void stage_plain(Shared& sh, __half* xs, const bf16* x, int K) {
  constexpr int kKeep = 5;
  const int tid = threadIdx.x, nch = K >> 3;
  const bool keep = nch <= kKeep * kThreads;
  uint4 raw[kKeep];
  float ss = 0.f, amax = 0.f;
  if (keep) {
#pragma unroll
    for (int u = 0; u < kKeep; ++u) {
      const int c8 = tid + u * kThreads;
      raw[u] = c8 < nch ? __ldcg(reinterpret_cast<const uint4*>(x + c8 * 8)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kKeep; ++u) {
      float v[8];
      unpack8(raw[u], v);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
  } else {
    for (int c8 = tid; c8 < nch; c8 += kThreads) {
      float v[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(x + c8 * 8)), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
  }
  block_sum_max(ss, amax, sh.red);
  const float c = pow2_at_least(fmaxf(amax, 1e-30f));
  if (tid == 0) sh.s_c = c;
  const float cinv = 1.f / c;
  if (keep) {
#pragma unroll
    for (int u = 0; u < kKeep; ++u) {
      const int c8 = tid + u * kThreads;
      if (c8 < nch) {
        float v[8];
        unpack8(raw[u], v);
        stage8(xs, c8 * 8, v, cinv);
      }
    }
  } else {
    for (int c8 = tid; c8 < nch; c8 += kThreads) {
      float v[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(x + c8 * 8)), v);
      stage8(xs, c8 * 8, v, cinv);
    }
  }
  __syncthreads();
}

// DeltaNet output: y[h, d] = bf16(o[h, d] * rsqrt(mean_d o^2 + eps) * gamma[d] * silu(z[h, d])); stage y.
__device__ __forceinline__ void stage_headnorm(const PkDecParams& p, Shared& sh, __half* xs, float* scratch,
                                               const float* o_raw, const bf16* z, const float* gamma) {
  const int VD = p.vh_l * kD, tid = threadIdx.x, nch = VD >> 3;
  float ss_unused = 0.f, amax = 0.f;
  // 16 consecutive threads cover one head; the loop bound is rounded up so that whole half-warps stay together
  for (int c0 = 0; c0 < nch; c0 += kThreads) {
    const int c8 = c0 + tid;
    const bool ok = c8 < nch;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (ok) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(o_raw + c8 * 8));
      const float4 b = __ldcg(reinterpret_cast<const float4*>(o_raw + c8 * 8 + 4));
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    float oo = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) oo += v[j] * v[j];
    oo += __shfl_xor_sync(0xffffffffu, oo, 8);
    oo += __shfl_xor_sync(0xffffffffu, oo, 4);
    oo += __shfl_xor_sync(0xffffffffu, oo, 2);
    oo += __shfl_xor_sync(0xffffffffu, oo, 1);
    if (ok) {
      const float r = rsqrtf(oo / (float)kD + p.eps);
      const int d0 = (c8 * 8) & (kD - 1);
      float zz[8];
      unpack8(__ldcg(reinterpret_cast<const uint4*>(z + c8 * 8)), zz);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[j] = bf16r(v[j] * r * __ldg(gamma + d0 + j) * silu(zz[j]));
        amax = fmaxf(amax, fabsf(v[j]));
      }
      *reinterpret_cast<float4*>(scratch + c8 * 8) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(scratch + c8 * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  block_sum_max(ss_unused, amax, sh.red);
  const float c = pow2_at_least(fmaxf(amax, 1e-30f));
  if (tid == 0) sh.s_c = c;
  const float cinv = 1.f / c;
  for (int c8 = tid; c8 < nch; c8 += kThreads) {
    const float4 a = *reinterpret_cast<const float4*>(scratch + c8 * 8);
    const float4 b = *reinterpret_cast<const float4*>(scratch + c8 * 8 + 4);
    const float t[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    stage8(xs, c8 * 8, t, cinv);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------------------
// one weight-streaming segment: y = W x for this block's row pairs, then the epilogue

enum Epi { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_LOGITS = 2, EPI_PUSH = 3 };

struct EpiArgs {
  int kind;
  bf16* y_bf16;     // EPI_BF16 / EPI_SWIGLU destination (already offset)
  float* y_f32;     // EPI_LOGITS
  int site;         // EPI_PUSH
  uint32_t seq;     // EPI_PUSH: sequence number of the site
};

__device__ __forceinline__ void run_segment(const PkDecParams& p, Shared& sh, Ring& r, int seg_id, const __half* xs,
                                            float* s_acc, const EpiArgs& e) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Seg s;
  load_seg(p, seg_id, warp, s);
  const int ngb = s.g_hi - s.g_lo;
  __syncthreads();   // the previous segment's epilogue may still be reading the accumulators
  for (int i = tid; i < ngb * 2; i += kThreads) s_acc[i] = 0.f;
  if (tid < kWarps * 2) sh.edge_g[tid >> 1][tid & 1] = -1;
  __syncthreads();

  const int kb_count = (s.K + 127) >> 7;
  int pos = s.begin;
  bool ok = true;
  while (pos < s.end && ok) {
    const int gl = pos / s.cpr, ch = pos - gl * s.cpr, g = s.g_lo + gl;
    const int ch_stop = min(s.cpr, ch + (s.end - pos));
    const int r0 = s.swiglu ? g : 2 * g;
    const int r1 = s.swiglu ? g + s.half_n : (2 * g + 1 < s.N ? 2 * g + 1 : 2 * g);
    float a0 = 0.f, a1 = 0.f;
    const float* sc0 = s.scale ? s.scale + (size_t)(r0 >> 7) * kb_count : nullptr;
    const float* sc1 = s.scale ? s.scale + (size_t)(r1 >> 7) * kb_count : nullptr;
#pragma unroll 1
    for (int c = ch; c < ch_stop; ++c) {
      const int slot = (int)(r.ck % kSlots);
      if (!sm100::mbar_wait(&r.bars[slot], (r.ck / kSlots) & 1u, &sh.abort, p.status, PK_DEC_ERR_RING)) {
        ok = false;
        break;
      }
      const uint8_t* sp = r.base + slot * kSlotBytes;
      if (s.elem == 1) {
#pragma unroll
        for (int u = 0; u < kRowSlot / 512; ++u) {
          const int kq = c * kRowSlot + u * 512;
          const int ka = kq + (lane << 4);
          if (ka < s.K) {
            const uint4 wa = *reinterpret_cast<const uint4*>(sp + u * 512 + (lane << 4));
            const uint4 wb = *reinterpret_cast<const uint4*>(sp + kRowSlot + u * 512 + (lane << 4));
            const float sa = __ldg(sc0 + (ka >> 7)), sb = __ldg(sc1 + (ka >> 7));
            const uint4 x0 = *reinterpret_cast<const uint4*>(xs + kq + (lane << 3));
            const uint4 x1 = *reinterpret_cast<const uint4*>(xs + kq + (lane << 3) + 256);
            a0 = fmaf(dot16_fp8(wa, x0, x1), sa, a0);
            a1 = fmaf(dot16_fp8(wb, x0, x1), sb, a1);
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < kRowSlot / 1024; ++u) {
          const int kq = c * (kRowSlot / 2) + u * 512;
          const int ka = kq + (lane << 4);
          if (ka < s.K) {
            const uint4 w00 = *reinterpret_cast<const uint4*>(sp + u * 1024 + (lane << 5));
            const uint4 w01 = *reinterpret_cast<const uint4*>(sp + u * 1024 + (lane << 5) + 16);
            const uint4 w10 = *reinterpret_cast<const uint4*>(sp + kRowSlot + u * 1024 + (lane << 5));
            const uint4 w11 = *reinterpret_cast<const uint4*>(sp + kRowSlot + u * 1024 + (lane << 5) + 16);
            const uint4 x0 = *reinterpret_cast<const uint4*>(xs + kq + (lane << 3));
            const uint4 x1 = *reinterpret_cast<const uint4*>(xs + kq + (lane << 3) + 256);
            a0 += dot16_bf16(w00, w01, x0, x1);
            a1 += dot16_bf16(w10, w11, x0, x1);
          }
        }
      }
      ++r.ck;
      __syncwarp();   // every lane has read the slot: it can be refilled
      ring_fill(p, r, warp, lane);
    }
    a0 = warp_sum(a0);
    a1 = warp_sum(a1);
    if (lane == 0) {
      const bool whole = ch == 0 && ch_stop == s.cpr;
      const int eidx = pos == s.begin ? 0 : 1;
      if (whole) {
        s_acc[gl * 2] = a0;
        s_acc[gl * 2 + 1] = a1;
      } else {
        sh.edge_g[warp][eidx] = gl;
        sh.edge_v[warp][eidx][0] = a0;
        sh.edge_v[warp][eidx][1] = a1;
      }
    }
    pos += ch_stop - ch;
  }
  __syncthreads();

  // ---- epilogue ----
  const float sc = sh.s_c;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int gl = tid; gl < ngb; gl += kThreads) {
    const int g = s.g_lo + gl;
    float v0 = s_acc[gl * 2], v1 = s_acc[gl * 2 + 1];
#pragma unroll
    for (int w = 0; w < kWarps; ++w)
#pragma unroll
      for (int q = 0; q < 2; ++q)
        if (sh.edge_g[w][q] == gl) {
          v0 += sh.edge_v[w][q][0];
          v1 += sh.edge_v[w][q][1];
        }
    v0 *= sc;
    v1 *= sc;
    if (e.kind == EPI_SWIGLU) {
      e.y_bf16[g] = __float2bfloat16(silu(v0) * v1);
    } else {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int n = 2 * g + q;
        if (n >= s.N) continue;
        const float v = q == 0 ? v0 : v1;
        if (e.kind == EPI_BF16) {
          e.y_bf16[n] = __float2bfloat16(v);
        } else if (e.kind == EPI_LOGITS) {
          e.y_f32[n] = v;
          if (v > best || (v == best && n < bi)) {
            best = v;
            bi = n;
          }
        } else {
          // {value, sequence number} in one 8-byte store per rank: the consumer's poll of the word is the whole protocol
          const size_t off = (size_t)p.rank * p.hidden + n;
          const uint2 word = make_uint2(__float_as_uint(v), e.seq);
          for (int pr = 0; pr < p.world; ++pr)
            asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p.slot[e.site & 1][pr] + off), "r"(word.x), "r"(word.y) : "memory");
        }
      }
    }
  }
  if (e.kind == EPI_LOGITS) {
    // block argmax (lowest index on ties) -> this block's candidate
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sh.cand_v[warp] = best;
      sh.cand_i[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kWarps; ++w) {
        const float ov = sh.cand_v[w];
        const int oi = sh.cand_i[w];
        if (ov > best || (ov == best && oi < bi)) {
          best = ov;
          bi = oi;
        }
      }
      p.cand_val[blockIdx.x] = best;
      p.cand_idx[blockIdx.x] = bi == 0x7fffffff ? bi : bi + p.vocab_start;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Gated DeltaNet step on (value head, 8 state columns) units; conv tails are read only (they are shifted after
// the next barrier, when no block reads them any more).

__device__ __forceinline__ float conv_silu(const float* conv_w, const float* conv_state, const bf16* proj, int ch) {
  const float4 w = __ldg(reinterpret_cast<const float4*>(conv_w + (size_t)ch * 4));
  const float* cs = conv_state + (size_t)ch * 3;
  const float x = ldcg_bf16(proj + ch);
  const float y = w.x * cs[0] + w.y * cs[1] + w.z * cs[2] + w.w * x;
  return bf16r(silu(y));
}

__device__ __forceinline__ void deltanet_phase(const PkDecParams& p, const PkDecLayer& L, float* gsm_base, int group_floats) {
  const int tid = threadIdx.x, grp = tid >> 7, t = tid & 127, lane = tid & 31, wg = (tid >> 5) & 3;
  float* gs = gsm_base + (size_t)grp * group_floats;
  float* s_q = gs;               // [128]
  float* s_k = gs + 128;         // [128]
  float* s_v = gs + 256;         // [8]
  float* s_gate = gs + 264;      // [2]
  float* red12 = gs + 268;       // [3][4]
  float* s_part = gs + 280;      // [4 warps][2][8]
  const int KH = p.kh_l, VH = p.vh_l, rep = VH / KH;
  const int KD = KH * kD, VD = VH * kD;
  const bf16* proj = (const bf16*)p.proj;
  const float* conv_w = L.conv_w;
  const float* conv_state = L.conv_state;
  const float* A_log = L.A_log;
  const float* dt_bias = L.dt_bias;
  float* lin_state = L.lin_state;
  const int units = VH * 16;
  const float qscale = rsqrtf((float)kD);
  for (int v = blockIdx.x + gridDim.x * grp; v < units; v += gridDim.x * kGroups) {
    const int h = v >> 4, cb = v & 15, hk = h / rep;
    const int col = t & 7, rsub = t >> 3;
    // state column piece first: its latency overlaps the conv / norm work
    float S[8];
    float* sp = lin_state + ((size_t)h * kD + rsub * 8) * kD + cb * 8 + col;
#pragma unroll
    for (int i = 0; i < 8; ++i) S[i] = sp[(size_t)i * kD];
    const float yq = conv_silu(conv_w, conv_state, proj, hk * kD + t);
    const float yk = conv_silu(conv_w, conv_state, proj, KD + hk * kD + t);
    group_bar(grp);   // the previous unit of this group is done with the group scratch
    s_q[t] = yq;
    s_k[t] = yk;
    if (t < 8) s_v[t] = conv_silu(conv_w, conv_state, proj, 2 * KD + h * kD + cb * 8 + t);
    if (t == 8) {
      const float a = ldcg_bf16(proj + 2 * KD + 2 * VD + h);
      const float b = ldcg_bf16(proj + 2 * KD + 2 * VD + VH + h);
      s_gate[0] = __expf(-__expf(__ldg(A_log + h)) * softplusf_(a + __ldg(dt_bias + h)));
      s_gate[1] = sigmoidf_(b);
    }
    // three sums over the group in one exchange
    const float w0 = warp_sum(yq * yq), w1 = warp_sum(yk * yk), w2 = warp_sum(yq * yk);
    if (lane == 0) {
      red12[wg] = w0;
      red12[4 + wg] = w1;
      red12[8 + wg] = w2;
    }
    group_bar(grp);
    const float qq = (red12[0] + red12[1]) + (red12[2] + red12[3]);
    const float kk = (red12[4] + red12[5]) + (red12[6] + red12[7]);
    const float kqr = (red12[8] + red12[9]) + (red12[10] + red12[11]);
    const float qn = rsqrtf(qq + 1e-6f) * qscale, kn = rsqrtf(kk + 1e-6f);
    const float kq = kqr * kn * qn;
    const float decay = s_gate[0], beta = s_gate[1];
    float kv = 0.f, qv = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      kv = fmaf(S[i], s_k[rsub * 8 + i], kv);
      qv = fmaf(S[i], s_q[rsub * 8 + i], qv);
    }
    // lanes of a warp: (rsub & 3) * 8 + col -> sum over the four row groups, then over the four warps
    kv += __shfl_xor_sync(0xffffffffu, kv, 8);
    kv += __shfl_xor_sync(0xffffffffu, kv, 16);
    qv += __shfl_xor_sync(0xffffffffu, qv, 8);
    qv += __shfl_xor_sync(0xffffffffu, qv, 16);
    if (lane < 8) {
      s_part[(wg * 2) * 8 + lane] = kv;
      s_part[(wg * 2 + 1) * 8 + lane] = qv;
    }
    group_bar(grp);
    kv = ((s_part[0 * 8 + col] + s_part[2 * 8 + col]) + (s_part[4 * 8 + col] + s_part[6 * 8 + col])) * kn;
    qv = ((s_part[1 * 8 + col] + s_part[3 * 8 + col]) + (s_part[5 * 8 + col] + s_part[7 * 8 + col])) * qn;
    const float delta = (s_v[col] - decay * kv) * beta;
    const float o = decay * qv + kq * delta;
#pragma unroll
    for (int i = 0; i < 8; ++i) sp[(size_t)i * kD] = fmaf(s_k[rsub * 8 + i] * kn, delta, S[i] * decay);
    if (rsub == 0) p.o_raw[h * kD + cb * 8 + col] = o;
  }
}

// After the barrier that follows the DeltaNet phase: shift the newest input into every channel's conv tail.
__device__ __forceinline__ void conv_shift(const PkDecParams& p, const PkDecLayer& L) {
  const int C = 2 * p.kh_l * kD + p.vh_l * kD;
  const bf16* proj = (const bf16*)p.proj;
  float* conv_state = L.conv_state;
  for (int ch = blockIdx.x * kThreads + threadIdx.x; ch < C; ch += gridDim.x * kThreads) {
    float* cs = conv_state + (size_t)ch * 3;
    const float s1 = cs[1], s2 = cs[2];
    cs[0] = s1;
    cs[1] = s2;
    cs[2] = ldcg_bf16(proj + ch);
  }
}

// ---------------------------------------------------------------------------------------------------------
// GQA attention: (kv head, context split) units. Every unit rebuilds the normalised, rotated q heads of its kv
// group and the new key from the projection row; split 0 appends K / V at `pos` and also attends to it.

struct AttnArgs {
  const bf16* proj;
  const float* q_norm;
  const float* k_norm;
  bf16* kcache;
  bf16* vcache;
  float* attn_ws;
  const float* rope_cs;   // [rotary_dim / 2] cos / sin of pos * inv_freq (shared memory, built once per token)
  const float* rope_sn;
  float* kscale;          // FP8 KV cache: one fp32 scale per 64 channels [Hkv, ctx_cap, 2]; null = bf16 caches
  float* vscale;
  int hq_l, hkv_l, ctx_cap, window, sink, rotary_dim;
  float eps;
};

template <int G>
__device__ __noinline__ void attn_split_phase(const AttnArgs p, int pos, int S, float* gsm_base, int group_floats) {
  const int tid = threadIdx.x, grp = tid >> 7, t = tid & 127, lane = tid & 31, wg = (tid >> 5) & 3;
  const int l16 = lane & 15, khalf = lane >> 4;
  float* gs = gsm_base + (size_t)grp * group_floats;
  float* s_kn = gs;                   // [128] new key (normalised, rotated, bf16-rounded)
  float* s_vn = gs + 128;             // [128] new value
  float* red = gs + 256;              // [(G + 1)][4] (G <= 8 -> 36 floats, padded to 40)
  float* s_q = gs + 296;              // [G][128] q heads, pre-scaled
  float* s_m = s_q + G * kD;          // [4][G]
  float* s_l = s_m + 4 * G;           // [4][G]
  float* s_a = s_l + 4 * G;           // [4][G][128]; also the pre-rotation scratch [(G + 1)][128]
  const bf16* proj = p.proj;
  const int Hq = p.hq_l, Hkv = p.hkv_l;
  const float scale = rsqrtf((float)kD);
  const int len = min(pos, p.ctx_cap);          // cached keys
  int per = (max(len, 1) + S - 1) / S;
  per = (per + 7) & ~7;
  const int win_lo = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
  const int hr = p.rotary_dim >> 1;
  const int units = Hkv * S;
  for (int v = blockIdx.x + gridDim.x * grp; v < units; v += gridDim.x * kGroups) {
    const int hk = v / S, split = v - hk * S;
    const int start = split * per, end = min(len, start + per);
    const bf16* kbase = p.kcache + (size_t)hk * p.ctx_cap * kD;
    const bf16* vbase = p.vcache + (size_t)hk * p.ctx_cap * kD;
    // ---- q heads of the group and the new key: RMSNorm (1 + gamma), partial rotation, all heads at once ----
    float x[G + 1];
#pragma unroll
    for (int j = 0; j <= G; ++j) {
      const int off = j < G ? (hk * G + j) * 2 * kD : Hq * 2 * kD + hk * kD;
      x[j] = ldcg_bf16(proj + off + t);
    }
    const float vnew = ldcg_bf16(proj + Hq * 2 * kD + Hkv * kD + hk * kD + t);
    group_bar(grp);   // group scratch free (previous unit done)
#pragma unroll
    for (int j = 0; j <= G; ++j) {
      const float w = warp_sum(x[j] * x[j]);
      if (lane == 0) red[j * 4 + wg] = w;
    }
    group_bar(grp);
    const float gq = __ldg(p.q_norm + t), gk = __ldg(p.k_norm + t);
#pragma unroll
    for (int j = 0; j <= G; ++j) {
      const float ss = (red[j * 4] + red[j * 4 + 1]) + (red[j * 4 + 2] + red[j * 4 + 3]);
      x[j] = bf16r(x[j] * rsqrtf(ss / (float)kD + p.eps) * (1.f + (j < G ? gq : gk)));
      s_a[j * kD + t] = x[j];
    }
    group_bar(grp);
    {
      const bool rot = t < p.rotary_dim;
      const int i = t < hr ? t : t - hr;
      const float cs = rot ? p.rope_cs[i] : 1.f, sn = rot ? p.rope_sn[i] : 0.f;
      const int ot = rot ? (t < hr ? t + hr : t - hr) : t;
#pragma unroll
      for (int j = 0; j <= G; ++j) {
        float y = x[j];
        if (rot) {
          const float other = s_a[j * kD + ot];
          y = t < hr ? y * cs - other * sn : y * cs + other * sn;
        }
        y = bf16r(y);
        if (j < G) s_q[j * kD + t] = y * scale;
        else s_kn[t] = y;
      }
    }
    s_vn[t] = vnew;
    if (p.kscale == nullptr) {
      if (split == 0 && pos >= 0 && pos < p.ctx_cap) {
        const size_t ci = ((size_t)hk * p.ctx_cap + pos) * kD + t;
        p.kcache[ci] = __float2bfloat16(s_kn[t]);
        p.vcache[ci] = __float2bfloat16(vnew);
      }
    } else if (split == 0) {
      // FP8 cache: E4M3 codes with one scale per 64 channels (amax / 448); the step attends to the stored values
      const float kvv = s_kn[t];
      const float ka = warp_max(fabsf(kvv)), va = warp_max(fabsf(vnew));
      group_bar(grp);   // the norm sums in `red` have been read by every thread
      if (lane == 0) {
        red[wg] = ka;
        red[4 + wg] = va;
      }
      group_bar(grp);
      const int half = t >> 6;
      const float kmax = fmaxf(red[2 * half], red[2 * half + 1]), vmax = fmaxf(red[4 + 2 * half], red[4 + 2 * half + 1]);
      const float ks = kmax > 0.f ? kmax / 448.f : 1.f, vs = vmax > 0.f ? vmax / 448.f : 1.f;
      const uint8_t kc = float_to_e4m3(kvv / ks), vc = float_to_e4m3(vnew / vs);
      s_kn[t] = e4m3_to_float(kc) * ks;
      s_vn[t] = e4m3_to_float(vc) * vs;
      if (pos >= 0 && pos < p.ctx_cap) {
        const size_t ri = (size_t)hk * p.ctx_cap + pos;
        reinterpret_cast<uint8_t*>(p.kcache)[ri * kD + t] = kc;
        reinterpret_cast<uint8_t*>(p.vcache)[ri * kD + t] = vc;
        if ((t & 63) == 0) {
          p.kscale[ri * 2 + half] = ks;
          p.vscale[ri * 2 + half] = vs;
        }
      }
    }
    group_bar(grp);

    float qv[G][8], mx[G], sum[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        qv[g][j] = s_q[g * kD + l16 * 8 + j];
        acc[g][j] = 0.f;
      }
      mx[g] = -INFINITY;
      sum[g] = 0.f;
    }
    auto step = [&](const float (&kf)[8], const float (&vf)[8], bool valid) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sdot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) sdot = fmaf(qv[g][j], kf[j], sdot);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 8);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 4);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 2);
        sdot += __shfl_xor_sync(0xffffffffu, sdot, 1);
        if (valid) {
          const float nm = fmaxf(mx[g], sdot);
          const float c = __expf(mx[g] - nm), ex = __expf(sdot - nm);
          sum[g] = sum[g] * c + ex;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(ex, vf[j], acc[g][j] * c);
          mx[g] = nm;
        }
      }
    };
    // cached keys: a warp takes keys t0 + khalf, two such pairs per iteration so that four 16-byte loads are in flight
    for (int t0 = start + wg * 2; t0 < end; t0 += 16) {
      uint4 kr[2], vr[2];
      float ksc[2] = {1.f, 1.f}, vsc[2] = {1.f, 1.f};
      bool valid[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int tt = t0 + u * 8 + khalf;
        valid[u] = tt < end && (p.window == 0 || tt >= win_lo || tt < p.sink);
        kr[u] = vr[u] = make_uint4(0, 0, 0, 0);
        if (valid[u]) {
          if (p.kscale == nullptr) {
            kr[u] = __ldcg(reinterpret_cast<const uint4*>(kbase + (size_t)tt * kD + l16 * 8));
            vr[u] = __ldcg(reinterpret_cast<const uint4*>(vbase + (size_t)tt * kD + l16 * 8));
          } else {
            // one byte per channel: 8 bytes per lane, and the scale of the lane's 64-channel group
            const size_t ri = (size_t)hk * p.ctx_cap + tt;
            const uint2 k8 = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.kcache) + ri * kD + l16 * 8));
            const uint2 v8 = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.vcache) + ri * kD + l16 * 8));
            kr[u] = make_uint4(k8.x, k8.y, 0, 0);
            vr[u] = make_uint4(v8.x, v8.y, 0, 0);
            ksc[u] = __ldcg(p.kscale + ri * 2 + (l16 >> 3));
            vsc[u] = __ldcg(p.vscale + ri * 2 + (l16 >> 3));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (t0 + u * 8 >= end) break;   // warp-uniform
        float kf[8], vf[8];
        if (p.kscale == nullptr) {
          unpack8(kr[u], kf);
          unpack8(vr[u], vf);
        } else {
          const uint32_t kw[2] = {kr[u].x, kr[u].y}, vw[2] = {vr[u].x, vr[u].y};
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float2 a = e4m3x2_to_float2((uint16_t)(kw[j] & 0xffffu)), b = e4m3x2_to_float2((uint16_t)(kw[j] >> 16));
            const float2 c2 = e4m3x2_to_float2((uint16_t)(vw[j] & 0xffffu)), d2 = e4m3x2_to_float2((uint16_t)(vw[j] >> 16));
            kf[4 * j] = a.x * ksc[u]; kf[4 * j + 1] = a.y * ksc[u]; kf[4 * j + 2] = b.x * ksc[u]; kf[4 * j + 3] = b.y * ksc[u];
            vf[4 * j] = c2.x * vsc[u]; vf[4 * j + 1] = c2.y * vsc[u]; vf[4 * j + 2] = d2.x * vsc[u]; vf[4 * j + 3] = d2.y * vsc[u];
          }
        }
        step(kf, vf, valid[u]);
      }
    }
    // the new key, from shared memory: warp 0 of split 0
    if (split == 0 && wg == 0) {
      float kf[8], vf[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        kf[j] = s_kn[l16 * 8 + j];
        vf[j] = s_vn[l16 * 8 + j];
      }
      step(kf, vf, khalf == 0);
    }
    // merge the two key halves of each warp, then the four warps of the group
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
        for (int j = 0; j < 8; ++j) s_a[(wg * G + g) * kD + l16 * 8 + j] = acc[g][j];
        if (l16 == 0) {
          s_m[wg * G + g] = mx[g];
          s_l[wg * G + g] = sum[g];
        }
      }
    }
    group_bar(grp);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float nm = fmaxf(fmaxf(s_m[g], s_m[G + g]), fmaxf(s_m[2 * G + g], s_m[3 * G + g]));
      float l = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float c = s_m[w * G + g] == -INFINITY ? 0.f : __expf(s_m[w * G + g] - nm);
        l += s_l[w * G + g] * c;
        a += s_a[(w * G + g) * kD + t] * c;
      }
      float* o = p.attn_ws + ((size_t)(hk * G + g) * S + split) * (kD + 2);
      o[t] = a;
      if (t == 0) {
        o[kD] = nm;
        o[kD + 1] = l;
      }
    }
  }
}

__device__ __forceinline__ void attn_merge_phase(const PkDecParams& p, int S) {
  const int tid = threadIdx.x, grp = tid >> 7, t = tid & 127;
  const bf16* proj = (const bf16*)p.proj;
  for (int h = blockIdx.x + gridDim.x * grp; h < p.hq_l; h += gridDim.x * kGroups) {
    const float* w = p.attn_ws + (size_t)h * S * (kD + 2);
    float nm = -INFINITY;
    for (int s = 0; s < S; ++s) nm = fmaxf(nm, __ldcg(w + s * (kD + 2) + kD));
    float l = 0.f, a = 0.f;
    for (int s = 0; s < S; ++s) {
      const float ms = __ldcg(w + s * (kD + 2) + kD);
      const float c = ms == -INFINITY ? 0.f : __expf(ms - nm);
      l += __ldcg(w + s * (kD + 2) + kD + 1) * c;
      a += __ldcg(w + s * (kD + 2) + t) * c;
    }
    float o = l > 0.f ? a / l : 0.f;
    if (p.attn_gate) o *= sigmoidf_(ldcg_bf16(proj + h * 2 * kD + kD + t));
    ((bf16*)p.attn_out)[h * kD + t] = __float2bfloat16(o);
  }
}

// ---------------------------------------------------------------------------------------------------------

// The token as a list of steps, seven per layer plus the head. Each step is (mixer phase | activation staging),
// an optional weight-streaming segment and an optional grid barrier; every device function has exactly one call
// site in the loop below, which keeps the kernel's code small enough to stay in the instruction cache (an earlier
// form with one inlined copy per phase was 500 KB of code and paid for the misses at every phase change).
//   0 input norm -> in_proj / qkv            (barrier on full-attention layers)
//   1 in_proj a|b rows, barrier             (linear layers)
//   2 DeltaNet step | attention splits, barrier
//   3 attention merge, barrier               (full-attention layers)
//   4 conv shift + head norm | attention output -> out_proj / o_proj, pushed to every rank
//   5 post norm (waits for the pushed rows) -> gate|up with SwiGLU, barrier
//   6 mlp activations -> down, pushed to every rank
template <int G>
__global__ void __launch_bounds__(kThreads, 1) decode_persistent_kernel(const PkDecParams p, const Plan plan) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ Shared sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __half* xs = reinterpret_cast<__half*>(smem);
  float* scratch = reinterpret_cast<float*>(smem + plan.off_scratch);
  float* gsm = reinterpret_cast<float*>(smem);
  float* s_acc = reinterpret_cast<float*>(smem + plan.off_acc);

  Ring ring;
  ring.base = smem + plan.off_ring + warp * (kSlots * kSlotBytes);
  ring.bars = reinterpret_cast<uint64_t*>(smem + plan.off_bar) + warp * kSlots;
  ring.pk = ring.ck = 0;
  ring.qk = 0;
  ring.f.seg = -1;
  ring.f.pos = ring.f.end = 0;
  ring.f.done = false;
  ring.q = ring.f;
  ring.done = false;
  if (tid == 0) sh.abort = *((volatile uint32_t*)p.status) != 0u ? 1u : 0u;
  if (tid < (p.rotary_dim >> 1) && tid < 64) {
    // same double-precision angle as the per-projection path: pos * theta^(-2i / rotary_dim)
    const double inv_freq = pow((double)p.theta, -2.0 * (double)tid / (double)p.rotary_dim);
    double sn, cs;
    sincos((double)p.pos[0] * inv_freq, &sn, &cs);
    sh.rope_cs[tid] = (float)cs;
    sh.rope_sn[tid] = (float)sn;
  }
  if (lane == 0) {
#pragma unroll
    for (int s2 = 0; s2 < kSlots; ++s2) sm100::mbar_init(&ring.bars[s2], 1);
    sm100::mbar_fence_init();
  }
  __syncthreads();
  const bool start_ok = sh.abort == 0u;

  Ctx c;
  c.base = *((const volatile unsigned long long*)p.bar_base);
  c.bar_idx = 0;
  c.mark = 0;
  c.epoch = *((const volatile uint32_t*)p.epoch);
  c.budget_ns = (uint64_t)p.timeout_us * 1000ull;
  const int token = p.token[0];
  const int pos = p.pos[0];
  const int n_layers = p.n_layers;
  bool ok = start_ok;

  if (start_ok) {
    ring_fill(p, ring, warp, lane);   // weights only: in flight before anything else happens
    mark(p, c, 0);
    const bf16* resid = (const bf16*)p.embed + (size_t)token * p.hidden;
    int cur = 0;
    int S = (pos + 15) / 16;          // attention context splits for this position
    S = max(1, min(S, p.max_splits));
    const int n_steps = 7 * n_layers + 1;
    for (int st = 0; st < n_steps && ok; ++st) {
      const int li = st / 7, m = st - li * 7;
      const bool head = li == n_layers;
      const PkDecLayer& L = p.layers[head ? 0 : li];
      const bool full = !head && L.full != 0;
      // ---- what this step consists of ----
      int pre = 0;      // 1 DeltaNet step, 2 attention splits, 3 attention merge
      int stage = 0;    // 1 norm (+ pushed rows of `site`), 2 plain bf16 vector, 3 DeltaNet head norm
      int seg = -1, epi = EPI_BF16, site = 0, push_site = 0;
      bool bar = false;
      const float* gamma = nullptr;
      const bf16* plain_src = nullptr;
      int plain_k = 0;
      bf16* ybf = nullptr;
      if (head) {
        stage = 1; site = 2 * n_layers - 1; gamma = p.final_norm;
        seg = 5 * n_layers; epi = EPI_LOGITS; bar = true;
      } else if (m == 0) {
        stage = 1; site = 2 * li - 1; gamma = L.input_norm;
        seg = 5 * li; epi = EPI_BF16; ybf = (bf16*)p.proj; bar = full;
      } else if (m == 1) {
        if (full) continue;
        seg = 5 * li + 1; epi = EPI_BF16; ybf = (bf16*)p.proj + L.lin[0].N; bar = true;
      } else if (m == 2) {
        pre = full ? 2 : 1; bar = true;
      } else if (m == 3) {
        if (!full) continue;
        pre = 3; bar = true;
      } else if (m == 4) {
        if (full) { stage = 2; plain_src = (const bf16*)p.attn_out; plain_k = p.hq_l * kD; }
        else stage = 3;
        seg = 5 * li + 2; epi = EPI_PUSH; push_site = 2 * li;
      } else if (m == 5) {
        stage = 1; site = 2 * li; gamma = L.post_norm;
        seg = 5 * li + 3; epi = EPI_SWIGLU; ybf = (bf16*)p.mlp_h; bar = true;
      } else {
        stage = 2; plain_src = (const bf16*)p.mlp_h; plain_k = p.inter_l;
        seg = 5 * li + 4; epi = EPI_PUSH; push_site = 2 * li + 1;
      }
      // ---- mixer phase ----
      if (pre == 1) {
        deltanet_phase(p, L, gsm, plan.group_floats);
        mark(p, c, 5);
      } else if (pre == 2) {
        const AttnArgs aa{(const bf16*)p.proj, L.q_norm, L.k_norm, (bf16*)L.kcache, (bf16*)L.vcache, p.attn_ws,
                          sh.rope_cs, sh.rope_sn, p.kv_fp8 ? L.kscale : nullptr, p.kv_fp8 ? L.vscale : nullptr, p.hq_l, p.hkv_l,
                          p.ctx_cap, p.window, p.sink, p.rotary_dim, p.eps};
        attn_split_phase<G>(aa, pos, S, gsm, plan.group_floats);
        mark(p, c, 6);
      } else if (pre == 3) {
        attn_merge_phase(p, S);
        mark(p, c, 7);
      }
      // ---- activation staging ----
      if (stage == 1) {
        ring_window(p, ring, warp, lane);     // the wait for the pushed words is a boundary too
        const bool has_parts = site >= 0;
        const uint2* parts = has_parts ? p.slot[site & 1][p.rank] : nullptr;
        bf16* hout = has_parts ? (bf16*)p.hidden_buf[cur] : nullptr;
        ok = stage_norm(p, c, sh, xs, scratch, resid, parts, has_parts ? p.world : 0, site, hout, gamma,
                        head ? (bf16*)p.norm_out : nullptr);
        if (has_parts) {
          resid = (const bf16*)p.hidden_buf[cur];
          cur ^= 1;
        }
        mark(p, c, 1);
        if (!ok) break;
      } else if (stage == 2) {
        stage_plain(sh, xs, plain_src, plain_k);
        mark(p, c, 8);
      } else if (stage == 3) {
        conv_shift(p, L);
        stage_headnorm(p, sh, xs, scratch, p.o_raw, (const bf16*)p.proj + 2 * p.kh_l * kD + p.vh_l * kD, L.lin_norm);
        mark(p, c, 9);
      }
      // ---- weight streaming ----
      if (seg >= 0) {
        const EpiArgs e{epi, ybf, p.logits, push_site, c.epoch * p.sites_per_epoch + (uint32_t)push_site + 1u};
        run_segment(p, sh, ring, seg, xs, s_acc, e);
        mark(p, c, head ? 20 : 10 + (seg - 5 * li));
      }
      if (bar) {
        ring_window(p, ring, warp, lane);
        ok = bar_grid(p, c, sh);
        mark(p, c, 3);
      }
    }
    if (ok && blockIdx.x == 0) {
      // merge the blocks' candidates (lowest token id on ties)
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int i = tid; i < (int)gridDim.x; i += kThreads) {
        const float v = __ldcg(p.cand_val + i);
        const int id = __ldcg(p.cand_idx + i);
        if (v > best || (v == best && id < bi)) {
          best = v;
          bi = id;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
          best = ov;
          bi = oi;
        }
      }
      if (lane == 0) {
        sh.cand_v[warp] = best;
        sh.cand_i[warp] = bi;
      }
      __syncthreads();
      if (tid == 0) {
        for (int w = 1; w < kWarps; ++w) {
          const float ov = sh.cand_v[w];
          const int oi = sh.cand_i[w];
          if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
          }
        }
        bool good = true;
        if (p.world > 1) {
          // sampler exchange: {logit, token} of every rank through peer memory
          const uint32_t seq = c.epoch * p.sites_per_epoch + (uint32_t)(2 * n_layers) + 1u;
          // rows of 32 entries per rank; entry 31 of the index row carries this rank's status word, so that a rank
          // whose wait ran out earlier in the step takes the others with it
          const int my_status = (int)*((volatile uint32_t*)p.status);
          for (int r = 0; r < p.world; ++r) {
            p.cand_val_peer[r][p.rank * 32] = best;
            p.cand_idx_peer[r][p.rank * 32] = bi;
            p.cand_idx_peer[r][p.rank * 32 + 31] = my_status;
          }
          publish_seq(p.cand_flag, p.world, p.rank, seq);
          const uint64_t t0 = global_timer_ns();
          uint32_t iter = 0;
          while (!all_reached(p.cand_flag[p.rank], p.world, seq)) {
            if (wait_failed(p, c, t0, iter)) {
              atomicCAS(p.status, 0u, PK_COMM_TIMEOUT);
              good = false;
              break;
            }
          }
          __threadfence_system();
          if (good) {
            best = -INFINITY;
            bi = 0x7fffffff;
            for (int r = 0; r < p.world; ++r) {
              if (__ldcg(p.cand_idx_peer[p.rank] + r * 32 + 31) != 0) atomicCAS(p.status, 0u, PK_COMM_PEER_FAILED);
              const float v = __ldcg(p.cand_val_peer[p.rank] + r * 32);
              const int id = __ldcg(p.cand_idx_peer[p.rank] + r * 32);
              if (v > best || (v == best && id < bi)) {
                best = v;
                bi = id;
              }
            }
          }
        }
        if (good) {
          p.next_tok[0] = bi;
          const int cnt = *p.out_counter;
          if (cnt < p.out_cap) p.out_tokens[cnt] = bi;
          *p.out_counter = cnt + 1;
          p.pos[0] = pos + 1;
        }
      }
    }
  }
  // ---- drain: copies still in flight must land before the block's shared memory is released ----
  while (ring.ck < ring.pk) {
    const int slot = (int)(ring.ck % kSlots);
    uint32_t spins = 0;
    while (!sm100::mbar_try_wait(&ring.bars[slot], (ring.ck / kSlots) & 1u)) {
      if (++spins > sm100::kSpinLimit) break;
    }
    ++ring.ck;
  }
}

__global__ void decode_prepare_kernel(uint32_t* epoch, const int* next_tok, int* token, const unsigned long long* bar_count,
                                      unsigned long long* bar_base) {
  *epoch += 1u;
  token[0] = next_tok[0];
  *bar_base = *bar_count;
}

bool make_plan(const PkDecParams& p, int grid, Plan& pl) {
  if (grid < 1 || p.hidden < 16 || (p.hidden & 15) || (p.max_k & 15) || p.max_k < p.hidden) return false;
  if (p.hkv_l > 0 && p.hq_l % p.hkv_l != 0) return false;
  const int G = p.hkv_l > 0 ? p.hq_l / p.hkv_l : 1;
  if (!(G == 1 || G == 2 || G == 4 || G == 5 || G == 8)) return false;
  if (p.kh_l > 0 && (p.vh_l % p.kh_l) != 0) return false;
  const size_t xs_bytes = ((size_t)((p.max_k + 511) & ~511)) * 2;
  const size_t scratch_floats = (size_t)(p.hidden > p.vh_l * kD ? p.hidden : p.vh_l * kD);
  if (p.rotary_dim > 128 || (p.rotary_dim & 1)) return false;
  const size_t attn_floats = 296 + (size_t)G * kD + 8 * G + (size_t)4 * G * kD;
  const size_t group_floats = (attn_floats > 320 ? attn_floats : 320) + 8;
  size_t region = xs_bytes + scratch_floats * 4;
  if (region < group_floats * 4 * kGroups) region = group_floats * 4 * kGroups;
  region = (region + 127) & ~(size_t)127;
  const int pairs = (((p.max_rows + 1) / 2) + grid - 1) / grid + 2;
  size_t off = region;
  pl.off_scratch = (int)xs_bytes;
  pl.off_acc = (int)off;
  off += (size_t)pairs * 2 * sizeof(float);
  off = (off + 127) & ~(size_t)127;
  pl.off_ring = (int)off;
  off += (size_t)kWarps * kSlots * kSlotBytes;
  pl.off_bar = (int)off;
  off += (size_t)kWarps * kSlots * sizeof(uint64_t);
  pl.group_floats = (int)group_floats;
  pl.total = (int)off;
  return off + 2048 <= (size_t)kSmemMax;
}

}  // namespace

PK_API int pk_decode_persistent_prepare(uint32_t* epoch, const int* next_tok, int* token, const unsigned long long* bar_count,
                                        unsigned long long* bar_base, cudaStream_t stream) {
  PK_LAUNCH(decode_prepare_kernel, dim3(1), dim3(1), 0, stream, epoch, next_tok, token, bar_count, bar_base);
  return PK_OK;
}

PK_API size_t pk_decode_persistent_smem(const PkDecParams* params, int grid) {
  Plan pl;
  if (params == nullptr || !make_plan(*params, grid, pl)) return 0;
  return (size_t)pl.total;
}

PK_API int pk_decode_persistent_step(const PkDecParams* params, int grid, cudaStream_t stream) {
  if (params == nullptr) return PK_ERR_BAD_ARG;
  Plan pl;
  if (!make_plan(*params, grid, pl)) return PK_ERR_UNSUPPORTED;
  const int G = params->hkv_l > 0 ? params->hq_l / params->hkv_l : 1;
  void (*kernel)(const PkDecParams, const Plan) = nullptr;
  switch (G) {
    case 1: kernel = decode_persistent_kernel<1>; break;
    case 2: kernel = decode_persistent_kernel<2>; break;
    case 4: kernel = decode_persistent_kernel<4>; break;
    case 5: kernel = decode_persistent_kernel<5>; break;
    case 8: kernel = decode_persistent_kernel<8>; break;
    default: return PK_ERR_UNSUPPORTED;
  }
  // the attribute belongs to the current device; setting it again is cheap and legal during capture
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.total);
  if (e != cudaSuccess) {
    pk_set_last_cuda_error((int)e);
    return PK_ERR_CUDA;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)pl.total;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // every block resident at once, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kernel, *params, pl);
  if (e != cudaSuccess) {
    pk_set_last_cuda_error((int)e);
    return PK_ERR_CUDA;
  }
  return PK_OK;
}

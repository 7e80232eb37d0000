// Persistent FP8 GEMM on the 5th-generation tensor cores, with the weights read as they are stored:
// C[M,N] = A[M,K] * W[N,K]^T, W in E4M3 codes with one fp32 scale per 128 x 128 block, A quantised to E4M3 per
// (row, 128-wide k block). No bf16 copy of the weights exists anywhere: the raw code bytes go from HBM to shared
// memory by TMA and into tcgen05.mma kind::f8f6f4 from there.
//
// Block scales do not commute with the sum over k, so every 128-wide k block is its own MMA group into a fresh TMEM
// accumulator (two of them, used in turn); the epilogue warps pull each finished block out of TMEM, multiply it by
// a_scale[row, kb] * w_scale[n block, kb] and add it to fp32 accumulators that live in registers for the whole tile.
// While they fold block kb the MMA warp is already running block kb + 1 in the other accumulator.
//
// Activation precision. One E4M3 term per activation keeps 4 significant bits. With TERMS = 2 the activation is
// the sum of two E4M3 terms (the code of x / s and the code of the rounding residue), about 8 significant bits like the
// bf16 it came from; both terms run against the same weight tile into the same accumulator, so the weight bytes
// still cross HBM and L2 once. The tensor-core time of two FP8 terms equals that of one bf16 GEMM; what is saved is
// half of the weight traffic and all of the expanded copy.
//
//   warp 0       TMA producer (per stage: TERMS A tiles 128 x 128 B and two W tiles 128 x 128 B, 128-byte swizzle,
//                no multicast)
//   warp 1       MMA issuer (tcgen05.mma kind::f8f6f4, M 128, N 256, K 32; 4 x TERMS per k block)
//   warps 2-17   scale-and-add of every k block, then the tile's epilogue (bf16 / residual add / SiLU(gate)*up /
//                fp32 / fp32 rows pushed into the owner rank's slot)
//
// Every wait is bounded (status word + CTA-wide abort flag), as in gemm_bf16.cu.
//
// Measured on B200 (M = 2048, N = 34816, K = 5120, SwiGLU epilogue): 1.57 PFLOP/s with one term, 1.15 with two (counting
// the product once), against 1.48 for the bf16 kernel on bf16 copies and 2.9 for the library's per-tensor-scaled FP8 GEMM.
// The same loop without the per-block hand-over of the accumulator streams at 2.4 (one term): the four-stage ring is
// bound by the latency of the tile loads, so every wait between "tile landed" and "stage released" lowers the bytes in
// flight. Tried and slower: one MMA group per 128-column half (N = 128 instructions re-read the A tile and run into
// the shared-memory operand bandwidth), one polling lane per warp, suspend-time hints, sleeping between polls.
//
// Reference counterpart: cpp_engine/cuda/qwen_half_ops.cu:379-583 (64 x 64 tiles, weights decoded to fp32 through a
// table, SIMT multiply-add).
#include <cstdlib>
#include <mutex>

#include <cuda_fp8.h>

#include "../common/pk_comm.cuh"
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;
using namespace pk::sm100;

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kABytes = BM * BK;          // 16 KB per term
constexpr int kBBytes = BN * BK;          // 32 KB
constexpr int kEpiWarps = 16;
constexpr int kThreads = 64 + kEpiWarps * 32;
constexpr uint32_t kTmemCols = 512;       // two accumulators of 256 columns

enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_F32 = 3, EPI_PUSH = 4, EPI_SCORE = 5 };

struct Params {
  int M, N, K, epi;
  bf16* C;
  float* Cf;
  const bf16* resid;
  const float* head_w;     // EPI_SCORE: weight of each of the 128 query heads
  int ldc;
  int tiles_m, tiles_n;
  int m_pad;               // rows of one term plane in the A tensor map
  const float* a_scale;    // [K / 128][a_ld]
  int a_ld;
  const float* w_scale;    // [ceil(N / 128)][w_ld]
  int w_ld;
  uint32_t* status;
  PkPush push;
  // stream-K: see gemm_bf16.cu
  int streamk;
  float* ws;
  uint32_t* flags;
  uint32_t seq;
  uint32_t timeout_us;
};

struct Seg {
  int tile, kb0, kb1;
};

// Same schedule as the bf16 kernel: CTA c works on m-tile c % tiles_m; whole tiles round-robin, or (stream-K) the
// k blocks of all column blocks laid end to end and cut into one contiguous range per group of tiles_m CTAs.
struct WorkIter {
  int num_kb, num_tiles, streamk, tiles_m, tm;
  long long pos, end;
  int t, stride;
  __device__ WorkIter(const Params& p, int nkb) : num_kb(nkb), num_tiles(p.tiles_m * p.tiles_n), streamk(p.streamk), tiles_m(p.tiles_m) {
    const int groups = gridDim.x / p.tiles_m, g = blockIdx.x / p.tiles_m;
    tm = blockIdx.x % p.tiles_m;
    const long long total = (long long)p.tiles_n * num_kb;
    pos = streamk ? total * g / groups : 0;
    end = streamk ? total * (g + 1) / groups : 0;
    t = blockIdx.x;
    stride = gridDim.x;
  }
  __device__ bool next(Seg& s) {
    if (!streamk) {
      if (t >= num_tiles) return false;
      s.tile = t;
      s.kb0 = 0;
      s.kb1 = num_kb;
      t += stride;
      return true;
    }
    if (pos >= end) return false;
    const int tn = (int)(pos / num_kb);
    s.tile = tn * tiles_m + tm;
    s.kb0 = (int)(pos - (long long)tn * num_kb);
    const long long left = end - pos;
    s.kb1 = (int)(left < (long long)(num_kb - s.kb0) ? s.kb0 + left : num_kb);
    pos += s.kb1 - s.kb0;
    return true;
  }
};

template <int TERMS>
struct __align__(1024) Smem {
  static constexpr int kStages = TERMS == 1 ? 4 : 3;
  uint8_t a[kStages][TERMS * kABytes];
  uint8_t b[kStages][kBBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  uint32_t part_done;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// First weight row of the two 128-row halves of tile column block `tn`.
__device__ __forceinline__ void weight_rows(const Params& p, int tn, int& r0, int& r1) {
  if (p.epi == EPI_SWIGLU) {
    r0 = tn * 128;
    r1 = (p.N >> 1) + tn * 128;
  } else {
    r0 = tn * BN;
    r1 = tn * BN + 128;
  }
}

// 32 consecutive output columns of row m, starting at column n (not SwiGLU).
__device__ __forceinline__ void emit32(const Params& p, int m, int n, const float (&r)[32]) {
  if (n >= p.N) return;
  if (p.epi == EPI_F32) {
    float* dst = p.Cf + (size_t)m * p.ldc + n;
    if (n + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
      for (int v = 0; v < 8; ++v) *reinterpret_cast<float4*>(dst + v * 4) = make_float4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n + i < p.N) dst[i] = r[i];
    }
  } else if (p.epi == EPI_PUSH) {
    // rows_per_rank > 0: reduce-scatter, the row goes to its owner only
    const int rpr = p.push.rows_per_rank;
    const int owner = rpr > 0 ? m / rpr : 0;
    const size_t off = rpr > 0 ? ((size_t)p.push.rank * rpr + (m - owner * rpr)) * p.ldc + n : ((size_t)p.push.rank * p.M + m) * p.ldc + n;
    const int pr_lo = rpr > 0 ? owner : 0, pr_hi = rpr > 0 ? owner + 1 : p.push.world;
    for (int pr = pr_lo; pr < pr_hi; ++pr) {
      float* dst = p.push.dst[pr] + off;
      if (n + 32 <= p.N) {
#pragma unroll
        for (int v = 0; v < 8; ++v) *reinterpret_cast<float4*>(dst + v * 4) = make_float4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (n + i < p.N) dst[i] = r[i];
      }
    }
  } else {
    bf16* dst = p.C + (size_t)m * p.ldc + n;
    const bf16* rs = p.epi == EPI_RESID ? p.resid + (size_t)m * p.ldc + n : nullptr;
    if (n + 32 <= p.N) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = r[v * 8 + e];
        if (rs) {
          const uint4 rr = *reinterpret_cast<const uint4*>(rs + v * 8);
          const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            f[2 * e] += __uint_as_float(w[e] << 16);
            f[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n + i < p.N) dst[i] = __float2bfloat16(r[i] + (rs ? __bfloat162float(rs[i]) : 0.f));
    }
  }
}

template <int TERMS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Params p) {
  using SmemT = Smem<TERMS>;
  constexpr int kStages = SmemT::kStages;
  extern __shared__ uint8_t smem_raw[];
  SmemT& sm = *reinterpret_cast<SmemT*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.acc_full[b], 1);
      mbar_init(&sm.acc_empty[b], kEpiWarps);
    }
    sm.abort_flag = 0;
    sm.part_done = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      uint32_t it = 0, issued = 0;
      WorkIter work(p, num_kb);
      Seg sg;
      while (!sm.abort_flag && work.next(sg)) {
        const int tm = sg.tile % p.tiles_m, tn = sg.tile / p.tiles_m;
        int r0, r1;
        weight_rows(p, tn, r0, r1);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&sm.empty[s], ((it / kStages) & 1) ^ 1, &sm.abort_flag, p.status, 31)) break;
          mbar_arrive_expect_tx(&sm.full[s], TERMS * kABytes + kBBytes);
#pragma unroll
          for (int t = 0; t < TERMS; ++t) tma_load_2d(sm.a[s] + t * kABytes, &tmap_a, &sm.full[s], kb * BK, t * p.m_pad + tm * BM);
          tma_load_2d(sm.b[s], &tmap_w, &sm.full[s], kb * BK, r0);
          tma_load_2d(sm.b[s] + kBBytes / 2, &tmap_w, &sm.full[s], kb * BK, r1);
          issued = it + 1;
        }
      }
      if (sm.abort_flag) {
        // Gave up: let the copies already in flight land before the CTA exits.
        for (uint32_t j = issued > (uint32_t)kStages ? issued - kStages : 0; j < issued; ++j) {
          const int s = j % kStages;
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(&sm.full[s], (j / kStages) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(0, 0, BM, BN);   // E4M3 x E4M3, fp32 accumulate
      uint32_t it = 0;
      WorkIter work(p, num_kb);
      Seg sg;
      bool ok = true;
      while (ok && !sm.abort_flag && work.next(sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % kStages;
          const int buf = it & 1;
          // the fold of the k block that used this accumulator two blocks ago must have read it (passes at once at first)
          if (!mbar_wait(&sm.acc_empty[buf], ((it >> 1) & 1) ^ 1, &sm.abort_flag, p.status, 32)) { ok = false; break; }
          if (!mbar_wait(&sm.full[s], (it / kStages) & 1, &sm.abort_flag, p.status, 33)) { ok = false; break; }
          tc_fence_after();
          const uint32_t tmem_acc = tmem_base + (uint32_t)buf * BN;
          const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
          for (int t = 0; t < TERMS; ++t)
#pragma unroll
            for (int k = 0; k < BK / 32; ++k)
              umma_f8f6f4(tmem_acc, smem_desc_k_sw128(a_addr + t * kABytes + k * 32), smem_desc_k_sw128(b_addr + k * 32), idesc, (t > 0 || k > 0) ? 1u : 0u);
          umma_commit(&sm.empty[s]);
          umma_commit(&sm.acc_full[buf]);
        }
      }
    }
  } else {
    // ---------------- per-block fold, then the tile's epilogue ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int cq = (warp - 2) >> 2;         // columns cq * 32 .. + 32 of both 128-column halves
    uint32_t it = 0;
    WorkIter work(p, num_kb);
    Seg sg;
    bool ok = true;
    while (ok && work.next(sg)) {
      const int tm = sg.tile % p.tiles_m, tn = sg.tile / p.tiles_m;
      int r0, r1;
      weight_rows(p, tn, r0, r1);
      const int row_in_tile = q * 32 + lane;
      const int m = tm * BM + row_in_tile;
      const bool row_ok = m < p.M;
      const float* as_ptr = p.a_scale + (row_ok ? m : p.M - 1);
      const int nb_last = (p.N - 1) >> 7;
      const float* ws0_ptr = p.w_scale + (size_t)min(r0 >> 7, nb_last) * p.w_ld;
      const float* ws1_ptr = p.w_scale + (size_t)min(r1 >> 7, nb_last) * p.w_ld;
      float acc0[32], acc1[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc0[i] = acc1[i] = 0.f;
      float as = __ldg(as_ptr + (size_t)sg.kb0 * p.a_ld), w0 = __ldg(ws0_ptr + sg.kb0), w1 = __ldg(ws1_ptr + sg.kb0);
      for (int kb = sg.kb0; kb < sg.kb1 && ok; ++kb, ++it) {
        const int buf = it & 1;
        const float s0 = as * w0, s1 = as * w1;
        if (kb + 1 < sg.kb1) {   // next block's scales, in flight during this block's wait
          as = __ldg(as_ptr + (size_t)(kb + 1) * p.a_ld);
          w0 = __ldg(ws0_ptr + kb + 1);
          w1 = __ldg(ws1_ptr + kb + 1);
        }
        if (!mbar_wait(&sm.acc_full[buf], (it >> 1) & 1, &sm.abort_flag, p.status, 34)) { ok = false; break; }
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(q * 32) << 16) + cq * 32;
        uint32_t r[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tmem_ld_32x16(lane_addr + h * 128 + c * 16, r);
            tmem_ld_wait();
            if (h == 1 && c == 1) {
              // the whole accumulator has been read: hand it back to the MMA warp before the last of the arithmetic
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
            }
            if (h == 0) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc0[c * 16 + i] = fmaf(__uint_as_float(r[i]), s0, acc0[c * 16 + i]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc1[c * 16 + i] = fmaf(__uint_as_float(r[i]), s1, acc1[c * 16 + i]);
            }
          }
        }
      }
      if (!ok) break;

      if (sg.kb0 > 0) {
        // Not the owner of this tile: park the fp32 partial in this CTA's workspace slot and publish it.
        float* dst = p.ws + ((size_t)blockIdx.x * BM + row_in_tile) * BN + cq * 32;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          *reinterpret_cast<float4*>(dst + v * 4) = make_float4(acc0[v * 4], acc0[v * 4 + 1], acc0[v * 4 + 2], acc0[v * 4 + 3]);
          *reinterpret_cast<float4*>(dst + 128 + v * 4) = make_float4(acc1[v * 4], acc1[v * 4 + 1], acc1[v * 4 + 2], acc1[v * 4 + 3]);
        }
        __threadfence();
        __syncwarp();
        if (lane == 0 && atomicAdd(&sm.part_done, 1u) == (uint32_t)kEpiWarps - 1u) {
          __threadfence();
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + blockIdx.x), "r"(p.seq) : "memory");
        }
        continue;
      }
      // Owner of a tile that other CTAs finish: their partials were computed first thing in their run.
      if (sg.kb1 < num_kb) {
        int n_parts = 0;
        const int groups = gridDim.x / p.tiles_m, g = blockIdx.x / p.tiles_m;
        const long long total = (long long)p.tiles_n * num_kb, block_end = (long long)(sg.tile / p.tiles_m + 1) * num_kb;
        for (int j = g + 1; j < groups && total * j / groups < block_end; ++j) ++n_parts;
        bool got = true;
        if (lane == 0) {
          const uint64_t t0 = global_timer_ns(), budget = (uint64_t)p.timeout_us * 1000ull;
          for (int j = 1; j <= n_parts && got; ++j) {
            uint32_t v;
            do {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flags + blockIdx.x + j * p.tiles_m) : "memory");
              if (v != p.seq && global_timer_ns() - t0 > budget) {
                got = false;
                sm.abort_flag = 1u;
                if (p.status) atomicCAS(p.status, 0u, 35u);
                break;
              }
            } while (v != p.seq);
          }
        }
        got = __shfl_sync(0xffffffffu, (int)got, 0) != 0;
        if (!got) n_parts = 0;
        const float* part0 = p.ws + ((size_t)(blockIdx.x + p.tiles_m) * BM + row_in_tile) * BN + cq * 32;
        for (int j = 0; j < n_parts; ++j) {
          const float* src = part0 + (size_t)j * p.tiles_m * BM * BN;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 x = __ldcg(reinterpret_cast<const float4*>(src + v * 4));
            const float4 y = __ldcg(reinterpret_cast<const float4*>(src + 128 + v * 4));
            acc0[v * 4] += x.x; acc0[v * 4 + 1] += x.y; acc0[v * 4 + 2] += x.z; acc0[v * 4 + 3] += x.w;
            acc1[v * 4] += y.x; acc1[v * 4 + 1] += y.y; acc1[v * 4 + 2] += y.z; acc1[v * 4 + 3] += y.w;
          }
        }
      }
      if (!row_ok) continue;
      if (p.epi == EPI_SWIGLU) {
        const int half_n = p.N >> 1;
        const int j0 = tn * 128 + cq * 32;
        bf16* dst = p.C + (size_t)m * p.ldc + j0;
        if (j0 + 32 <= half_n) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = v * 8 + e * 2;
              o[e] = pack2(silu(acc0[i]) * acc1[i], silu(acc0[i + 1]) * acc1[i + 1]);
            }
            *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (j0 + i < half_n) dst[i] = __float2bfloat16(silu(acc0[i]) * acc1[i]);
        }
      } else if (p.epi == EPI_SCORE) {
        // Chunk scorer: column h holds q_hi[h] . k and column 128 + h holds q_lo[h] . k; this thread's share of
        // sum_h relu(q[h] . k) * w[h] goes to partial[cq][row] (four partials per row, added by the caller's next kernel).
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) part = fmaf(fmaxf(acc0[i] + acc1[i], 0.f), __ldg(p.head_w + cq * 32 + i), part);
        p.Cf[(size_t)cq * p.ldc + m] = part;
      } else {
        emit32(p, m, tn * BN + cq * 32, acc0);
        emit32(p, m, tn * BN + 128 + cq * 32, acc1);
      }
    }
    if (p.epi == EPI_PUSH) __threadfence_system();
  }

  tc_fence_before();
  __syncthreads();
  if (p.epi == EPI_PUSH && threadIdx.x == 0) publish_after_block_sync(p.push);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// One warp per (row, 128-wide k block): amax, scale = amax / 448, E4M3 code of x / scale, and (two terms) the code of
// the rounding residue. Scales are stored k-block-major so that the GEMM's fold reads them coalesced over rows.
__global__ void __launch_bounds__(256)
quant_act_fp8_kernel(const bf16* __restrict__ x, int ldx, int M, int K, int terms, uint8_t* __restrict__ q, int m_pad, float* __restrict__ scale_t,
                     int s_ld) {
  const int lane = threadIdx.x & 31;
  const int nkb = K >> 7;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)M * nkb) return;
  const int m = (int)(unit / nkb), kb = (int)(unit % nkb);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)m * ldx + kb * 128 + lane * 4);
  float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / s;
  uint32_t hi = 0, lo = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float y = v[i] * inv;
    const __nv_fp8_storage_t c = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
    hi |= (uint32_t)c << (8 * i);
    const float back = __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));
    lo |= (uint32_t)__nv_cvt_float_to_fp8(y - back, __NV_SATFINITE, __NV_E4M3) << (8 * i);
  }
  const size_t off = (size_t)m * K + kb * 128 + lane * 4;
  *reinterpret_cast<uint32_t*>(q + off) = hi;
  if (terms > 1) *reinterpret_cast<uint32_t*>(q + (size_t)m_pad * K + off) = lo;
  if (lane == 0) scale_t[(size_t)kb * s_ld + m] = s;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)sym;
  }
  return fn;
}

struct StreamKBuffers {
  float* ws = nullptr;
  uint32_t* flags = nullptr;
  uint32_t seq = 0;
  int ctas = 0;
};

StreamKBuffers* streamk_buffers(int ctas) {
  static StreamKBuffers per_device[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  StreamKBuffers& b = per_device[dev];
  if (b.ws == nullptr || b.ctas < ctas) {
    if (b.ws) cudaFree(b.ws);
    if (b.flags) cudaFree(b.flags);
    b = StreamKBuffers();
    if (cudaMalloc(&b.ws, (size_t)ctas * BM * BN * sizeof(float)) != cudaSuccess) return nullptr;
    if (cudaMalloc(&b.flags, (size_t)ctas * sizeof(uint32_t)) != cudaSuccess || cudaMemset(b.flags, 0, (size_t)ctas * sizeof(uint32_t)) != cudaSuccess) {
      cudaFree(b.ws);
      b = StreamKBuffers();
      return nullptr;
    }
    b.ctas = ctas;
  }
  return &b;
}

// Stream-K: 0 never (POCKET_GEMM_NO_STREAMK or POCKET_GEMM_STREAMK=0), 2 whenever the schedule allows it
// (POCKET_GEMM_STREAMK=1: tests), 1 only with long k ranges (default).
int streamk_mode() {
  if (getenv("POCKET_GEMM_NO_STREAMK") != nullptr) return 0;
  const char* v = getenv("POCKET_GEMM_STREAMK");
  if (v == nullptr) return 1;
  return v[0] == '1' ? 2 : 0;
}

bool encode_u8_2d(EncodeTiledFn encode, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes) {
  const cuuint64_t gdim[2] = {inner, outer};
  const cuuint64_t gstride[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t estr[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int TERMS>
int launch(const CUtensorMap& ta, const CUtensorMap& tw, const Params& p, int grid, cudaStream_t stream) {
  const size_t smem = sizeof(Smem<TERMS>) + 1024;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel<TERMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  gemm_fp8_kernel<TERMS><<<grid, kThreads, smem, stream>>>(ta, tw, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

}  // namespace

// x [M, K] bf16 (row stride ldx elements, 8-byte aligned rows), K a multiple of 128 -> q [terms][m_pad][K] E4M3 codes and
// scale_t [K / 128][s_ld] fp32 (s_ld >= M). Rows M .. m_pad of q are left as they are (keep them zero).
PK_API int pk_quant_act_fp8(const void* x, int ldx, int M, int K, int terms, void* q, int m_pad, float* scale_t, int s_ld, cudaStream_t stream) {
  if (M < 1 || K < 128 || (K & 127) != 0 || (terms != 1 && terms != 2) || m_pad < M || s_ld < M) return PK_ERR_BAD_ARG;
  if (((uintptr_t)x & 7) != 0 || (ldx & 3) != 0 || ((uintptr_t)q & 3) != 0) return PK_ERR_BAD_ARG;
  const long long units = (long long)M * (K >> 7);
  quant_act_fp8_kernel<<<(unsigned)((units + 7) / 8), 256, 0, stream>>>((const pk::bf16*)x, ldx, M, K, terms, (uint8_t*)q, m_pad, scale_t, s_ld);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Aq: [terms][m_pad][K] E4M3 codes from pk_quant_act_fp8 (m_pad a multiple of 128 when terms == 2), a_scale [K / 128][a_ld];
// W [N, K] E4M3 codes, w_scale [ceil(N / 128)][K / 128] fp32. Epilogues as in pk_gemm_bf16; for SwiGLU (epi 1) W holds
// N / 2 gate rows then N / 2 up rows and N / 2 must be a multiple of 128 (else PK_ERR_UNSUPPORTED).
PK_API int pk_gemm_fp8(const void* Aq, int terms, int m_pad, const float* a_scale, int a_ld, const void* W, const float* w_scale, int M, int N,
                       int K, int epi, void* C, const void* resid, int ldc, uint32_t* status, const PkPush* push, int sm_count,
                       cudaStream_t stream) {
  if (M < 1 || N < 1 || K < BK || (K % BK) != 0 || (terms != 1 && terms != 2)) return PK_ERR_BAD_ARG;
  if (m_pad < M || a_ld < M || (terms == 2 && (m_pad % BM) != 0)) return PK_ERR_BAD_ARG;
  if (((uintptr_t)Aq & 15) != 0 || ((uintptr_t)W & 15) != 0 || a_scale == nullptr || w_scale == nullptr) return PK_ERR_BAD_ARG;
  if (epi < EPI_BF16 || epi > EPI_PUSH) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N & 1) != 0)) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N >> 1) % 128) != 0) return PK_ERR_UNSUPPORTED;
  if ((ldc & 7) != 0 && epi != EPI_F32) return PK_ERR_BAD_ARG;
  if (epi == EPI_PUSH && (push == nullptr || (ldc & 3) != 0)) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;
  CUtensorMap tmap_a, tmap_w;
  if (!encode_u8_2d(encode, &tmap_a, Aq, (uint64_t)K, (uint64_t)(terms == 2 ? 2 * m_pad : M), (uint64_t)K)) return PK_ERR_CUDA;
  if (!encode_u8_2d(encode, &tmap_w, W, (uint64_t)K, (uint64_t)N, (uint64_t)K)) return PK_ERR_CUDA;
  Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.epi = epi;
  p.C = (pk::bf16*)C;
  p.Cf = (float*)C;
  p.resid = (const pk::bf16*)resid;
  p.ldc = ldc;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = epi == EPI_SWIGLU ? ((N >> 1) + 127) / 128 : (N + BN - 1) / BN;
  p.m_pad = m_pad;
  p.a_scale = a_scale;
  p.a_ld = a_ld;
  p.w_scale = w_scale;
  p.w_ld = K / BK;
  p.status = status;
  if (push) p.push = *push;
  const int tiles = p.tiles_m * p.tiles_n;
  const int sms = sm_count > 0 ? sm_count : 148;
  int grid = tiles < sms ? tiles : sms;
  const int num_kb = K / BK;
  const double rounds = (double)tiles / sms;
  const double eff = rounds / (double)((tiles + sms - 1) / sms);
  const int groups = p.tiles_m <= sms ? sms / p.tiles_m : 0;
  if (eff < 0.88 && groups >= 2 && (long long)p.tiles_n * num_kb >= (long long)groups * 4 && streamk_mode() != 0 &&
      (streamk_mode() == 2 || (long long)p.tiles_n * num_kb >= (long long)groups * 48)) {
    StreamKBuffers* b = streamk_buffers(sms);
    if (b != nullptr) {
      p.streamk = 1;
      p.ws = b->ws;
      p.flags = b->flags;
      p.seq = ++b->seq;
      p.timeout_us = 2000000;
      grid = groups * p.tiles_m;
    }
  }
  return terms == 1 ? launch<1>(tmap_a, tmap_w, p, grid, stream) : launch<2>(tmap_a, tmap_w, p, grid, stream);
}

// Chunk scorer of the long-context retriever as one FP8 GEMM: keys [n_chunks, 128] E4M3 codes with one fp32 scale per
// chunk, queries as 256 rows of E4M3 codes (row h: first term of head h, row 128 + h: its rounding residue; unused rows
// zero) whose per-head scale is already folded into head_w[128]. partial [4][ld] receives four partial sums per chunk of
// sum_h relu(q[h] . k) * head_w[h]. ones2: two floats equal to 1 (the weight-scale operand of the GEMM).
PK_API int pk_fp8_chunk_scores(const void* keys, const float* key_scale, int n_chunks, const void* qcodes, const float* head_w, const float* ones2,
                               float* partial, int ld, uint32_t* status, int sm_count, cudaStream_t stream) {
  if (n_chunks < 1 || ld < n_chunks || keys == nullptr || key_scale == nullptr || qcodes == nullptr || head_w == nullptr || ones2 == nullptr ||
      partial == nullptr)
    return PK_ERR_BAD_ARG;
  if (((uintptr_t)keys & 15) != 0 || ((uintptr_t)qcodes & 15) != 0) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;
  CUtensorMap tmap_a, tmap_w;
  if (!encode_u8_2d(encode, &tmap_a, keys, 128, (uint64_t)n_chunks, 128)) return PK_ERR_CUDA;
  if (!encode_u8_2d(encode, &tmap_w, qcodes, 128, 256, 128)) return PK_ERR_CUDA;
  Params p{};
  p.M = n_chunks;
  p.N = 256;
  p.K = 128;
  p.epi = EPI_SCORE;
  p.Cf = partial;
  p.ldc = ld;
  p.head_w = head_w;
  p.tiles_m = (n_chunks + BM - 1) / BM;
  p.tiles_n = 1;
  p.m_pad = n_chunks;
  p.a_scale = key_scale;
  p.a_ld = n_chunks;
  p.w_scale = ones2;
  p.w_ld = 1;
  p.status = status;
  const int sms = sm_count > 0 ? sm_count : 148;
  return launch<1>(tmap_a, tmap_w, p, p.tiles_m < sms ? p.tiles_m : sms, stream);
}

// Persistent bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T with fused epilogues.
//
// Differences from gemm_umma.cu (which keeps the weights quantised and decodes them in shared memory):
//   * 128 x 256 output tiles: per k-step a CTA moves 48 KB into shared memory for 128 x 256 x 64 MMAs
//     (87 flop per byte against 64 for 128 x 128); the 128 x 128 kernel is bound by L2-to-SM bandwidth.
//   * persistent CTAs (one per SM) walk a static list of tiles, m fastest, so that the CTAs working on
//     the same weight columns run at the same time and the weights cross HBM once;
//   * the fp32 accumulator is double buffered in TMEM (2 x 256 columns): the epilogue warps drain tile i
//     while the MMA warp is already accumulating tile i + 1; the TMA ring never stops between tiles.
//
//   warp 0      TMA producer (A tile 128 x 64 and W tile 256 x 64 per stage, 128-byte swizzle, no multicast)
//   warp 1      MMA issuer (tcgen05.mma kind::f16, M 128, N 256, K 16; four per stage)
//   warps 2-9   epilogue (tcgen05.ld, then bf16 store / residual add / SiLU(gate)*up / fp32 / push to peers)
//
// Every mbarrier wait is bounded (status word + CTA-wide abort flag), as in gemm_umma.cu.
#include <cstdlib>
#include <mutex>

#include "../common/pk_comm.cuh"
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;
using namespace pk::sm100;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;      // 16 KB
constexpr int kBBytes = BN * BK * 2;      // 32 KB
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + kEpiWarps * 32;
constexpr uint32_t kTmemCols = 512;       // two accumulators of 256 columns

enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_F32 = 3, EPI_PUSH = 4 };

struct Params {
  int M, N, K, epi;
  bf16* C;
  float* Cf;
  const bf16* resid;
  int ldc;
  int tiles_m, tiles_n;
  uint32_t* status;
  PkPush push;
  // stream-K: the k-steps of all tiles, laid end to end, are cut into one contiguous range per CTA
  int streamk;
  float* ws;            // [gridDim.x][BM][BN] fp32 partial accumulators (each CTA writes at most one)
  uint32_t* flags;      // [gridDim.x] sequence number of the launch whose partial is in ws
  uint32_t seq;
  uint32_t timeout_us;
  // grouped mode (routed experts): rows seg[g] .. seg[g + 1] of A belong to group g, whose weights are rows
  // g * N .. (g + 1) * N of W; m-tiles never cross a group boundary on the output side (rows past the group's end are
  // computed and not stored)
  const int* seg;
  int n_groups;
};

constexpr int kMaxGroups = 512;

// One stretch of k-steps of one tile. A CTA's first segment may start in the middle of a tile (the CTA before it
// owns that tile and adds this partial); its last one may end early (then this CTA owns the tile and adds the
// partials of the CTAs after it, which computed them at the very start of their run).
struct Seg {
  int tile, kb0, kb1;
};

// Stream-K keeps the CTAs that share weight columns in lockstep: CTA c belongs to group c / tiles_m and always works
// on m-tile c % tiles_m; the k-steps of all column blocks, laid end to end, are cut into one contiguous range per
// GROUP, so the tiles_m CTAs of a group read the same weight tiles at the same time (one HBM read, L2 hits for the
// others) exactly as in the whole-tile schedule.
struct WorkIter {
  int num_kb, num_tiles, streamk, tiles_m, tm;
  long long pos, end;     // stream-K: flattened (column block, k-step) of this CTA's group
  int t, stride;          // tile mode
  __device__ WorkIter(const Params& p, int nkb, int tiles_m_) : num_kb(nkb), num_tiles(tiles_m_ * p.tiles_n), streamk(p.streamk), tiles_m(tiles_m_) {
    const int tmd = tiles_m_ > 0 ? tiles_m_ : 1;
    const int groups = gridDim.x / tmd, g = blockIdx.x / tmd;
    tm = blockIdx.x % tmd;
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

struct __align__(1024) Smem {
  uint8_t a[kStages][kABytes];
  uint8_t b[kStages][kBBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  uint32_t part_done;     // epilogue warps that have stored their share of this CTA's partial
  int mt_prefix[kMaxGroups + 1];   // grouped mode: m-tiles before each group
};

// Where tile `tile` reads and writes: column block, first A row, row offset into W, rows that are real.
__device__ __forceinline__ void tile_coords(const Params& p, const Smem& sm, int tile, int tiles_m, int& tn, int& a_row, int& w_off, int& rows) {
  tn = tile / tiles_m;
  const int g = tile - tn * tiles_m;
  if (p.seg == nullptr) {
    a_row = g * BM;
    w_off = 0;
    rows = p.M - a_row;
    return;
  }
  int lo = 0, hi = p.n_groups;   // mt_prefix[lo] <= g < mt_prefix[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sm.mt_prefix[mid] <= g) lo = mid;
    else hi = mid;
  }
  a_row = __ldg(p.seg + lo) + (g - sm.mt_prefix[lo]) * BM;
  rows = __ldg(p.seg + lo + 1) - a_row;
  w_off = lo * p.N;
}

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

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
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
    if (p.seg != nullptr) {
      int run = 0;
      for (int g = 0; g < p.n_groups; ++g) {
        sm.mt_prefix[g] = run;
        run += (p.seg[g + 1] - p.seg[g] + BM - 1) / BM;
      }
      sm.mt_prefix[p.n_groups] = run;
    }
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_base;
  const int tiles_m = p.seg != nullptr ? sm.mt_prefix[p.n_groups] : p.tiles_m;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      uint32_t it = 0, issued = 0;
      WorkIter work(p, num_kb, tiles_m);
      Seg sg;
      while (!sm.abort_flag && work.next(sg)) {
        int tn, a_row, w_off, rows;
        tile_coords(p, sm, sg.tile, tiles_m, tn, a_row, w_off, rows);
        int r0, r1;
        weight_rows(p, tn, r0, r1);
        r0 += w_off;
        r1 += w_off;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&sm.empty[s], ((it / kStages) & 1) ^ 1, &sm.abort_flag, p.status, 21)) break;
          mbar_arrive_expect_tx(&sm.full[s], kABytes + kBBytes);
          tma_load_2d(sm.a[s], &tmap_a, &sm.full[s], kb * BK, a_row);
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
      constexpr uint32_t idesc = umma_idesc(1, 1, BM, BN);
      uint32_t it = 0;
      int local = 0;
      WorkIter work(p, num_kb, tiles_m);
      Seg sg;
      for (; !sm.abort_flag && work.next(sg); ++local) {
        const int buf = local & 1;
        const uint32_t use = (uint32_t)local >> 1;
        // the epilogue must have drained this accumulator (passes at once for its first use)
        if (!mbar_wait(&sm.acc_empty[buf], (use & 1) ^ 1, &sm.abort_flag, p.status, 22)) break;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + (uint32_t)buf * BN;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&sm.full[s], (it / kStages) & 1, &sm.abort_flag, p.status, 23)) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16(tmem_acc, smem_desc_k_sw128(a_addr + k * 32), smem_desc_k_sw128(b_addr + k * 32), idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          umma_commit(&sm.empty[s]);
        }
        umma_commit(&sm.acc_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int ch = (warp - 2) >> 2;         // which half of the tile's columns
    int local = 0;
    WorkIter work(p, num_kb, tiles_m);
    Seg sg;
    for (; work.next(sg); ++local) {
      const int buf = local & 1;
      const uint32_t use = (uint32_t)local >> 1;
      int tn, a_row, w_off, rows;
      tile_coords(p, sm, sg.tile, tiles_m, tn, a_row, w_off, rows);
      if (!mbar_wait(&sm.acc_full[buf], use & 1, &sm.abort_flag, p.status, 24)) break;
      tc_fence_after();
      const int m = a_row + q * 32 + lane;
      const bool row_ok = q * 32 + lane < rows;
      const uint32_t lane_addr = tmem_base + (uint32_t)buf * BN + ((uint32_t)(q * 32) << 16);
      const int row_in_tile = q * 32 + lane;
      if (sg.kb0 > 0) {
        // Not the owner of this tile: park the fp32 partial in this CTA's workspace slot and publish it.
        float* dst = p.ws + ((size_t)blockIdx.x * BM + row_in_tile) * BN + ch * 128;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + ch * 128 + cc * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(dst + cc * 32 + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        }
        __threadfence();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&sm.acc_empty[buf]);
          if (atomicAdd(&sm.part_done, 1u) == (uint32_t)kEpiWarps - 1u) {
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + blockIdx.x), "r"(p.seq) : "memory");
          }
        }
        continue;
      }
      // Owner of a tile that other CTAs finish: their partials were computed first thing in their run.
      int n_parts = 0;
      if (sg.kb1 < num_kb) {
        const int groups = gridDim.x / p.tiles_m, g = blockIdx.x / p.tiles_m;
        const long long total = (long long)p.tiles_n * num_kb, block_end = (long long)(sg.tile / p.tiles_m + 1) * num_kb;
        for (int j = g + 1; j < groups && total * j / groups < block_end; ++j) ++n_parts;
        bool ok = true;
        if (lane == 0) {
          const uint64_t t0 = global_timer_ns(), budget = (uint64_t)p.timeout_us * 1000ull;
          for (int j = 1; j <= n_parts && ok; ++j) {
            uint32_t v;
            do {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flags + blockIdx.x + j * p.tiles_m) : "memory");
              if (v != p.seq && global_timer_ns() - t0 > budget) {
                ok = false;
                sm.abort_flag = 1u;
                if (p.status) atomicCAS(p.status, 0u, 25u);
                break;
              }
            } while (v != p.seq);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) n_parts = 0;
      }
      const float* part0 = p.ws + ((size_t)(blockIdx.x + p.tiles_m) * BM + row_in_tile) * BN;
      // adds the parked partials of the following CTAs to one 32-column chunk
      auto add_parts = [&](int c0, uint32_t (&r)[32]) {
        for (int j = 0; j < n_parts; ++j) {
          const float* src = part0 + (size_t)j * p.tiles_m * BM * BN + c0;
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 x = __ldcg(reinterpret_cast<const float4*>(src + v * 4));
            r[v * 4] = __float_as_uint(__uint_as_float(r[v * 4]) + x.x);
            r[v * 4 + 1] = __float_as_uint(__uint_as_float(r[v * 4 + 1]) + x.y);
            r[v * 4 + 2] = __float_as_uint(__uint_as_float(r[v * 4 + 2]) + x.z);
            r[v * 4 + 3] = __float_as_uint(__uint_as_float(r[v * 4 + 3]) + x.w);
          }
        }
      };
      if (p.epi == EPI_SWIGLU) {
        const int half_n = p.N >> 1;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          const int c0 = ch * 64 + cc * 32;                 // column inside the gate half
          uint32_t g[32], u[32];
          tmem_ld_32x32(lane_addr + c0, g);
          tmem_ld_32x32(lane_addr + 128 + c0, u);
          tmem_ld_wait();
          if (n_parts) {
            add_parts(c0, g);
            add_parts(128 + c0, u);
          }
          if (!row_ok) continue;
          const int j0 = tn * 128 + c0;
          bf16* dst = p.C + (size_t)m * p.ldc + j0;
          if (j0 + 32 <= half_n) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = v * 8 + e * 2;
                o[e] = pack2(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]), silu(__uint_as_float(g[i + 1])) * __uint_as_float(u[i + 1]));
              }
              *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (j0 + i < half_n) dst[i] = __float2bfloat16(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]));
          }
        }
      } else {
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          const int c0 = ch * 128 + cc * 32;
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + c0, r);
          tmem_ld_wait();
          if (n_parts) add_parts(c0, r);
          if (!row_ok) continue;
          const int n = tn * BN + c0;
          if (n >= p.N) continue;
          if (p.epi == EPI_F32) {
            float* dst = p.Cf + (size_t)m * p.ldc + n;
            if (n + 32 <= p.N && (p.ldc & 3) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (n + i < p.N) dst[i] = __uint_as_float(r[i]);
            }
          } else if (p.epi == EPI_PUSH) {
            // rows_per_rank > 0: reduce-scatter, the row goes to its owner only (1 / world of the bytes of push-to-all)
            const int rpr = p.push.rows_per_rank;
            const int owner = rpr > 0 ? m / rpr : 0;
            const size_t off = rpr > 0 ? ((size_t)p.push.rank * rpr + (m - owner * rpr)) * p.ldc + n
                                       : ((size_t)p.push.rank * p.M + m) * p.ldc + n;
            const int pr_lo = rpr > 0 ? owner : 0, pr_hi = rpr > 0 ? owner + 1 : p.push.world;
            for (int pr = pr_lo; pr < pr_hi; ++pr) {
              float* dst = p.push.dst[pr] + off;
              if (n + 32 <= p.N) {
#pragma unroll
                for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
              } else {
                for (int i = 0; i < 32; ++i)
                  if (n + i < p.N) dst[i] = __uint_as_float(r[i]);
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
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
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
              for (int i = 0; i < 32; ++i)
                if (n + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]) + (rs ? __bfloat162float(rs[i]) : 0.f));
            }
          }
        }
      }
      // this warp is done reading the accumulator: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
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

// Per-device stream-K scratch: one fp32 tile and one flag per CTA. Allocated on first use.
struct StreamKBuffers {
  float* ws = nullptr;
  uint32_t* flags = nullptr;
  uint32_t seq = 0;
  int ctas = 0;
};

// Stream-K mode: 0 = never (POCKET_GEMM_NO_STREAMK, or POCKET_GEMM_STREAMK=0), 2 = whenever the schedule allows it
// (POCKET_GEMM_STREAMK=1: tests), 1 = only with long k ranges (default). Measured at M = 512 on B200: K = 12288, N = 5120
// gains 7 % (104 k-steps per CTA group), K = 5120, N = 4096 loses 25 % (35 k-steps per group: the fix-up dominates).
static int streamk_mode() {
  if (getenv("POCKET_GEMM_NO_STREAMK") != nullptr) return 0;
  const char* v = getenv("POCKET_GEMM_STREAMK");
  if (v == nullptr) return 1;
  return v[0] == '1' ? 2 : 0;
}


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

bool encode_bf16_2d(EncodeTiledFn encode, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                    uint32_t box_inner, uint32_t box_outer) {
  const cuuint64_t gdim[2] = {inner, outer};
  const cuuint64_t gstride[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Grouped form for routed experts: A [R, K] bf16 rows sorted by group, seg [n_groups + 1] (device) the first row of every
// group, W [n_groups * N, K] bf16 (group g's [N, K] matrix at row g * N). C rows are A's rows. Epilogues 0 (bf16),
// 1 (SwiGLU: every group's matrix holds N / 2 gate rows then N / 2 up rows) and 3 (fp32). One persistent launch walks
// every (group, row tile, column block) that has rows; the tile list is derived from seg on the device, so the host
// never reads the routing.
PK_API int pk_gemm_bf16_grouped(const void* A, int lda, const void* W, const int* seg, int n_groups, int R, int N, int K, int epi, void* C, int ldc,
                                uint32_t* status, int sm_count, cudaStream_t stream) {
  if (R < 1 || N < 1 || K < BK || (K % BK) != 0 || seg == nullptr || n_groups < 1 || n_groups > kMaxGroups) return PK_ERR_BAD_ARG;
  if (((uintptr_t)A & 15) != 0 || ((size_t)lda * 2) % 16 != 0 || ((uintptr_t)W & 15) != 0) return PK_ERR_BAD_ARG;
  if (epi != EPI_BF16 && epi != EPI_SWIGLU && epi != EPI_F32) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N & 1) != 0)) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N >> 1) % 128) != 0) return PK_ERR_UNSUPPORTED;
  if (epi != EPI_SWIGLU && (N % 128) != 0) return PK_ERR_UNSUPPORTED;      // a column block must not reach into the next group's rows
  if ((ldc & 7) != 0 && epi != EPI_F32) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;
  CUtensorMap tmap_a, tmap_w;
  if (!encode_bf16_2d(encode, &tmap_a, A, (uint64_t)K, (uint64_t)R, (uint64_t)lda * 2, BK, BM)) return PK_ERR_CUDA;
  if (!encode_bf16_2d(encode, &tmap_w, W, (uint64_t)K, (uint64_t)n_groups * N, (uint64_t)K * 2, BK, 128)) return PK_ERR_CUDA;
  Params p{};
  p.M = R;
  p.N = N;
  p.K = K;
  p.epi = epi;
  p.C = (pk::bf16*)C;
  p.Cf = (float*)C;
  p.ldc = ldc;
  p.tiles_m = 0;
  p.tiles_n = epi == EPI_SWIGLU ? ((N >> 1) + 127) / 128 : (N + BN - 1) / BN;
  p.status = status;
  p.seg = seg;
  p.n_groups = n_groups;
  const size_t smem = sizeof(Smem) + 1024;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  gemm_bf16_kernel<<<sm_count > 0 ? sm_count : 148, kThreads, smem, stream>>>(tmap_a, tmap_w, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// A [M, K] bf16 (row stride lda elements), W [N, K] bf16 row-major, K a multiple of 64. Epilogues as in pk_gemm_umma;
// for SwiGLU (epi 1) W holds N/2 gate rows then N/2 up rows and N/2 must be a multiple of 128 (else PK_ERR_UNSUPPORTED).
PK_API int pk_gemm_bf16(const void* A, int lda, const void* W, int M, int N, int K, int epi, void* C, const void* resid, int ldc,
                        uint32_t* status, const PkPush* push, int sm_count, cudaStream_t stream) {
  if (M < 1 || N < 1 || K < BK || (K % BK) != 0) return PK_ERR_BAD_ARG;
  if (((uintptr_t)A & 15) != 0 || ((size_t)lda * 2) % 16 != 0 || ((uintptr_t)W & 15) != 0) return PK_ERR_BAD_ARG;
  if (epi < EPI_BF16 || epi > EPI_PUSH) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N & 1) != 0)) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N >> 1) % 128) != 0) return PK_ERR_UNSUPPORTED;   // the up half of a tile must start on its own row block
  if ((ldc & 7) != 0 && epi != EPI_F32) return PK_ERR_BAD_ARG;
  if (epi == EPI_PUSH && (push == nullptr || (ldc & 3) != 0)) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;
  CUtensorMap tmap_a, tmap_w;
  if (!encode_bf16_2d(encode, &tmap_a, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM)) return PK_ERR_CUDA;
  if (!encode_bf16_2d(encode, &tmap_w, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, 128)) return PK_ERR_CUDA;
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
  p.status = status;
  if (push) p.push = *push;
  const size_t smem = sizeof(Smem) + 1024;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int sms = sm_count > 0 ? sm_count : 148;
  int grid = tiles < sms ? tiles : sms;
  // Stream-K when whole tiles would leave many SMs idle in the last round (or the whole time).
  const int num_kb = K / BK;
  const double rounds = (double)tiles / sms;
  const double eff = rounds / (double)((tiles + sms - 1) / sms);
  p.streamk = 0;
  const int groups = p.tiles_m <= sms ? sms / p.tiles_m : 0;
  if (eff < 0.88 && groups >= 2 && (long long)p.tiles_n * num_kb >= (long long)groups * 8 && streamk_mode() != 0 &&
      (streamk_mode() == 2 || (long long)p.tiles_n * num_kb >= (long long)groups * 96)) {
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
  gemm_bf16_kernel<<<grid, kThreads, smem, stream>>>(tmap_a, tmap_w, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Prefill GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * dequant(W[N,K])^T.
//
//   A    bf16 activations, moved by TMA (2-D tiled, 128-byte swizzle, no multicast) into a
//        5-stage shared-memory ring.
//   W    quantised weights that are NEVER expanded in HBM. The raw FP8 E4M3 tile (128 rows x
//        64 bytes) rides the same TMA ring; two groups of eight decode warps (alternating
//        stages) turn it into the bf16 K-major
//        tile in the 128-byte swizzle the tensor core expects, applying the fp32 scale of
//        its 128x128 block on the way. bf16 weights skip the decode: TMA writes the
//        swizzled tile directly.
//   MMA  one elected thread issues tcgen05.mma (kind::f16, 128x128x16) with the fp32
//        accumulator in TMEM; tcgen05.commit releases ring slots and signals the epilogue.
//   EPI  the decode warps read TMEM with tcgen05.ld and fuse: bf16 store, residual add,
//        SiLU(gate)*up (gate and up rows share a tile), or an fp32 partial store.
//
// Replaces the reference's prefill paths: cpp_engine/cuda/qwen_half_ops.cu:379-583 (SIMT
// tiles with an LUT decode) and cpp_engine/cuda/fp8_ops.cu:142-300 (whole-weight dequant
// to fp16 in HBM followed by cublasGemmEx).
#include "../common/pk_comm.cuh"
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;
using namespace pk::sm100;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 5;
constexpr int kTileBytes = BM * BK * 2;   // 16 KB per bf16 operand tile
constexpr int kRawBytes = BN * BK;        // 8 KB of raw FP8 per stage
constexpr int kDecodeWarps = 8;
constexpr int kDecodeGroups = 2;          // groups alternate ring stages so that decode latency overlaps
constexpr int kThreads = 64 + kDecodeGroups * kDecodeWarps * 32;  // warp0 TMA, warp1 MMA, then decode (+ epilogue) warps
constexpr int kMaxScaleKb = 512;          // K <= 65536 for the shared-memory scale table
constexpr uint32_t kTmemCols = 128;

enum { WFMT_FP8_BLOCK128 = 0, WFMT_BF16 = 1 };
enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_F32 = 3, EPI_PUSH = 4 };

struct GemmParams {
  const float* scale;   // fp8: [ceil(N/128), ceil(K/128)]
  int wfmt;
  int M, N, K;
  int epi;
  bf16* C;              // EPI_BF16 / EPI_RESID: [M, ldc]; EPI_SWIGLU: [M, ldc] with N/2 columns
  float* Cf;            // EPI_F32
  const bf16* resid;    // EPI_RESID: [M, ldc]
  int ldc;
  uint32_t* status;     // device status word, 0 = ok
  PkPush push;          // EPI_PUSH: fp32 partial tile into every rank's slot [world][M][ldc], then a flag
};

struct __align__(1024) SmemLayout {
  uint8_t a[kStages][kTileBytes];
  uint8_t b[kStages][kTileBytes];
  uint8_t raw[kStages][kRawBytes];
  uint64_t full_in[kStages];   // TMA landed (A tile + raw or bf16 weight tile)
  uint64_t full_b[kStages];    // decode warps finished the bf16 weight tile
  uint64_t empty[kStages];     // MMAs that read the stage completed
  uint64_t accum_full;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
  float scale_tab[2][kMaxScaleKb];  // block scales of the tile's two 64-row halves along K
};

// First weight row of each 64-row half of the tile. For SwiGLU the first half holds gate
// rows and the second the matching up rows, so one epilogue thread owns both values.
__device__ __forceinline__ void tile_rows(const GemmParams& p, int n0, int& r0, int& r1) {
  if (p.epi == EPI_SWIGLU) {
    r0 = n0 >> 1;
    r1 = (p.N >> 1) + (n0 >> 1);
  } else {
    r0 = n0;
    r1 = n0 + 64;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // m-tiles vary fastest so that the CTAs sharing a weight tile run together and the
  // weights cross HBM once.
  const int n0 = blockIdx.y * BN, m0 = blockIdx.x * BM;
  const int num_kb = p.K / BK;
  const bool fp8 = p.wfmt == WFMT_FP8_BLOCK128;
  int wr0, wr1;
  tile_rows(p, n0, wr0, wr1);
  // Rows of the second half that do not exist (N edge) must read as zero: TMA fills
  // out-of-range rows with zeros, but a SwiGLU "up" half always starts inside the matrix,
  // so its tail rows are masked in the epilogue instead.

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full_in[s], 1);
      mbar_init(&sm.full_b[s], kDecodeWarps * 32);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.accum_full, 1);
    sm.abort_flag = 0;
    mbar_fence_init();
  }
  if (fp8) {
    // Block scales of this tile along K, one row of the table per 64-row half.
    const int kb_scale = (p.K + 127) >> 7;
    for (int i = threadIdx.x; i < 2 * kb_scale; i += kThreads) {
      const int hfi = i / kb_scale, kk = i % kb_scale;
      const int row = min(hfi == 0 ? wr0 : wr1, p.N - 1);
      sm.scale_tab[hfi][kk] = __ldg(p.scale + (size_t)(row >> 7) * kb_scale + kk);
    }
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = sm.tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      const uint32_t tx = kTileBytes + (fp8 ? kRawBytes : kTileBytes);
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait(&sm.empty[s], ((kb / kStages) & 1) ^ 1, &sm.abort_flag, p.status, 11)) break;
        mbar_arrive_expect_tx(&sm.full_in[s], tx);
        tma_load_2d(sm.a[s], &tmap_a, &sm.full_in[s], kb * BK, m0);
        if (fp8) {
          tma_load_2d(sm.raw[s], &tmap_w, &sm.full_in[s], kb * BK, wr0);
          tma_load_2d(sm.raw[s] + kRawBytes / 2, &tmap_w, &sm.full_in[s], kb * BK, wr1);
        } else {
          tma_load_2d(sm.b[s], &tmap_w, &sm.full_in[s], kb * BK, wr0);
          tma_load_2d(sm.b[s] + kTileBytes / 2, &tmap_w, &sm.full_in[s], kb * BK, wr1);
        }
        issued = kb + 1;
      }
      if (sm.abort_flag) {
        // Gave up: let the copies already in flight land before the CTA exits.
        for (int kb = max(0, issued - kStages); kb < issued; ++kb) {
          const int s = kb % kStages;
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(&sm.full_in[s], (kb / kStages) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1, 1, BM, BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1;
        mbar_wait(&sm.full_in[s], ph, &sm.abort_flag, p.status, 12);
        if (fp8) mbar_wait(&sm.full_b[s], ph, &sm.abort_flag, p.status, 13);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = smem_desc_k_sw128(a_addr + k * 32);
          const uint64_t db = smem_desc_k_sw128(b_addr + k * 32);
          umma_f16(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&sm.empty[s]);
      }
      umma_commit(&sm.accum_full);
    }
  } else {
    // ---------------- weight decode, then epilogue ----------------
    const int grp = (warp - 2) / kDecodeWarps;             // decode group of this warp
    const int t = (threadIdx.x - 64) % (kDecodeWarps * 32);  // 0..255 within the group
    if (fp8) {
      const int r = t >> 1;                // tile row 0..127
      const int hf = t & 1;                // which 32 of the row's 64 K-elements
      const int grow = (r < 64 ? wr0 + r : wr1 + (r - 64));
      const bool row_valid = p.epi == EPI_SWIGLU ? ((n0 >> 1) + (r & 63)) < (p.N >> 1) : grow < p.N;
      const float* stab = sm.scale_tab[r >> 6];
      for (int kb = grp; kb < num_kb; kb += kDecodeGroups) {
        const int s = kb % kStages;
        const float sc = row_valid ? stab[(kb * BK) >> 7] : 0.f;
        mbar_wait(&sm.full_in[s], (kb / kStages) & 1, &sm.abort_flag, p.status, 14);
        const uint4 q0 = *reinterpret_cast<const uint4*>(sm.raw[s] + r * BK + hf * 32);
        const uint4 q1 = *reinterpret_cast<const uint4*>(sm.raw[s] + r * BK + hf * 32 + 16);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t o[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 a = e4m3x2_to_float2((uint16_t)(w[j] & 0xffffu));
          const float2 b = e4m3x2_to_float2((uint16_t)(w[j] >> 16));
          o[2 * j] = pack_bf16(a.x * sc, a.y * sc);
          o[2 * j + 1] = pack_bf16(b.x * sc, b.y * sc);
        }
        uint8_t* rowp = sm.b[s] + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int chunk = hf * 4 + c;    // 16-byte chunk of the 128-byte row
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(&sm.full_b[s]);
      }
    }
    if (grp != 0) goto done;  // the first group also runs the epilogue

    // ---------------- epilogue ----------------
    mbar_wait(&sm.accum_full, 0, &sm.abort_flag, p.status, 15);
    tc_fence_after();
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int ch = (warp - 2) >> 2;         // which half of the columns
    const int m = m0 + q * 32 + lane;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(q * 32) << 16);
    const bool row_ok = m < p.M && !sm.abort_flag;
    if (p.epi == EPI_SWIGLU) {
      const int half_n = p.N >> 1;
      const int j0 = (n0 >> 1) + ch * 32;
      uint32_t g[32], u[32];
      tmem_ld_32x32(lane_addr + ch * 32, g);
      tmem_ld_32x32(lane_addr + 64 + ch * 32, u);
      tmem_ld_wait();
      if (row_ok) {
        bf16* dst = p.C + (size_t)m * p.ldc + j0;
        if (j0 + 32 <= half_n) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = v * 8 + e * 2;
              o[e] = pack_bf16(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]),
                               silu(__uint_as_float(g[i + 1])) * __uint_as_float(u[i + 1]));
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
      for (int cc = 0; cc < 2; ++cc) {
        const int c = ch * 2 + cc;
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        const int n = n0 + c * 32;
        if (p.epi == EPI_F32) {
          float* dst = p.Cf + (size_t)m * p.ldc + n;
          for (int i = 0; i < 32; ++i)
            if (n + i < p.N) dst[i] = __uint_as_float(r[i]);
        } else if (p.epi == EPI_PUSH) {
          // The scatter side of the all-reduce, issued tile by tile from the epilogue: this
          // rank's fp32 partial goes straight into every peer's slot over NVLink.
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
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
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
              *reinterpret_cast<uint4*>(dst + v * 8) =
                  make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            }
          } else {
            for (int i = 0; i < 32; ++i)
              if (n + i < p.N)
                dst[i] = __float2bfloat16(__uint_as_float(r[i]) + (rs ? __bfloat162float(rs[i]) : 0.f));
          }
        }
      }
    }
    if (p.epi == EPI_PUSH) __threadfence_system();
    tc_fence_before();
  }

done:
  __syncthreads();
  if (p.epi == EPI_PUSH && threadIdx.x == 0) publish_after_block_sync(p.push);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = (EncodeTiledFn)sym;
    }
  }
  return fn;
}

bool encode_2d(EncodeTiledFn encode, CUtensorMap* map, CUtensorMapDataType dt, int elem, const void* base,
               uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
               CUtensorMapSwizzle swz) {
  const cuuint64_t gdim[2] = {inner, outer};
  const cuuint64_t gstride[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  (void)elem;
  return encode(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// A: [M, K] bf16 row-major with row stride lda elements (lda*2 bytes a multiple of 16, base
// 16-byte aligned). W: [N, K] row-major, 16-byte aligned base. K must be a multiple of 64.
// For epi == 1 (SwiGLU) W holds N/2 gate rows followed by N/2 up rows and C has N/2 columns.
PK_API int pk_gemm_umma(const void* A, int lda, const void* W, const float* scale, int wfmt, int M, int N,
                        int K, int epi, void* C, const void* resid, int ldc, uint32_t* status,
                        const PkPush* push, cudaStream_t stream) {
  if (M < 1 || N < 1 || K < BK || (K % BK) != 0) return PK_ERR_BAD_ARG;
  if (((uintptr_t)A & 15) != 0 || ((size_t)lda * 2) % 16 != 0 || ((uintptr_t)W & 15) != 0) return PK_ERR_BAD_ARG;
  if (wfmt != WFMT_FP8_BLOCK128 && wfmt != WFMT_BF16) return PK_ERR_UNSUPPORTED;
  if (wfmt == WFMT_FP8_BLOCK128 && scale == nullptr) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N & 1) != 0)) return PK_ERR_BAD_ARG;
  if ((ldc & 7) != 0 && epi != EPI_F32) return PK_ERR_BAD_ARG;
  if (epi == EPI_PUSH && (push == nullptr || (ldc & 3) != 0)) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;

  CUtensorMap tmap_a, tmap_w;
  if (!encode_2d(encode, &tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                 BK, BM, CU_TENSOR_MAP_SWIZZLE_128B))
    return PK_ERR_CUDA;
  const bool ok_w = wfmt == WFMT_FP8_BLOCK128
                        ? encode_2d(encode, &tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, (uint64_t)K, (uint64_t)N,
                                    (uint64_t)K, BK, 64, CU_TENSOR_MAP_SWIZZLE_NONE)
                        : encode_2d(encode, &tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, (uint64_t)K, (uint64_t)N,
                                    (uint64_t)K * 2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok_w) return PK_ERR_CUDA;

  GemmParams p{};
  p.scale = scale;
  p.wfmt = wfmt;
  p.M = M;
  p.N = N;
  p.K = K;
  p.epi = epi;
  p.C = (pk::bf16*)C;
  p.Cf = (float*)C;
  p.resid = (const pk::bf16*)resid;
  p.ldc = ldc;
  p.status = status;
  if (push) p.push = *push;

  const size_t smem = sizeof(SmemLayout) + 1024;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  const dim3 grid((M + BM - 1) / BM, (N + BN - 1) / BN);
  if (grid.y > 65535 || (K + 127) / 128 > kMaxScaleKb) return PK_ERR_UNSUPPORTED;
  gemm_umma_kernel<<<grid, kThreads, smem, stream>>>(tmap_a, tmap_w, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

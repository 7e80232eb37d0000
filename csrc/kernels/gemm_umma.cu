// Prefill GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * dequant(W[N,K])^T.
//
//   A   bf16 activations, moved by TMA (2-D tiled, 128-byte swizzle, no multicast) into a
//       4-stage shared-memory ring.
//   W   quantised weights that are NEVER expanded in HBM: four producer warps read the
//       raw tile (FP8 E4M3 with one fp32 scale per 128x128 block, or plain bf16), decode
//       it in registers and write the bf16 K-major tile into shared memory in the same
//       128-byte swizzle the tensor core expects.
//   MMA one elected thread issues tcgen05.mma (kind::f16, 128x128x16) with the fp32
//       accumulator in TMEM; tcgen05.commit releases ring slots and signals the epilogue.
//   EPI the producer warps read TMEM with tcgen05.ld and fuse: bf16 store, residual add,
//       SiLU(gate)*up (gate and up rows share a tile), or an fp32 partial store.
//
// Replaces the reference's prefill paths: cpp_engine/cuda/qwen_half_ops.cu:379-583 (SIMT
// tiles with an LUT decode) and cpp_engine/cuda/fp8_ops.cu:142-300 (whole-weight dequant
// to fp16 in HBM followed by cublasGemmEx).
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;
using namespace pk::sm100;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 4;
constexpr int kTileBytes = BM * BK * 2;  // 16 KB per operand tile (bf16)
constexpr int kThreads = 192;            // warp0 TMA, warp1 MMA, warps 2-5 dequant + epilogue
constexpr uint32_t kTmemCols = 128;

enum { WFMT_FP8_BLOCK128 = 0, WFMT_BF16 = 1 };
enum { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_RESID = 2, EPI_F32 = 3 };

struct GemmParams {
  const void* W;        // [N, K] raw weights
  const float* scale;   // fp8: [ceil(N/128), ceil(K/128)]
  int wfmt;
  int M, N, K;
  int epi;
  bf16* C;              // EPI_BF16 / EPI_RESID: [M, ldc]; EPI_SWIGLU: [M, ldc] with N/2 columns
  float* Cf;            // EPI_F32
  const bf16* resid;    // EPI_RESID: [M, ldc]
  int ldc;
  uint32_t* status;     // device status word, 0 = ok
};

struct __align__(1024) SmemLayout {
  uint8_t a[kStages][kTileBytes];
  uint8_t b[kStages][kTileBytes];
  uint64_t full_a[kStages];
  uint64_t full_b[kStages];
  uint64_t empty[kStages];
  uint64_t accum_full;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// Tile row -> weight row. For SwiGLU the first 64 tile rows are gate rows and the last
// 64 the matching up rows, so that one thread of the epilogue owns both values.
__device__ __forceinline__ int weight_row(const GemmParams& p, int n0, int r) {
  if (p.epi == EPI_SWIGLU) {
    const int half_n = p.N >> 1;
    const int j = (n0 >> 1) + (r & 63);
    if (j >= half_n) return -1;
    return r < 64 ? j : half_n + j;
  }
  const int n = n0 + r;
  return n < p.N ? n : -1;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  SmemLayout& sm = *reinterpret_cast<SmemLayout*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int num_kb = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full_a[s], 1);
      mbar_init(&sm.full_b[s], 128);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.accum_full, 1);
    sm.abort_flag = 0;
    mbar_fence_init();
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
    // ---------------- TMA producer for A ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % kStages;
        if (!mbar_wait(&sm.empty[s], ((kb / kStages) & 1) ^ 1, &sm.abort_flag, p.status, 11)) break;
        mbar_arrive_expect_tx(&sm.full_a[s], kTileBytes);
        tma_load_2d(sm.a[s], &tmap_a, &sm.full_a[s], kb * BK, m0);
        issued = kb + 1;
      }
      if (sm.abort_flag) {
        // Gave up: let the copies already in flight land before the CTA exits.
        for (int kb = max(0, issued - kStages); kb < issued; ++kb) {
          const int s = kb % kStages;
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(&sm.full_a[s], (kb / kStages) & 1)) break;
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
        mbar_wait(&sm.full_a[s], ph, &sm.abort_flag, p.status, 12);
        mbar_wait(&sm.full_b[s], ph, &sm.abort_flag, p.status, 13);
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
    // ---------------- weight decode producers, then epilogue ----------------
    const int t = threadIdx.x - 64;        // 0..127
    const int chunk = t & 3;               // which 16 K-elements of the 64-wide tile row
    const int rbase = t >> 2;              // row within a group of 32
    const int kb_scale = (p.K + 127) >> 7;
    int wrow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wrow[i] = weight_row(p, n0, rbase + 32 * i);

    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % kStages;
      const int k0 = kb * BK + chunk * 16;
      // Issue the global loads before waiting for the slot.
      uint4 raw[4][2];
      float sc[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        raw[i][0] = make_uint4(0, 0, 0, 0);
        raw[i][1] = raw[i][0];
        sc[i] = 0.f;
        if (wrow[i] >= 0) {
          if (p.wfmt == WFMT_FP8_BLOCK128) {
            raw[i][0] = ld_stream_u4((const uint8_t*)p.W + (size_t)wrow[i] * p.K + k0);
            sc[i] = __ldg(p.scale + (size_t)(wrow[i] >> 7) * kb_scale + (k0 >> 7));
          } else {
            const bf16* src = (const bf16*)p.W + (size_t)wrow[i] * p.K + k0;
            raw[i][0] = ld_stream_u4(src);
            raw[i][1] = ld_stream_u4(src + 8);
          }
        }
      }
      mbar_wait(&sm.empty[s], ((kb / kStages) & 1) ^ 1, &sm.abort_flag, p.status, 14);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = rbase + 32 * i;
        uint4 lo, hi;
        if (p.wfmt == WFMT_FP8_BLOCK128) {
          const uint32_t w[4] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w};
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = e4m3x2_to_float2((uint16_t)(w[j] & 0xffffu));
            const float2 b = e4m3x2_to_float2((uint16_t)(w[j] >> 16));
            o[2 * j] = pack_bf16(a.x * sc[i], a.y * sc[i]);
            o[2 * j + 1] = pack_bf16(b.x * sc[i], b.y * sc[i]);
          }
          lo = make_uint4(o[0], o[1], o[2], o[3]);
          hi = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
          lo = raw[i][0];
          hi = raw[i][1];
        }
        uint8_t* rowp = sm.b[s] + (r >> 3) * 1024 + (r & 7) * 128;
        *reinterpret_cast<uint4*>(rowp + (((2 * chunk) ^ (r & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(rowp + (((2 * chunk + 1) ^ (r & 7)) << 4)) = hi;
      }
      fence_proxy_async_smem();
      mbar_arrive(&sm.full_b[s]);
    }

    // ---------------- epilogue ----------------
    mbar_wait(&sm.accum_full, 0, &sm.abort_flag, p.status, 15);
    tc_fence_after();
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int m = m0 + q * 32 + lane;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(q * 32) << 16);
    const bool row_ok = m < p.M && !sm.abort_flag;
    if (p.epi == EPI_SWIGLU) {
      const int half_n = p.N >> 1;
      const int j0 = n0 >> 1;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(lane_addr + c * 32, g);
        tmem_ld_32x32(lane_addr + 64 + c * 32, u);
        tmem_ld_wait();
        if (row_ok) {
          bf16* dst = p.C + (size_t)m * p.ldc + j0 + c * 32;
          if (j0 + c * 32 + 32 <= half_n) {
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
              if (j0 + c * 32 + i < half_n)
                dst[i] = __float2bfloat16(silu(__uint_as_float(g[i])) * __uint_as_float(u[i]));
          }
        }
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + c * 32, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        const int n = n0 + c * 32;
        if (p.epi == EPI_F32) {
          float* dst = p.Cf + (size_t)m * p.ldc + n;
          for (int i = 0; i < 32; ++i)
            if (n + i < p.N) dst[i] = __uint_as_float(r[i]);
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
    tc_fence_before();
  }

  __syncthreads();
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

}  // namespace

// A: [M, K] bf16 row-major with row stride lda elements (lda*2 bytes a multiple of 16, base
// 16-byte aligned). K must be a multiple of 64. For epi == 1 (SwiGLU) W holds N/2 gate rows
// followed by N/2 up rows and C has N/2 columns.
PK_API int pk_gemm_umma(const void* A, int lda, const void* W, const float* scale, int wfmt, int M, int N,
                        int K, int epi, void* C, const void* resid, int ldc, uint32_t* status,
                        cudaStream_t stream) {
  if (M < 1 || N < 1 || K < BK || (K % BK) != 0) return PK_ERR_BAD_ARG;
  if (((uintptr_t)A & 15) != 0 || ((size_t)lda * 2) % 16 != 0) return PK_ERR_BAD_ARG;
  if (wfmt != WFMT_FP8_BLOCK128 && wfmt != WFMT_BF16) return PK_ERR_UNSUPPORTED;
  if (wfmt == WFMT_FP8_BLOCK128 && (scale == nullptr || ((uintptr_t)W & 15) != 0)) return PK_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU && ((N & 1) != 0)) return PK_ERR_BAD_ARG;
  if ((ldc & 7) != 0 && epi != EPI_F32) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;

  CUtensorMap tmap;
  const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t gstride[1] = {(cuuint64_t)lda * 2};
  const cuuint32_t box[2] = {BK, BM};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(A), gdim, gstride, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    return PK_ERR_CUDA;
  }

  GemmParams p{};
  p.W = W;
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

  const size_t smem = sizeof(SmemLayout) + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    configured = true;
  }
  const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_umma_kernel<<<grid, kThreads, smem, stream>>>(tmap, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

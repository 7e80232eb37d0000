// Causal GQA attention for prefill chunks on the 5th-generation tensor cores.
//
// One CTA works one (query head, tile of 128 query rows). For every tile of 128 cached positions up to the causal limit:
//   S  = Q K^T          tcgen05.mma kind::f16, both operands K-major (head dim contiguous), fp32 S in TMEM
//   P  = exp2(S - m)    four softmax warps, one query row per thread: tcgen05.ld, mask, running max / sum, bf16 P written
//                       into shared memory in the K-major 128-byte-swizzle operand layout
//   PV = P V            tcgen05.mma with V as an MN-major operand (the cache stores a position's 128 channels
//                       contiguously, which is the MN direction of this product), fresh accumulator in TMEM
//   O  = O * alpha + PV folded into fp32 registers of the softmax warps (the same hand-over as the FP8 GEMM's k blocks)
// K and V tiles arrive by TMA (no multicast) into two alternating buffers, the next tile's loads in flight during the
// current tile's arithmetic. The output is divided by the row sum, gated (sigmoid of the projection's gate half) and
// written as bf16.
//
// Every wait is bounded (status word + CTA-wide abort flag).
//
// Reference counterpart: cpp_engine/cuda/qwen_gqa_optimized.cu:106-249 (tiled prefill attention on SIMT lanes) and
// cpp_engine/cuda/qwen_half_ops.cu:1161 (gqa_prefill_f16_kernel).
#include "../common/pk_sm100.cuh"

namespace {

using namespace pk;
using namespace pk::sm100;

constexpr int kD = 128;
constexpr int kTile = 128;
constexpr int kPanel = kTile * 128;        // bytes of one 64-element-wide panel of a 128-row bf16 tile
constexpr int kTileBytes = 2 * kPanel;     // 32 KB
constexpr int kThreads = 32 + 128;         // warp 0: TMA + MMA issue; warps 1-4: softmax, fold, epilogue
constexpr uint32_t kTmemCols = 256;        // S and PV, 128 fp32 columns each

struct Params {
  int M, Hq, Hkv, cap;
  const int* pos;          // [M] positions of the query rows (consecutive)
  float scale_log2;        // softmax scale * log2(e)
  const bf16* gate;        // [M, ld] or null; gate of head h at h * 256 + 128
  int ld;
  bf16* out;               // [M, Hq * 128]
  uint32_t* status;
};

struct __align__(1024) Smem {
  uint8_t q[kTileBytes];
  uint8_t k[2][kTileBytes];
  uint8_t v[2][kTileBytes];
  uint8_t p[kTileBytes];
  uint64_t q_full, kv_full[2], s_full, p_ready, pv_full;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

// MN-major operand with the 128-byte swizzle: 64 contiguous elements (128 B) per row, 8 rows per 1024-byte atom; atoms
// follow each other along K every `sbo` bytes and along MN every `lbo` bytes.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
gqa_prefill_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const Params p) {
  extern __shared__ uint8_t smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, row0 = blockIdx.x * kTile;
  const int kvh = h / (p.Hq / p.Hkv);
  // positions are consecutive: the last row of this tile decides how far the cache is read
  const int pos0 = __ldg(p.pos);
  const int last_row = min(row0 + kTile, p.M) - 1;
  const int n_tiles = (pos0 + last_row) / kTile + 1;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.kv_full[0], 1);
    mbar_init(&sm.kv_full[1], 1);
    mbar_init(&sm.s_full, 1);
    mbar_init(&sm.p_ready, 4);
    mbar_init(&sm.pv_full, 1);
    sm.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = sm.tmem_base, tmem_pv = sm.tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      auto load_kv = [&](int t) {
        const int b = t & 1;
        mbar_arrive_expect_tx(&sm.kv_full[b], 2 * kTileBytes);
        const int y = kvh * p.cap + t * kTile;
        tma_load_2d(sm.k[b], &tmap_k, &sm.kv_full[b], 0, y);
        tma_load_2d(sm.k[b] + kPanel, &tmap_k, &sm.kv_full[b], 64, y);
        tma_load_2d(sm.v[b], &tmap_v, &sm.kv_full[b], 0, y);
        tma_load_2d(sm.v[b] + kPanel, &tmap_v, &sm.kv_full[b], 64, y);
      };
      mbar_arrive_expect_tx(&sm.q_full, kTileBytes);
      tma_load_2d(sm.q, &tmap_q, &sm.q_full, h * kD, row0);
      tma_load_2d(sm.q + kPanel, &tmap_q, &sm.q_full, h * kD + 64, row0);
      load_kv(0);
      constexpr uint32_t idesc_s = umma_idesc(1, 1, kTile, kTile);                  // bf16 x bf16, both K-major
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, kTile, kD) | (1u << 16);       // B (= V) MN-major
      bool ok = mbar_wait(&sm.q_full, 0, &sm.abort_flag, p.status, 41);
      int issued = 1;     // K/V tiles whose loads were issued
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int b = t & 1;
        if (!mbar_wait(&sm.kv_full[b], (t >> 1) & 1, &sm.abort_flag, p.status, 42)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sm.q), ka = smem_u32(sm.k[b]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma_f16(tmem_s, smem_desc_k_sw128(qa + (j >> 2) * kPanel + (j & 3) * 32), smem_desc_k_sw128(ka + (j >> 2) * kPanel + (j & 3) * 32), idesc_s, j > 0 ? 1u : 0u);
        umma_commit(&sm.s_full);
        // the other buffer was last read by the PV product of tile t - 1, whose completion the loop waited for below
        if (t + 1 < n_tiles) {
          load_kv(t + 1);
          issued = t + 2;
        }
        if (!mbar_wait(&sm.p_ready, t & 1, &sm.abort_flag, p.status, 43)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sm.p), va = smem_u32(sm.v[b]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma_f16(tmem_pv, smem_desc_k_sw128(pa + (j >> 2) * kPanel + (j & 3) * 32), smem_desc_mn_sw128(va + j * 2048, kPanel, 1024), idesc_pv, j > 0 ? 1u : 0u);
        umma_commit(&sm.pv_full);
        // S of the next tile overwrites the S columns (read before p_ready), its loads reuse this tile's buffers only
        // after the PV product is done
        if (!mbar_wait(&sm.pv_full, t & 1, &sm.abort_flag, p.status, 44)) { ok = false; break; }
      }
      if (!ok) {
        // gave up: let the tile loads in flight land before the CTA exits
        for (int t = max(issued - 2, 0); t < issued; ++t)
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(&sm.kv_full[t & 1], (t >> 1) & 1)) break;
      }
    }
  } else {
    const int q4 = warp & 3;                       // TMEM lane quarter of this warp
    const int r = q4 * 32 + lane;                  // query row inside the tile
    const int m = row0 + r;
    const bool row_ok = m < p.M;
    const int q_pos = pos0 + (row_ok ? m : p.M - 1);
    const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
    float o[kD];
#pragma unroll
    for (int i = 0; i < kD; ++i) o[i] = 0.f;
    float mx = -INFINITY, sum = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      if (!mbar_wait(&sm.s_full, t & 1, &sm.abort_flag, p.status, 45)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = t * kTile;
      // pass 1: the row's maximum over the positions it may see
      float tmax = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_s + lane_off + c * 32, s);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (kv0 + c * 32 + i <= q_pos) tmax = fmaxf(tmax, __uint_as_float(s[i]));
      }
      const float m_new = fmaxf(mx, tmax * p.scale_log2);
      const float alpha = mx == -INFINITY ? 0.f : exp2f(mx - m_new);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      // pass 2: probabilities, row sum, bf16 P into the operand layout
      float tsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(tmem_s + lane_off + c * 32, s);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a = kv0 + c * 32 + i <= q_pos ? exp2f(__uint_as_float(s[i]) * p.scale_log2 - base) : 0.f;
          const float b2 = kv0 + c * 32 + i + 1 <= q_pos ? exp2f(__uint_as_float(s[i + 1]) * p.scale_log2 - base) : 0.f;
          const __nv_bfloat162 pr = __floats2bfloat162_rn(a, b2);
          // the sum runs over the rounded values, which are what the PV product multiplies
          tsum += __bfloat162float(pr.x) + __bfloat162float(pr.y);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        uint8_t* prow = sm.p + (c >> 1) * kPanel + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = ((c & 1) * 4 + g) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
        }
      }
      sum = sum * alpha + tsum;
      mx = m_new;
      // P is complete for this warp's rows and S has been read: let the MMA thread go on
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_ready);
      if (!mbar_wait(&sm.pv_full, t & 1, &sm.abort_flag, p.status, 46)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pv[32];
        tmem_ld_32x32(tmem_pv + lane_off + c * 32, pv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(pv[i]));
      }
      tc_fence_before();
    }
    if (ok && row_ok) {
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      bf16* dst = p.out + (size_t)m * p.Hq * kD + h * kD;
      const bf16* g = p.gate ? p.gate + (size_t)m * p.ld + h * 2 * kD + kD : nullptr;
#pragma unroll
      for (int v = 0; v < 16; ++v) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = o[v * 8 + e] * inv;
        if (g) {
          const uint4 gg = *reinterpret_cast<const uint4*>(g + v * 8);
          const uint32_t w[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            f[2 * e] *= 1.f / (1.f + __expf(-__uint_as_float(w[e] << 16)));
            f[2 * e + 1] *= 1.f / (1.f + __expf(-__uint_as_float(w[e] & 0xffff0000u)));
          }
        }
        uint32_t o4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 pr = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
          o4[e] = *reinterpret_cast<const uint32_t*>(&pr);
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(sm.tmem_base, kTmemCols);
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

bool encode_rows(EncodeTiledFn encode, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer) {
  const cuuint64_t gdim[2] = {inner, outer};
  const cuuint64_t gstride[1] = {inner * 2};
  const cuuint32_t box[2] = {64, kTile};
  const cuuint32_t estr[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// q [M, Hq, 128] bf16 (normalised and rotated), kcache / vcache [Hkv, ctx_cap, 128] bf16 already holding the rows of this
// chunk, pos [M] consecutive positions (pos[m] = pos[0] + m), full causal attention (no window). gate_proj as in
// pk_gqa_decode. Cache rows behind the last position are read (and masked): they must hold finite values.
PK_API int pk_gqa_prefill_umma(const void* q, const void* kcache, const void* vcache, const int* pos, int M, int Hq, int Hkv, int head_dim, int ctx_cap,
                               float scale, const void* gate_proj, int ld, void* out, uint32_t* status, cudaStream_t stream) {
  if (head_dim != kD) return PK_ERR_UNSUPPORTED;
  if (M < 1 || Hkv < 1 || Hq < Hkv || (Hq % Hkv) != 0 || ctx_cap < 1 || pos == nullptr || out == nullptr) return PK_ERR_BAD_ARG;
  if (((uintptr_t)q & 15) != 0 || ((uintptr_t)kcache & 15) != 0 || ((uintptr_t)vcache & 15) != 0 || ((uintptr_t)out & 15) != 0) return PK_ERR_BAD_ARG;
  if (gate_proj != nullptr && (((uintptr_t)gate_proj & 15) != 0 || (ld & 7) != 0)) return PK_ERR_BAD_ARG;
  EncodeTiledFn encode = encode_fn();
  if (encode == nullptr) return PK_ERR_UNSUPPORTED;
  CUtensorMap tq, tk, tv;
  if (!encode_rows(encode, &tq, q, (uint64_t)Hq * kD, (uint64_t)M)) return PK_ERR_CUDA;
  if (!encode_rows(encode, &tk, kcache, kD, (uint64_t)Hkv * ctx_cap)) return PK_ERR_CUDA;
  if (!encode_rows(encode, &tv, vcache, kD, (uint64_t)Hkv * ctx_cap)) return PK_ERR_CUDA;
  Params p{M, Hq, Hkv, ctx_cap, pos, scale * 1.4426950408889634f, (const pk::bf16*)gate_proj, ld, (pk::bf16*)out, status};
  const size_t smem = sizeof(Smem) + 1024;
  static PkDeviceOnce once;
  if (PkDeviceOnceGuard once_guard{once}; once_guard.needed()) {
    if (cudaFuncSetAttribute(gqa_prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      pk_set_last_cuda_error((int)cudaGetLastError());
      return PK_ERR_CUDA;
    }
    once_guard.done();
  }
  gqa_prefill_umma_kernel<<<dim3((M + kTile - 1) / kTile, Hq), kThreads, smem, stream>>>(tq, tk, tv, p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

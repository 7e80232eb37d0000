// Long-context chunk scorer ("FlashMemory"): for one decode token, score every compressed-KV chunk of a layer so that
// only the best chunks have to be resident on the device.
//
//   q_lora = RMSNorm(wq_a . hidden) * gamma          q[h] = Hadamard(RoPE(bf16(wq_b[h] . q_lora)))
//   w[h]   = (weights_proj[h] . hidden) / sqrt(head_dim * n_heads)
//   score[c] = sigmoid( sum_h relu(q[h] . k[c]) * w[h] )
//
// The sum over heads of 128-long dot products against every chunk key is a [n_chunks, 128] x [128, n_heads] matrix
// product: 16 kFLOP per 132 bytes of key, far above what SIMT lanes can do at HBM rate. So the keys stay E4M3 (one
// fp32 scale per chunk) and go through the FP8 tensor-core GEMM; the query side is tiny and is built by two SIMT kernels
// that end by writing each head as two E4M3 terms (code of q / s_h, code of the rounding residue) with s_h folded into
// w[h] (relu commutes with a positive scale).
//
// Reference counterpart: cpp_engine/cuda/flashmemory_ops.cu (matvec 319, rmsnorm 342, rope_hadamard 88, scale 367,
// score_chunks 130, score_float_keys 192, ensemble 233, topk 256, write_global_indices 308) and
// cpp_engine/include/flashmemory_ops.hpp.
#include <cuda_fp8.h>

#include "../common/pk_common.cuh"

extern "C" int pk_fp8_chunk_scores(const void* keys, const float* key_scale, int n_chunks, const void* qcodes, const float* head_w,
                                   const float* ones2, float* partial, int ld, uint32_t* status, int sm_count, cudaStream_t stream);

namespace {

using namespace pk;

constexpr int kHeadDim = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

// y[r] = W[r, :] . x, one warp per row.
__global__ void __launch_bounds__(256) fm_matvec_kernel(const float* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* w = W + (size_t)r * cols;
  float acc = 0.f;
  for (int c = lane; c < cols; c += 32) acc = fmaf(__ldg(w + c), __ldg(x + c), acc);
  acc = warp_sum(acc);
  if (lane == 0) y[r] = acc;
}

// One block of 128 threads per head: norm of q_lora, the head's 128 rows of wq_b, bf16 rounding, rotation of the last
// rope_dim entries (interleaved pairs), normalised Walsh-Hadamard transform, two-term E4M3 codes, and the head's weight.
__global__ void __launch_bounds__(128)
fm_query_kernel(const float* __restrict__ qlora, const float* __restrict__ gamma, const float* __restrict__ wq_b, const float* __restrict__ hidden,
                const float* __restrict__ weights_proj, const float* __restrict__ inv_freqs, int rank, int hidden_dim, int n_heads, int rope_dim,
                float eps, long long position, uint8_t* __restrict__ qcodes, float* __restrict__ head_w, float* __restrict__ q_out) {
  extern __shared__ float sm[];
  float* xl = sm;            // [rank] normalised q_lora
  float* vec = sm + rank;    // [128]
  __shared__ float red[4];
  const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float ss = 0.f;
  for (int i = tid; i < rank; i += 128) {
    const float v = qlora[i];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  const float inv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)rank + eps);
  for (int i = tid; i < rank; i += 128) xl[i] = qlora[i] * inv * gamma[i];
  __syncthreads();
  for (int r = warp * 32; r < warp * 32 + 32; ++r) {
    const float* w = wq_b + ((size_t)h * kHeadDim + r) * rank;
    float acc = 0.f;
    for (int c = lane; c < rank; c += 32) acc = fmaf(__ldg(w + c), xl[c], acc);
    acc = warp_sum(acc);
    if (lane == 0) vec[r] = round_bf16(acc);
  }
  __syncthreads();
  const int rope_start = kHeadDim - rope_dim;
  if (tid * 2 < rope_dim) {
    const int off = rope_start + tid * 2;
    float sn, cs;
    sincosf((float)position * inv_freqs[tid], &sn, &cs);
    const float a = vec[off], b = vec[off + 1];
    vec[off] = round_bf16(a * cs - b * sn);
    vec[off + 1] = round_bf16(a * sn + b * cs);
  }
  __syncthreads();
  for (int stride = 1; stride < kHeadDim; stride <<= 1) {
    if ((tid & stride) == 0) {
      const float a = vec[tid], b = vec[tid + stride];
      vec[tid] = a + b;
      vec[tid + stride] = a - b;
    }
    __syncthreads();
  }
  const float v = vec[tid] * rsqrtf((float)kHeadDim);
  if (q_out) q_out[(size_t)h * kHeadDim + tid] = v;
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __syncthreads();
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float s = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float y = v / s;
  const __nv_fp8_storage_t hi = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
  const float back = __half2float(__half(__nv_cvt_fp8_to_halfraw(hi, __NV_E4M3)));
  qcodes[(size_t)h * kHeadDim + tid] = hi;
  qcodes[(size_t)(128 + h) * kHeadDim + tid] = __nv_cvt_float_to_fp8(y - back, __NV_SATFINITE, __NV_E4M3);
  // the head's weight, with the code scale folded in
  const float* wp = weights_proj + (size_t)h * hidden_dim;
  float acc = 0.f;
  for (int c = tid; c < hidden_dim; c += 128) acc = fmaf(__ldg(wp + c), __ldg(hidden + c), acc);
  acc = warp_sum(acc);
  __syncthreads();
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (tid == 0) head_w[h] = (red[0] + red[1] + red[2] + red[3]) * rsqrtf((float)kHeadDim) * rsqrtf((float)n_heads) * s;
}

// fp32 keys [n, 128] -> E4M3 codes + one scale (amax / 448) per chunk; one warp per chunk.
__global__ void __launch_bounds__(256) fm_quant_keys_kernel(const float* __restrict__ keys, int n, uint8_t* __restrict__ codes, float* __restrict__ scale) {
  const int c = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (c >= n) return;
  const float4 v = *reinterpret_cast<const float4*>(keys + (size_t)c * kHeadDim + lane * 4);
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax * (1.f / 448.f) : 1.f, inv = 1.f / s;
  const uint32_t packed = (uint32_t)__nv_cvt_float_to_fp8(v.x * inv, __NV_SATFINITE, __NV_E4M3) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v.y * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v.z * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                          ((uint32_t)__nv_cvt_float_to_fp8(v.w * inv, __NV_SATFINITE, __NV_E4M3) << 24);
  *reinterpret_cast<uint32_t*>(codes + (size_t)c * kHeadDim + lane * 4) = packed;
  if (lane == 0) scale[c] = s;
}

// The reference's packed rows (128 code bytes followed by the 4 bytes of the fp32 scale) -> separate arrays.
__global__ void __launch_bounds__(256) fm_unpack_keys_kernel(const uint8_t* __restrict__ packed, int n, uint8_t* __restrict__ codes, float* __restrict__ scale) {
  const int c = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (c >= n) return;
  const uint8_t* row = packed + (size_t)c * (kHeadDim + 4);
#pragma unroll
  for (int i = 0; i < 4; ++i) codes[(size_t)c * kHeadDim + i * 32 + lane] = row[i * 32 + lane];
  if (lane == 0) {
    const uint32_t b = (uint32_t)row[128] | ((uint32_t)row[129] << 8) | ((uint32_t)row[130] << 16) | ((uint32_t)row[131] << 24);
    scale[c] = __uint_as_float(b);
  }
}

// scores[c] = f(sum of the four partials of chunk c)
__global__ void __launch_bounds__(256) fm_finish_kernel(const float* __restrict__ partial, int ld, int n, int apply_sigmoid, float* __restrict__ scores) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= n) return;
  const float x = partial[c] + partial[(size_t)ld + c] + partial[(size_t)2 * ld + c] + partial[(size_t)3 * ld + c];
  scores[c] = apply_sigmoid ? 1.f / (1.f + __expf(-x)) : x;
}

__global__ void __launch_bounds__(256) fm_ensemble_kernel(const float* __restrict__ layer_scores, int n_layers, int n, int stride, int use_max, float* __restrict__ out) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= n) return;
  float acc = layer_scores[c];
  for (int l = 1; l < n_layers; ++l) {
    const float v = layer_scores[(size_t)l * stride + c];
    acc = use_max ? fmaxf(acc, v) : acc + v;
  }
  out[c] = use_max ? acc : acc / (float)n_layers;
}

__global__ void __launch_bounds__(256) fm_offset_indices_kernel(const int* __restrict__ logical, int keep, int offset, int* __restrict__ out) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < keep) out[i] = logical[i] < 0 ? -1 : logical[i] + offset;
}

}  // namespace

// Query side of the scorer. qlora_scratch [rank], qcodes [256 * 128] bytes (zeroed here), head_w [128] (zeroed here),
// q_out optional fp32 [n_heads, 128] (the rotated query, for tests). head_dim is 128, n_heads <= 128.
PK_API int pk_flashmemory_build_query(const float* hidden, const float* wq_a, const float* wq_b, const float* q_norm, const float* weights_proj,
                                      const float* inv_freqs, int n_heads, int q_lora_rank, int hidden_dim, int rope_dim, float eps,
                                      long long position, float* qlora_scratch, void* qcodes, float* head_w, float* q_out, cudaStream_t stream) {
  if (n_heads < 1 || n_heads > 128 || q_lora_rank < 1 || hidden_dim < 1 || rope_dim < 2 || rope_dim > kHeadDim || (rope_dim & 1)) return PK_ERR_BAD_ARG;
  if (hidden == nullptr || wq_a == nullptr || wq_b == nullptr || q_norm == nullptr || weights_proj == nullptr || inv_freqs == nullptr ||
      qlora_scratch == nullptr || qcodes == nullptr || head_w == nullptr)
    return PK_ERR_BAD_ARG;
  const size_t smem = (size_t)(q_lora_rank + kHeadDim) * sizeof(float);
  if (smem > 48 * 1024) return PK_ERR_UNSUPPORTED;
  if (cudaMemsetAsync(qcodes, 0, 256 * kHeadDim, stream) != cudaSuccess || cudaMemsetAsync(head_w, 0, 128 * sizeof(float), stream) != cudaSuccess)
    return PK_ERR_CUDA;
  fm_matvec_kernel<<<(q_lora_rank + 7) / 8, 256, 0, stream>>>(wq_a, hidden, qlora_scratch, q_lora_rank, hidden_dim);
  PK_CHECK_LAUNCH();
  fm_query_kernel<<<n_heads, 128, smem, stream>>>(qlora_scratch, q_norm, wq_b, hidden, weights_proj, inv_freqs, q_lora_rank, hidden_dim, n_heads,
                                                  rope_dim, eps, position, (uint8_t*)qcodes, head_w, q_out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_flashmemory_quant_keys(const float* keys, int n_chunks, void* codes, float* scale, cudaStream_t stream) {
  if (keys == nullptr || codes == nullptr || scale == nullptr || n_chunks < 1 || ((uintptr_t)keys & 15) != 0 || ((uintptr_t)codes & 3) != 0) return PK_ERR_BAD_ARG;
  fm_quant_keys_kernel<<<(n_chunks + 7) / 8, 256, 0, stream>>>(keys, n_chunks, (uint8_t*)codes, scale);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

PK_API int pk_flashmemory_unpack_keys(const void* packed, int n_chunks, void* codes, float* scale, cudaStream_t stream) {
  if (packed == nullptr || codes == nullptr || scale == nullptr || n_chunks < 1) return PK_ERR_BAD_ARG;
  fm_unpack_keys_kernel<<<(n_chunks + 7) / 8, 256, 0, stream>>>((const uint8_t*)packed, n_chunks, (uint8_t*)codes, scale);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Scores of every chunk against a built query. partial: fp32 scratch [4 * n_chunks]; ones2: two floats equal to 1.
PK_API int pk_flashmemory_score_chunks(const void* key_codes, const float* key_scale, int n_chunks, const void* qcodes, const float* head_w,
                                       const float* ones2, float* partial, int apply_sigmoid, float* scores, uint32_t* status, int sm_count,
                                       cudaStream_t stream) {
  if (scores == nullptr) return PK_ERR_BAD_ARG;
  const int rc = pk_fp8_chunk_scores(key_codes, key_scale, n_chunks, qcodes, head_w, ones2, partial, n_chunks, status, sm_count, stream);
  if (rc != PK_OK) return rc;
  fm_finish_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>(partial, n_chunks, n_chunks, apply_sigmoid, scores);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Max or mean over scorer layers: layer_scores [n_layers][stride] -> out [n_chunks].
PK_API int pk_flashmemory_ensemble(const float* layer_scores, int n_layers, int n_chunks, int stride, int use_max, float* out, cudaStream_t stream) {
  if (layer_scores == nullptr || out == nullptr || n_layers < 1 || n_chunks < 1 || stride < n_chunks) return PK_ERR_BAD_ARG;
  fm_ensemble_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>(layer_scores, n_layers, n_chunks, stride, use_max, out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// out[i] = logical[i] + offset (the position of a logical chunk behind a layer's window rows); -1 stays -1.
PK_API int pk_flashmemory_write_global_indices(const int* logical, int keep, int offset, int* out, cudaStream_t stream) {
  if (logical == nullptr || out == nullptr || keep < 1) return PK_ERR_BAD_ARG;
  fm_offset_indices_kernel<<<(keep + 255) / 256, 256, 0, stream>>>(logical, keep, offset, out);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

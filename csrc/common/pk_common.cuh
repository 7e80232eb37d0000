// Shared device helpers for every kernel of the library: dtype conversion, warp and
// block reductions, FP8 E4M3 / FP4 E2M1 / E8M0 decoding, bounded waits.
#pragma once
#include <mutex>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PK_API extern "C" __attribute__((visibility("default")))

// Return codes of every launcher in the library.
enum PkStatus : int {
  PK_OK = 0,
  PK_ERR_BAD_ARG = 1,      // shape / alignment contract broken, nothing launched
  PK_ERR_CUDA = 2,         // a CUDA runtime call failed (see pk_last_cuda_error)
  PK_ERR_TIMEOUT = 3,      // a bounded device wait gave up
  PK_ERR_UNSUPPORTED = 4,
};

#define PK_CHECK_LAUNCH()                                   \
  do {                                                      \
    cudaError_t e__ = cudaGetLastError();                   \
    if (e__ != cudaSuccess) {                               \
      pk_set_last_cuda_error((int)e__);                     \
      return PK_ERR_CUDA;                                   \
    }                                                       \
  } while (0)

// ---- debug build (-DPK_DEBUG_BOUNDS=1): index checks that record instead of faulting ----
// The release kernels either guard an index silently (a KV position outside the cache is not written) or trust the
// caller (route ids). The debug library records the first bad index of every translation unit as
// {code, index, limit, count} in a device word that the host reads with pk_debug_bounds_read(), and skips the access.
// Codes: 101 KV-cache position, 102 routed expert id, 103 selected row.
#if defined(PK_DEBUG_BOUNDS) && PK_DEBUG_BOUNDS && defined(__CUDACC__)
extern "C" void pk_debug_register(int (*read)(unsigned*), int (*clear)());
namespace pk {
namespace dbg {
static __device__ unsigned int g_word[4];
__device__ __forceinline__ void record(unsigned code, long long index, long long limit) {
  if (atomicCAS(&g_word[0], 0u, code) == 0u) {
    g_word[1] = (unsigned)index;
    g_word[2] = (unsigned)limit;
  }
  atomicAdd(&g_word[3], 1u);
}
static int read_tu(unsigned* out)   // internal linkage: one per translation unit, next to its own word
 { return cudaMemcpyFromSymbol(out, g_word, sizeof(unsigned) * 4) == cudaSuccess ? 0 : 1; }
static int clear_tu() {
  const unsigned z[4] = {0, 0, 0, 0};
  return cudaMemcpyToSymbol(g_word, z, sizeof z) == cudaSuccess ? 0 : 1;
}
struct Registrar {
  Registrar() { pk_debug_register(&read_tu, &clear_tu); }
};
static Registrar g_registrar;
}  // namespace dbg
}  // namespace pk
#define PK_DEBUG_RECORD(code, index, limit) pk::dbg::record((code), (long long)(index), (long long)(limit))
#define PK_DEBUG_BUILD 1
#else
#define PK_DEBUG_RECORD(code, index, limit) ((void)0)
#define PK_DEBUG_BUILD 0
#endif

PK_API void pk_set_last_cuda_error(int code);
PK_API int pk_last_cuda_error();

namespace pk {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
  return __uint_as_float(((uint32_t)b) << 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum. `scratch` holds at least 33 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Two FP8 E4M3 codes (low byte first) -> two floats.
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// E8M0 exponent-only scale: 2^(code - 127). Code 255 is NaN in the format; the
// loaders never emit it.
__device__ __forceinline__ float e8m0_to_float(uint8_t code) {
  return __uint_as_float(code == 0 ? 0x00400000u : ((uint32_t)code) << 23);
}

// FP4 E2M1 value table {0, .5, 1, 1.5, 2, 3, 4, 6} with sign in bit 3.
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  const uint32_t mag = nib & 7u;
  // 0,0.5,1,1.5,2,3,4,6
  float v = mag < 2 ? 0.5f * (float)mag
                    : __uint_as_float(((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22));
  return (nib & 8u) ? -v : v;
}

// Programmatic dependent launch. `pdl_wait` returns once every kernel this grid depends on has
// completed and its writes are visible; before it a kernel may only touch data that no kernel
// writes (weights). `pdl_trigger` lets the next kernel of the stream be scheduled as blocks of
// this one retire. Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) {
  return x > 20.f ? x : log1pf(__expf(x));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// 128-bit streaming load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}

}  // namespace pk

// Per-device one-time set-up of a kernel (cudaFuncSetAttribute applies to the current device only, so a process that
// drives several GPUs must repeat it on each). Usage:
//   static PkDeviceOnce once;
//   if (PkDeviceOnceGuard g{once}; g.needed()) { ...set attributes...; g.done(); }
// The guard holds the object's mutex for the length of the if statement, so two host threads cannot race.
struct PkDeviceOnce {
  std::mutex mu;
  unsigned long long configured[4] = {0, 0, 0, 0};   // one bit per device ordinal (256 devices)
};
class PkDeviceOnceGuard {
 public:
  explicit PkDeviceOnceGuard(PkDeviceOnce& o) : o_(o), lock_(o.mu) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    word_ = (dev >> 6) & 3;
    bit_ = 1ull << (dev & 63);
  }
  bool needed() const { return (o_.configured[word_] & bit_) == 0ull; }
  void done() { o_.configured[word_] |= bit_; }

 private:
  PkDeviceOnce& o_;
  std::lock_guard<std::mutex> lock_;
  int word_ = 0;
  unsigned long long bit_ = 1ull;
};

// On by default (about 4% on the 27B decode graph in same-box A/B runs); POCKET_PDL=0 in the
// environment falls back to plain stream order.
PK_API int pk_pdl_enabled();

// Every kernel of the decode graph asks for the same shared-memory carve-out (the maximum): a kernel
// boundary where the preferred L1 / shared split changes makes the SMs drain and reconfigure.
inline void pk_prefer_max_smem(const void* fn) {
  static const void* seen_fn[1024];
  static int seen_dev[1024];
  static int n = 0;
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n; ++i)
    if (seen_fn[i] == fn && seen_dev[i] == dev) return;   // the hint belongs to one device
  cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (n < 1024) {
    seen_fn[n] = fn;
    seen_dev[n++] = dev;
  }
}

// Launch through cudaLaunchKernelEx; `pdl` adds programmatic stream serialization (see pdl_wait /
// pdl_trigger) when it is switched on.
template <class... KArgs, class... Args>
inline cudaError_t pk_launch_ex(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
  pk_prefer_max_smem((const void*)kernel);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && pk_pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define PK_LAUNCH_EX_(pdl, kernel, grid, block, smem, stream, ...)                                  \
  do {                                                                                              \
    cudaError_t e__ = pk_launch_ex(pdl, kernel, grid, block, smem, stream, __VA_ARGS__);            \
    if (e__ != cudaSuccess) {                                                                       \
      pk_set_last_cuda_error((int)e__);                                                             \
      return PK_ERR_CUDA;                                                                           \
    }                                                                                               \
  } while (0)
// for kernels that begin with pdl_wait()
#define PK_LAUNCH_PDL(kernel, grid, block, smem, stream, ...) PK_LAUNCH_EX_(true, kernel, grid, block, smem, stream, __VA_ARGS__)
// plain stream order
#define PK_LAUNCH(kernel, grid, block, smem, stream, ...) PK_LAUNCH_EX_(false, kernel, grid, block, smem, stream, __VA_ARGS__)

// All-reduce (sum, fp32) with the reduction done inside NVSwitch: `multimem.ld_reduce` on a multicast address
// returns the sum of the same element of every rank's buffer, and `multimem.st` writes one value into every rank's
// buffer. The unicast kernel of peer_allreduce.cu stores each rank's data into every peer (world x the payload out of
// every GPU); here a rank writes its data ONCE into its own memory and the switch does the fan-in.
//
// Every rank owns a symmetric buffer (same layout, mapped by every peer and bound to one multicast object):
//     data[2][capacity] fp32 | flags[2][2][world] u32 | seq | pushed | pushed2 | status | left
// One launch per rank:
//   1. every block copies its tiles of the input into data[parity] of its OWN buffer, fences at system scope;
//   2. the last block to finish publishes flag[parity][0][rank] = seq in every rank's buffer (plain peer stores);
//   3. every block waits (bounded, ld.acquire.sys) for all ranks' flags in its own buffer;
//   one shot (small payloads): every rank reads the whole vector with multimem.ld_reduce straight into `out`;
//   two shot (large payloads): rank r reduces slice r with multimem.ld_reduce and broadcasts it with multimem.st back
//   into data[parity] of every rank (nobody else reads that slice before the second barrier), then a second
//   publish / wait round on flag[parity][1][*], then every rank copies data[parity] into `out` from local memory:
//   each element crosses every link once in each direction.
// Two data sets alternate, as in the unicast kernel: a rank can be one call ahead of a peer, never two.
// A wait that runs out records PK_COMM_TIMEOUT in the status word and the kernel returns with `out` unspecified.
//
// The buffer and its multicast mapping come from the caller (the Python side takes them from
// torch.distributed._symmetric_memory); this file only holds the kernel and its launcher.
// Role in the reference: none (its all-reduce is NCCL or the CUDA-IPC kernel of src/csrc/cuda_kernel_impl.cu:4788-4829);
// this is the NVLink-switch form of the same collective.
#include <cuda_runtime.h>

#include "../common/pk_comm.cuh"

namespace {
using namespace pk;

struct MmParams {
  float* buf[PK_MAX_RANKS];   // unicast mapping of rank r's buffer (own buffer at index `rank`)
  float* mc;                  // multicast mapping of the same buffer
  int world, rank, two_shot;
  size_t capacity;            // floats per data set
  uint32_t timeout_us;
  const float* in;
  float* out;
  size_t n;
};

__device__ __forceinline__ uint32_t* mm_ctl(float* buf, size_t capacity) {
  return reinterpret_cast<uint32_t*>(buf + (size_t)2 * capacity);
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, const float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// out[4 i .. 4 i + 3] = v, clipped at n.
__device__ __forceinline__ void store_out(const MmParams& p, size_t i, const float4 v) {
  if (4 * i + 3 < p.n) {
    reinterpret_cast<float4*>(p.out)[i] = v;
  } else {
    p.out[4 * i] = v.x;
    if (4 * i + 1 < p.n) p.out[4 * i + 1] = v.y;
    if (4 * i + 2 < p.n) p.out[4 * i + 2] = v.z;
  }
}

// One thread per block: count this block in; the last one publishes `seq` to every rank; then wait for every rank.
__device__ __forceinline__ bool publish_and_wait(const MmParams& p, uint32_t* counter, int round, int parity, uint32_t seq, uint32_t* status_p) {
  uint32_t* c = mm_ctl(p.buf[p.rank], p.capacity);
  const uint32_t done = atomicAdd(counter, 1u) + 1u;
  if (done == gridDim.x) {
    *counter = 0u;   // every block has added exactly once: re-arm for the next launch
    __threadfence_system();
    for (int r = 0; r < p.world; ++r) st_relaxed_sys(mm_ctl(p.buf[r], p.capacity) + (parity * 2 + round) * p.world + p.rank, seq);
  }
  bool ok = *((volatile uint32_t*)status_p) == 0u;
  const uint64_t t0 = global_timer_ns(), budget = (uint64_t)p.timeout_us * 1000ull;
  while (ok && !all_reached(c + (parity * 2 + round) * p.world, p.world, seq)) {
    if (global_timer_ns() - t0 > budget) {
      atomicExch(status_p, PK_COMM_TIMEOUT);
      ok = false;
      break;
    }
    __nanosleep(40);
  }
  __threadfence_system();
  return ok;
}

__global__ void __launch_bounds__(256) multimem_allreduce_kernel(const MmParams p) {
  float* mine = p.buf[p.rank];
  uint32_t* c = mm_ctl(mine, p.capacity);
  uint32_t* seq_p = c + 4 * p.world;
  uint32_t* pushed_p = seq_p + 1;
  uint32_t* pushed2_p = seq_p + 2;
  uint32_t* status_p = seq_p + 3;
  uint32_t* left_p = seq_p + 4;
  const uint32_t seq = *((volatile uint32_t*)seq_p) + 1u;
  const int parity = (int)(seq & 1u);
  const size_t n4 = (p.n + 3) >> 2;          // the data sets are padded to whole float4s (capacity is a multiple of 4)
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  float* data = mine + (size_t)parity * p.capacity;
  float* data_mc = p.mc + (size_t)parity * p.capacity;

  // 1. this rank's data into its own buffer (the tail of the last float4 is zero filled)
  for (size_t i = tid; i < n4; i += stride) {
    float4 v;
    if (4 * i + 3 < p.n) {
      v = reinterpret_cast<const float4*>(p.in)[i];
    } else {
      v.x = p.in[4 * i];
      v.y = 4 * i + 1 < p.n ? p.in[4 * i + 1] : 0.f;
      v.z = 4 * i + 2 < p.n ? p.in[4 * i + 2] : 0.f;
      v.w = 0.f;
    }
    reinterpret_cast<float4*>(data)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool s_ok;
  if (threadIdx.x == 0) s_ok = publish_and_wait(p, pushed_p, 0, parity, seq, status_p);
  __syncthreads();
  bool ok = s_ok;

  if (ok && !p.two_shot) {
    // 2. one shot: the switch sums the element of every rank
    // four independent loads in flight per thread: a load through the switch takes a few microseconds
    for (size_t i0 = tid; i0 < n4; i0 += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < n4) v[u] = multimem_ld_reduce_f32x4(data_mc + 4 * (i0 + u * stride));
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < n4) store_out(p, i0 + u * stride, v[u]);
    }
  } else if (ok) {
    // 2. two shot: reduce this rank's slice in the switch and broadcast it into every rank's data set
    const size_t per = (n4 + p.world - 1) / p.world, lo = (size_t)p.rank * per, hi = lo + per < n4 ? lo + per : n4;
    for (size_t i0 = lo + tid; i0 < hi; i0 += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < hi) v[u] = multimem_ld_reduce_f32x4(data_mc + 4 * (i0 + u * stride));
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * stride < hi) multimem_st_f32x4(data_mc + 4 * (i0 + u * stride), v[u]);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_ok = publish_and_wait(p, pushed2_p, 1, parity, seq, status_p);
    __syncthreads();
    ok = s_ok;
    if (ok) {
      // written by other ranks through the multicast mapping: read past L1
      for (size_t i = tid; i < n4; i += stride) store_out(p, i, __ldcg(reinterpret_cast<const float4*>(data) + i));
    }
  }
  // The last block to leave advances the sequence number and re-arms its counter.
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t left = atomicAdd(left_p, 1u) + 1u;
    if (left == gridDim.x) {
      *left_p = 0u;
      *pushed_p = 0u;      // also after a timeout, where a block may have skipped a round
      *pushed2_p = 0u;
      *seq_p = seq;
      __threadfence();
    }
  }
}

}  // namespace

// Bytes of one rank's symmetric buffer for `world` ranks and `capacity` floats per call (capacity a multiple of 4).
PK_API size_t pk_mm_buffer_bytes(int world, size_t capacity) {
  return (size_t)2 * capacity * sizeof(float) + ((size_t)4 * world + 5) * sizeof(uint32_t);
}

// bufs[r]: unicast mapping of rank r's buffer (zeroed before the first call); mc: multicast mapping of the same buffer.
// in / out fp32, 16-byte aligned, n <= capacity; out may alias in. two_shot: reduce-scatter + all-gather through the switch.
PK_API int pk_mm_allreduce(void* const* bufs, void* mc, int world, int rank, size_t capacity, const float* in, float* out, size_t n,
                           int two_shot, unsigned timeout_us, int sm_count, cudaStream_t stream) {
  if (world < 1 || world > PK_MAX_RANKS || rank < 0 || rank >= world || n == 0 || n > capacity || mc == nullptr) return PK_ERR_BAD_ARG;
  if (((uintptr_t)in & 15) || ((uintptr_t)out & 15) || ((uintptr_t)mc & 15) || (capacity & 3)) return PK_ERR_BAD_ARG;
  MmParams p{};
  for (int r = 0; r < world; ++r) {
    if (bufs[r] == nullptr || ((uintptr_t)bufs[r] & 15)) return PK_ERR_BAD_ARG;
    p.buf[r] = (float*)bufs[r];
  }
  p.mc = (float*)mc;
  p.world = world;
  p.rank = rank;
  p.two_shot = two_shot;
  p.capacity = capacity;
  p.timeout_us = timeout_us;
  p.in = in;
  p.out = out;
  p.n = n;
  const size_t want = ((n + 3) / 4 + 255) / 256;
  const int cap = sm_count > 0 ? sm_count : 148;                  // every block must be resident while it waits
  const int blocks = (int)(want < 1 ? 1 : want > (size_t)cap ? (size_t)cap : want);
  multimem_allreduce_kernel<<<blocks, 256, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Reads (and optionally clears) the status word of a buffer; 0xffffffff if the copy fails.
PK_API unsigned pk_mm_status(void* buf, int world, size_t capacity, int clear) {
  uint32_t* status = (uint32_t*)((float*)buf + (size_t)2 * capacity) + 4 * world + 3;
  uint32_t v = 0xffffffffu;
  if (cudaMemcpy(&v, status, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
  if (clear && v != 0u) cudaMemset(status, 0, 4);
  return v;
}

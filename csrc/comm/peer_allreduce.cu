// One-kernel all-reduce (sum, fp32) over peer memory for small and medium payloads: the latency
// path of expert-parallel MoE combines and of any Python-level tensor-parallel runtime.
//
// Each rank owns an arena laid out as
//     slots[2][world][capacity] fp32 | flags[2][world] u32 | seq u32 | done u32 | status u32
// and maps every peer's arena (CUDA IPC). One launch per rank does all of:
//   1. every block copies its tiles of the input into slot[parity][my_rank] of EVERY rank
//      (plain stores over NVLink), fences at system scope;
//   2. the last block to finish publishes flag[parity][my_rank] = seq in every rank's arena
//      (st.release.sys);
//   3. every block waits (ld.acquire.sys, time budget) until all ranks' flags in its OWN arena
//      reached seq, then sums the `world` slots of its tiles into the output.
// `seq` lives in device memory and is advanced by the kernel itself, so the launch can sit in a
// CUDA graph. Two slot sets alternate: a rank can be one call ahead of a peer, never two (its
// call n+1 cannot finish before the peer has published n+1, which the peer does after reading n).
// The grid never exceeds one block per SM, so every block is resident while it waits.
// A wait that runs out records PK_COMM_TIMEOUT in the status word and the kernel returns; the
// output of that call is unspecified and the host is expected to check `pk_par_status`.
//
// Role of the reference's CUDA-IPC decode all-reduce (src/csrc/cuda_kernel_impl.cu:4788-4829 and
// `_DecodeCustomAllreduce`, src/models/deepseek_v4/runtime.py:206-289), for any world size <= 8.
#include <cuda_runtime.h>

#include "../common/pk_comm.cuh"

namespace {
using namespace pk;

struct ParParams {
  float* slot_base[PK_MAX_RANKS];      // arena of rank r (own arena at index `rank`)
  int world, rank;
  size_t capacity;                     // floats per slot
  uint32_t timeout_us;
  const float* in;
  float* out;
  size_t n;
  // MoE combine (in == nullptr): the value pushed for element (t, h) is this rank's weighted sum of the token's routes
  // through its local experts, taken from the per-route outputs in route order; the kernel is then dispatch (stores into
  // every rank), signal, wait and sum in one launch, with the per-token reduce as its producer.
  const float* ybuf;        // [routes, H] per-route expert outputs, expert-sorted
  const float* route_w;     // [routes] weight of each route (expert-sorted)
  const int* route_pos;     // [T * topk] position of route (t, k) in the expert-sorted order
  const int* seg;           // [E + 1]
  int topk, H, expert_offset, local_experts;
};

// This rank's contribution to element i = t * H + h of the MoE output.
__device__ __forceinline__ float moe_value(const ParParams& p, size_t i, int lo, int hi) {
  const int t = (int)(i / (size_t)p.H), h = (int)(i - (size_t)t * p.H);
  float acc = 0.f;
  for (int k = 0; k < p.topk; ++k) {
    const int pos = p.route_pos[t * p.topk + k];
    if (pos >= lo && pos < hi) acc = fmaf(p.route_w[pos], p.ybuf[(size_t)pos * p.H + h], acc);
  }
  return acc;
}

__device__ __forceinline__ float* slot(float* arena, size_t capacity, int world, int parity, int r) {
  return arena + ((size_t)parity * world + r) * capacity;
}
__device__ __forceinline__ uint32_t* ctl(float* arena, size_t capacity, int world) {
  return reinterpret_cast<uint32_t*>(arena + (size_t)2 * world * capacity);
}
// ctl layout: flags[2][world], seq, pushed, status, left

__global__ void __launch_bounds__(256) peer_allreduce_kernel(const ParParams p) {
  float* mine = p.slot_base[p.rank];
  uint32_t* c = ctl(mine, p.capacity, p.world);
  uint32_t* seq_p = c + 2 * p.world;
  uint32_t* pushed_p = seq_p + 1;   // blocks that have stored their part (first pass)
  uint32_t* status_p = seq_p + 2;
  uint32_t* left_p = seq_p + 3;     // blocks that have finished reading (second pass)
  const uint32_t seq = *((volatile uint32_t*)seq_p) + 1u;
  const int parity = (int)(seq & 1u);
  const size_t n4 = p.n >> 2;

  // 1. push
  if (p.in != nullptr) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      const float4 v = reinterpret_cast<const float4*>(p.in)[i];
      for (int r = 0; r < p.world; ++r) reinterpret_cast<float4*>(slot(p.slot_base[r], p.capacity, p.world, parity, p.rank))[i] = v;
    }
    for (size_t i = (n4 << 2) + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += (size_t)gridDim.x * blockDim.x) {
      const float v = p.in[i];
      for (int r = 0; r < p.world; ++r) slot(p.slot_base[r], p.capacity, p.world, parity, p.rank)[i] = v;
    }
  } else {
    // H is a multiple of 4, so a float4 never straddles two tokens
    const int lo = p.seg[p.expert_offset], hi = p.seg[p.expert_offset + p.local_experts];
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      const float4 v = make_float4(moe_value(p, 4 * i, lo, hi), moe_value(p, 4 * i + 1, lo, hi), moe_value(p, 4 * i + 2, lo, hi), moe_value(p, 4 * i + 3, lo, hi));
      for (int r = 0; r < p.world; ++r) reinterpret_cast<float4*>(slot(p.slot_base[r], p.capacity, p.world, parity, p.rank))[i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish (last block)
  __shared__ bool s_ok;
  if (threadIdx.x == 0) {
    // Two counters: with one, a block that skips the wait (status already set) could add its second-pass
    // increment before another block's first-pass one, and "every block has pushed" would be declared early.
    const uint32_t pushed = atomicAdd(pushed_p, 1u) + 1u;
    if (pushed == gridDim.x) {
      *pushed_p = 0u;   // every block has added exactly once: re-arm for the next launch
      // one fence, then the flag stores leave back to back (a release store per rank would wait for the one before it)
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        st_relaxed_sys(ctl(p.slot_base[r], p.capacity, p.world) + parity * p.world + p.rank, seq);
    }
    // 3a. wait for every rank (own arena): all flags polled together
    bool ok = *((volatile uint32_t*)status_p) == 0u;
    const uint64_t t0 = global_timer_ns(), budget = (uint64_t)p.timeout_us * 1000ull;
    while (ok && !all_reached(c + parity * p.world, p.world, seq)) {
      if (global_timer_ns() - t0 > budget) {
        atomicExch(status_p, PK_COMM_TIMEOUT);
        ok = false;
        break;
      }
      __nanosleep(40);
    }
    __threadfence_system();
    s_ok = ok;
  }
  __syncthreads();
  // 3b. reduce (also after a timeout, so that the kernel's memory traffic stays bounded and defined)
  if (s_ok) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      float4 a = reinterpret_cast<const float4*>(slot(mine, p.capacity, p.world, parity, 0))[i];
      for (int r = 1; r < p.world; ++r) {
        const float4 b = reinterpret_cast<const float4*>(slot(mine, p.capacity, p.world, parity, r))[i];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      reinterpret_cast<float4*>(p.out)[i] = a;
    }
    for (size_t i = (n4 << 2) + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n; i += (size_t)gridDim.x * blockDim.x) {
      float a = 0.f;
      for (int r = 0; r < p.world; ++r) a += slot(mine, p.capacity, p.world, parity, r)[i];
      p.out[i] = a;
    }
  }
  // The last block to leave advances the sequence number and re-arms its counter.
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t left = atomicAdd(left_p, 1u) + 1u;
    if (left == gridDim.x) {
      *left_p = 0u;
      *seq_p = seq;
      __threadfence();
    }
  }
}

}  // namespace

// Bytes of an arena for `world` ranks and `capacity` floats per call.
PK_API size_t pk_par_arena_bytes(int world, size_t capacity) {
  return ((size_t)2 * world * capacity) * sizeof(float) + ((size_t)2 * world + 4) * sizeof(uint32_t);
}

// A zeroed arena from cudaMalloc (a whole allocation, so that its IPC handle maps the same bytes on a peer).
PK_API void* pk_par_alloc(int world, size_t capacity) {
  void* p = nullptr;
  const size_t bytes = pk_par_arena_bytes(world, capacity);
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    pk_set_last_cuda_error((int)cudaGetLastError());
    return nullptr;
  }
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    pk_set_last_cuda_error((int)cudaGetLastError());
    cudaFree(p);
    return nullptr;
  }
  return p;
}

PK_API void pk_par_free(void* arena) {
  if (arena) cudaFree(arena);
}

// arenas[r] = mapped arena of rank r (own arena at r == rank); in/out fp32 with n <= capacity; out may alias in.
// in, out and capacity * 4 bytes must be 16-byte aligned.
PK_API int pk_par_allreduce(void* const* arenas, int world, int rank, size_t capacity, const float* in, float* out, size_t n,
                            unsigned timeout_us, int sm_count, cudaStream_t stream) {
  if (world < 1 || world > PK_MAX_RANKS || rank < 0 || rank >= world || n == 0 || n > capacity) return PK_ERR_BAD_ARG;
  if (((uintptr_t)in & 15) || ((uintptr_t)out & 15) || (capacity & 3)) return PK_ERR_BAD_ARG;
  ParParams p{};
  for (int r = 0; r < world; ++r) {
    if (arenas[r] == nullptr) return PK_ERR_BAD_ARG;
    p.slot_base[r] = (float*)arenas[r];
  }
  p.world = world;
  p.rank = rank;
  p.capacity = capacity;
  p.timeout_us = timeout_us;
  p.in = in;
  p.out = out;
  p.n = n;
  const size_t want = (n / 4 + 255) / 256;
  const int cap = sm_count > 0 ? sm_count : 148;                  // every block must be resident while it waits
  const int blocks = (int)(want < 1 ? 1 : want > (size_t)cap ? (size_t)cap : want);
  peer_allreduce_kernel<<<blocks, 256, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Reads (and optionally clears) the status word of an arena; returns 0xffffffff if the copy fails.
PK_API unsigned pk_par_status(void* arena, int world, size_t capacity, int clear) {
  uint32_t* status = (uint32_t*)((float*)arena + (size_t)2 * world * capacity) + 2 * world + 2;
  uint32_t v = 0xffffffffu;
  if (cudaMemcpy(&v, status, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 0xffffffffu;
  if (clear && v != 0u) cudaMemset(status, 0, 4);
  return v;
}

// MoE combine over peer memory: out [T, H] fp32 = sum over ranks of each rank's weighted per-token sum of its local
// experts' route outputs. ybuf [routes, H] and route_w [routes] are expert-sorted, route_pos [T * topk] maps route (t, k)
// to its sorted position, seg [E + 1] are the expert segments; this rank's experts are [expert_offset,
// expert_offset + local_experts). One launch: per-token reduce -> stores into every rank -> signal -> wait -> sum.
PK_API int pk_par_moe_combine(void* const* arenas, int world, int rank, size_t capacity, const float* ybuf, const float* route_w, const int* route_pos,
                              const int* seg, int expert_offset, int local_experts, int T, int topk, int H, float* out, uint32_t timeout_us,
                              int sm_count, cudaStream_t stream) {
  if (world < 1 || world > PK_MAX_RANKS || rank < 0 || rank >= world || T < 1 || topk < 1 || H < 4 || (H & 3) != 0) return PK_ERR_BAD_ARG;
  if (ybuf == nullptr || route_w == nullptr || route_pos == nullptr || seg == nullptr || out == nullptr) return PK_ERR_BAD_ARG;
  const size_t n = (size_t)T * H;
  if (n > capacity || ((uintptr_t)out & 15) != 0) return PK_ERR_BAD_ARG;
  ParParams p{};
  for (int r = 0; r < world; ++r) {
    if (arenas[r] == nullptr) return PK_ERR_BAD_ARG;
    p.slot_base[r] = (float*)arenas[r];
  }
  p.world = world;
  p.rank = rank;
  p.capacity = capacity;
  p.timeout_us = timeout_us;
  p.in = nullptr;
  p.out = out;
  p.n = n;
  p.ybuf = ybuf;
  p.route_w = route_w;
  p.route_pos = route_pos;
  p.seg = seg;
  p.topk = topk;
  p.H = H;
  p.expert_offset = expert_offset;
  p.local_experts = local_experts;
  const size_t want = (n / 4 + 255) / 256;
  const int cap = sm_count > 0 ? sm_count : 148;
  const int grid = (int)(want < (size_t)cap ? (want ? want : 1) : (size_t)cap);
  peer_allreduce_kernel<<<grid, 256, 0, stream>>>(p);
  PK_CHECK_LAUNCH();
  return PK_OK;
}

// Peer-memory signalling used by fused compute+collective kernels.
//
// Contract (the bounded-wait + status-word contract of the reference's CUDA-IPC
// all-reduce, src/csrc/cuda_kernel_impl.cu:4788-4829, with its multi-block defects
// fixed): a producer kernel stores its partial result into every peer's slot buffer,
// every block fences, the LAST block to finish publishes `flag[peer][my_rank] = seq`
// with release semantics at system scope. A consumer kernel's blocks each poll their
// own GPU's flag words with acquire loads until all ranks reached `seq` or a time
// budget runs out; on expiry the kernel records PK_COMM_TIMEOUT in a status word and
// carries on with whatever data is there (the host checks the word after the step and
// falls back to NCCL or raises). Nothing ever spins without a limit.
#pragma once

#include <stdint.h>

#include "pk_common.cuh"

#include "pk_comm_types.h"

namespace pk {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Publishing a sequence number to every rank: ONE system fence, then one relaxed store per rank. A release store per
// rank would wait for the acknowledgement of the store before it (a round trip over NVLink each): at eight ranks that
// was most of the latency of a small all-reduce. The fence followed by relaxed stores is the same release pattern.
__device__ __forceinline__ void publish_seq(uint32_t* const* flag, int world, int rank, uint32_t seq) {
  __threadfence_system();
  for (int r = 0; r < world; ++r) st_relaxed_sys(flag[r] + rank, seq);
}

// One polling round over the `world` words at `flag`: the loads are issued together, then compared. True when every
// word has reached `target` (sequence numbers only grow; a later one also satisfies the wait). The caller runs
// __threadfence_system() after the round that succeeded (relaxed loads + fence = acquire).
__device__ __forceinline__ bool all_reached(const uint32_t* flag, int world, uint32_t target) {
  uint32_t v[PK_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < PK_MAX_RANKS; ++r) v[r] = r < world ? ld_relaxed_sys(flag + r) : target;
  bool all = true;
#pragma unroll
  for (int r = 0; r < PK_MAX_RANKS; ++r) all = all && (int32_t)(v[r] - target) >= 0;
  return all;
}

__device__ __forceinline__ uint32_t comm_seq(const uint32_t* epoch, uint32_t sites, uint32_t site) {
  return (*((const volatile uint32_t*)epoch)) * sites + site + 1u;
}

// Called by ONE thread of a block. Returns false if the budget ran out.
__device__ __forceinline__ bool wait_all_ranks(const PkWait& w) {
  if (w.flag == nullptr || w.world <= 1) return true;
  // Once a wait of this step has given up, later waits return at once: the step is lost
  // anyway and the kernels only have to drain.
  if (*((volatile uint32_t*)w.status) != 0u) return false;
  const uint32_t target = comm_seq(w.epoch, w.sites_per_epoch, w.site);
  const uint64_t t0 = global_timer_ns();
  const uint64_t budget = (uint64_t)w.timeout_us * 1000ull;
  while (!all_reached(w.flag, w.world, target)) {
    if (global_timer_ns() - t0 > budget) {
      atomicExch(w.status, PK_COMM_TIMEOUT);
      return false;
    }
    __nanosleep(40);
  }
  __threadfence_system();
  return true;
}

// Called by every thread of every block after its last store of the producer kernel.
__device__ __forceinline__ void publish_when_grid_done(const PkPush& p) {
  if (p.world <= 1 && p.flag[0] == nullptr) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t nblocks = gridDim.x * gridDim.y * gridDim.z;
    const uint32_t done = atomicAdd(p.block_counter, 1u) + 1u;
    if (done == nblocks) {
      *p.block_counter = 0u;  // ready for the next launch (stream-ordered)
      publish_seq(p.flag, p.world, p.rank, comm_seq(p.epoch, p.sites_per_epoch, p.site));
    }
  }
}

// Variant for kernels whose threads already ran __threadfence_system() after their last
// store and met at a block barrier: called by ONE thread of each block.
__device__ __forceinline__ void publish_after_block_sync(const PkPush& p) {
  if (p.world <= 1 && p.flag[0] == nullptr) return;
  const uint32_t nblocks = gridDim.x * gridDim.y * gridDim.z;
  const uint32_t done = atomicAdd(p.block_counter, 1u) + 1u;
  if (done == nblocks) {
    *p.block_counter = 0u;
    publish_seq(p.flag, p.world, p.rank, comm_seq(p.epoch, p.sites_per_epoch, p.site));
  }
}

}  // namespace pk

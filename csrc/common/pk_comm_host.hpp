// Host model of the peer-memory all-reduce protocol (two slot sets, per-rank sequence flags, bounded waits,
// status word), with std::atomic in place of system-scope loads and stores and threads in place of GPUs.
// The rules are the ones of csrc/comm/peer_allreduce.cu: push into slot[seq & 1][my_rank] of every rank,
// publish flag[seq & 1][my_rank] = seq with release order, wait with acquire loads under a time budget until
// all ranks reached seq, sum, advance seq. Compiled for the host so that ordering mistakes, flag reuse and
// time-outs can be unit-tested (also under ThreadSanitizer) without a GPU.
#pragma once

#include <atomic>
#include <chrono>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

namespace pk {

struct HostArena {
  HostArena(int world, size_t capacity) : world(world), capacity(capacity), slots((size_t)2 * world * capacity), flags(2 * world) {
    for (auto& f : flags) f.store(0);
  }
  int world;
  size_t capacity;
  std::vector<float> slots;                       // [2][world][capacity]
  std::vector<std::atomic<uint32_t>> flags;       // [2][world]
  uint32_t seq = 0;
  std::atomic<uint32_t> status{0};
  float* slot(int parity, int r) { return slots.data() + ((size_t)parity * world + r) * capacity; }
};

// One call of rank `rank`. Returns false when the wait ran out (status is set, out is unspecified).
inline bool host_allreduce(std::vector<HostArena*>& arenas, int rank, const float* in, float* out, size_t n, int timeout_ms) {
  HostArena& mine = *arenas[rank];
  const int world = mine.world;
  const uint32_t seq = mine.seq + 1;
  const int parity = (int)(seq & 1u);
  for (int r = 0; r < world; ++r) {
    float* dst = arenas[r]->slot(parity, rank);
    for (size_t i = 0; i < n; ++i) dst[i] = in[i];
  }
  for (int r = 0; r < world; ++r) arenas[r]->flags[parity * world + rank].store(seq, std::memory_order_release);
  bool ok = mine.status.load() == 0;
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; ok && r < world; ++r) {
    while ((int32_t)(mine.flags[parity * world + r].load(std::memory_order_acquire) - seq) < 0) {
      if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) {
        mine.status.store(1);
        ok = false;
        break;
      }
      std::this_thread::yield();
    }
  }
  if (ok) {
    for (size_t i = 0; i < n; ++i) {
      float a = 0.f;
      for (int r = 0; r < world; ++r) a += mine.slot(parity, r)[i];
      out[i] = a;
    }
  }
  mine.seq = seq;
  return ok;
}

// Host model of the block counters of one launch of the peer all-reduce kernel. Every block makes two
// announcements: "my part is stored" (first pass) and "I am done reading" (second pass). The flag may be published
// only when EVERY block has stored. `two_counters == false` models a single shared counter compared against the
// grid size: a block that skips its wait (the status word was already set) can make its second announcement before
// another block's first, and the count reaches the grid size too early. Returns the number of blocks that had
// stored when the publish decision fired, or -1 when it never fired.
struct BlockEvent { int block; int pass; };   // pass 1 or 2, in the order the atomics are served
inline int stored_at_publish(int grid, const std::vector<BlockEvent>& order, bool two_counters) {
  int pushed = 0, left = 0, shared = 0, stored = 0;
  for (const BlockEvent& e : order) {
    if (e.pass == 1) ++stored;
    if (two_counters) {
      if (e.pass == 1) { if (++pushed == grid) return stored; }
      else ++left;
    } else {
      if (++shared == grid && e.pass == 1) return stored;   // the kernel publishes from the first-pass increment only
    }
  }
  (void)left;
  return -1;
}


}  // namespace pk

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

// Host model of the in-switch all-reduce (csrc/comm/multimem_allreduce.cu): every rank owns data[2][capacity] and
// flags[2][2][world]; `multimem.ld_reduce` is modelled as a read of the same element of every rank's buffer and
// `multimem.st` as a write of one value into every rank's buffer. One shot: write own data, publish, wait, read the sum
// of everything. Two shot: write own data, publish, wait, reduce this rank's slice and store it into EVERY rank's data
// set in place, publish the second flag, wait, copy out of the own data set. Run under ThreadSanitizer this checks that
// no rank writes a buffer another rank may still read (two data sets, in-place broadcast of disjoint slices, calls of
// both kinds mixed).
struct HostMmBuffer {
  HostMmBuffer(int world, size_t capacity) : world(world), capacity(capacity), data((size_t)2 * capacity), flags(4 * world) {
    for (auto& f : flags) f.store(0);
  }
  int world;
  size_t capacity;
  std::vector<float> data;                        // [2][capacity]
  std::vector<std::atomic<uint32_t>> flags;       // [2][2][world]
  uint32_t seq = 0;
  std::atomic<uint32_t> status{0};
};

inline bool host_mm_wait(HostMmBuffer& mine, int parity, int round, uint32_t seq, int timeout_ms) {
  if (mine.status.load() != 0) return false;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    bool all = true;
    // one polling round over all flags (the device polls relaxed and fences once; acquire loads are the same ordering
    // in a form ThreadSanitizer can follow: it does not model stand-alone fences)
    for (int r = 0; r < mine.world; ++r)
      all = all && (int32_t)(mine.flags[(parity * 2 + round) * mine.world + r].load(std::memory_order_acquire) - seq) >= 0;
    if (all) break;
    if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) {
      mine.status.store(1);
      return false;
    }
    std::this_thread::yield();
  }
  return true;
}

inline void host_mm_publish(std::vector<HostMmBuffer*>& bufs, int rank, int parity, int round, uint32_t seq) {
  // the device runs one system fence and then relaxed stores; release stores are the same ordering
  for (HostMmBuffer* b : bufs) b->flags[(parity * 2 + round) * b->world + rank].store(seq, std::memory_order_release);
}

inline bool host_mm_allreduce(std::vector<HostMmBuffer*>& bufs, int rank, const float* in, float* out, size_t n, bool two_shot,
                              int timeout_ms) {
  HostMmBuffer& mine = *bufs[rank];
  const int world = mine.world;
  const uint32_t seq = mine.seq + 1;
  const int parity = (int)(seq & 1u);
  float* data = mine.data.data() + (size_t)parity * mine.capacity;
  for (size_t i = 0; i < n; ++i) data[i] = in[i];
  host_mm_publish(bufs, rank, parity, 0, seq);
  bool ok = host_mm_wait(mine, parity, 0, seq, timeout_ms);
  if (ok && !two_shot) {
    for (size_t i = 0; i < n; ++i) {
      float a = 0.f;
      for (int r = 0; r < world; ++r) a += bufs[r]->data[(size_t)parity * bufs[r]->capacity + i];
      out[i] = a;
    }
  } else if (ok) {
    const size_t per = (n + world - 1) / world, lo = (size_t)rank * per, hi = lo + per < n ? lo + per : n;
    for (size_t i = lo; i < hi; ++i) {
      float a = 0.f;
      for (int r = 0; r < world; ++r) a += bufs[r]->data[(size_t)parity * bufs[r]->capacity + i];
      for (int r = 0; r < world; ++r) bufs[r]->data[(size_t)parity * bufs[r]->capacity + i] = a;
    }
    host_mm_publish(bufs, rank, parity, 1, seq);
    ok = host_mm_wait(mine, parity, 1, seq, timeout_ms);
    if (ok)
      for (size_t i = 0; i < n; ++i) out[i] = data[i];
  }
  mine.seq = seq;
  return ok;
}

}  // namespace pk

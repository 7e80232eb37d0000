// Host-to-device staging for weights that live in host memory (experts beyond what stays resident):
//   LruSlotMap         which key (expert id) sits in which of n device slots; keys of the current step are never
//                      evicted for one another (pure bookkeeping, no CUDA)
//   PinnedStagingRing  page-locked bounce slots with one event each: copy pageable bytes into a free slot, then an
//                      asynchronous copy to the device on the caller's stream; a slot is reused once its copy is done
//   ExpertSlotArena    device slots + LruSlotMap + ring: `ensure(keys)` makes the needed experts resident and returns
//                      their device addresses
// Counterparts in the reference: GgufPinnedStagingRing, DeviceFp4ActiveArena / HostFp4ExpertSlot
// (cpp_engine/src/dsv4_engine.cpp:1432-1569). The Python twin is pocketllm_b200/moe/expert_cache.py.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <list>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pk {

class LruSlotMap {
 public:
  explicit LruSlotMap(int slots);
  // Slot of every needed key (same order, duplicates allowed) and the (key, slot) pairs whose contents must be loaded.
  // Throws std::runtime_error when the distinct keys outnumber the slots.
  std::vector<int> assign(const std::vector<long long>& needed, std::vector<std::pair<long long, int>>* loads);
  int slots() const { return n_; }
  int resident() const { return (int)where_.size(); }
  bool contains(long long key) const { return where_.count(key) != 0; }
  long long hits = 0, misses = 0, evictions = 0;

 private:
  int n_;
  std::list<long long> order_;   // least recently used first
  std::unordered_map<long long, std::pair<int, std::list<long long>::iterator>> where_;
  std::vector<int> free_;
};

class PinnedStagingRing {
 public:
  PinnedStagingRing(int slots, size_t slot_bytes);
  ~PinnedStagingRing();
  PinnedStagingRing(const PinnedStagingRing&) = delete;
  PinnedStagingRing& operator=(const PinnedStagingRing&) = delete;
  // Copies `bytes` (<= slot_bytes) from pageable host memory to `dst_device` through the next slot; returns the slot.
  int stage(const void* src_host, size_t bytes, void* dst_device, cudaStream_t stream);
  void drain();   // wait for every copy in flight
  int slots() const { return (int)host_.size(); }
  size_t slot_bytes() const { return slot_bytes_; }
  long long waits = 0;   // times stage() had to wait for a slot's previous copy

 private:
  size_t slot_bytes_;
  std::vector<void*> host_;
  std::vector<cudaEvent_t> done_;
  std::vector<bool> used_;
  int next_ = 0;
};

class ExpertSlotArena {
 public:
  ExpertSlotArena(int device_slots, size_t expert_bytes, int ring_slots);
  ~ExpertSlotArena();
  ExpertSlotArena(const ExpertSlotArena&) = delete;
  ExpertSlotArena& operator=(const ExpertSlotArena&) = delete;
  // Host copy of the experts: `base + key * expert_bytes` is expert `key`.
  void set_host_store(const void* base, long long n_experts);
  // Makes every needed expert resident (copies ordered on `stream`) and writes its device address to out_ptrs[i].
  void ensure(const long long* keys, int n, void** out_ptrs, cudaStream_t stream);
  const LruSlotMap& map() const { return map_; }
  const PinnedStagingRing& ring() const { return ring_; }
  long long bytes_copied = 0;

 private:
  size_t expert_bytes_;
  LruSlotMap map_;
  PinnedStagingRing ring_;
  void* device_ = nullptr;
  const uint8_t* host_base_ = nullptr;
  long long n_experts_ = 0;
};

}  // namespace pk

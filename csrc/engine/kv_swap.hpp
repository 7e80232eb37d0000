// Host tier of a layer's compressed KV cache for contexts whose cache does not fit the device: every compressed row
// lives in page-locked host memory; the device holds `device_slots` rows. Per decode step the indexer's selection is
// made resident: rows already on the device are hits, the others are packed into a pinned bounce buffer, copied with
// ONE host-to-device transfer and scattered into least-recently-used slots by a kernel, and the selection is rewritten
// to physical rows (`window + slot`, the slots sit behind the layer's window rows in the attention kernel's KV array).
// Rows selected in the same step are never evicted for one another.
//
// Counterpart of the reference's GgufKvSwapLayerState / gguf_kv_swap_in_selected
// (cpp_engine/src/dsv4_engine.cpp:5260-5434), which copies one row per cudaMemcpyAsync.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <vector>

#include "staging.hpp"

namespace pk {

struct KvSwapStats {
  uint64_t hits = 0, misses = 0, h2d_bytes = 0, d2h_bytes = 0, evictions = 0, steps = 0;
};

class KvSwapTier {
 public:
  // capacity: logical rows the host store can hold; device_slots: rows resident at once (clamped to capacity);
  // row_bytes: bytes of one compressed row (a multiple of 16); window: first physical row of slot 0.
  // host_only: "device" pointers are host pointers and copies are memcpy (tests without a GPU).
  KvSwapTier(int capacity, int device_slots, size_t row_bytes, int window, bool host_only);
  ~KvSwapTier();
  KvSwapTier(const KvSwapTier&) = delete;
  KvSwapTier& operator=(const KvSwapTier&) = delete;

  // `count` new rows (logical ids first .. first + count) produced on the device at `rows_device`: copied to the host
  // store (the tier is write-through, a row is never lost when its slot is reused). Synchronises `stream`.
  void store(int first, int count, const void* rows_device, cudaStream_t stream);
  // Make the selected logical rows (`selected_device`, n int32 ids on the device, -1 = no row) resident in `pool_device`
  // ([device_slots][row_bytes]) and write their physical rows to `physical_device` (n int32). Throws std::runtime_error
  // when the distinct rows outnumber the slots or a row was never stored. Synchronises `stream` once (to read the ids).
  void swap_in(const int* selected_device, int n, void* pool_device, int* physical_device, cudaStream_t stream);
  void reset();                                // forget every row and slot (new sequence)
  const KvSwapStats& stats() const { return stats_; }
  int capacity() const { return capacity_; }
  int device_slots() const { return slots_; }
  int stored_rows() const { return stored_; }
  size_t host_bytes() const { return (size_t)capacity_ * row_bytes_; }

 private:
  int capacity_, slots_, window_;
  size_t row_bytes_;
  bool host_only_;
  uint8_t* host_ = nullptr;        // [capacity][row_bytes] pinned
  uint8_t* bounce_ = nullptr;      // [device_slots][row_bytes] pinned: this step's misses, packed
  int* ids_host_ = nullptr;        // pinned: selection in, physical rows out
  int ids_cap_ = 0;
  uint8_t* bounce_dev_ = nullptr;  // device twin of bounce_
  int* slot_ids_dev_ = nullptr;    // [device_slots] destination slot of every packed miss
  int* slot_ids_host_ = nullptr;   // pinned
  std::vector<uint8_t> ready_;     // per logical row: stored on the host
  int stored_ = 0;
  LruSlotMap lru_;
  KvSwapStats stats_;
  void ensure_ids(int n);
};

}  // namespace pk

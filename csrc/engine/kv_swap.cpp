#include "kv_swap.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>

#include "pk_kernels.h"

namespace pk {

namespace {
void ck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("kv swap: ") + what + ": " + cudaGetErrorString(e));
}
}  // namespace

KvSwapTier::KvSwapTier(int capacity, int device_slots, size_t row_bytes, int window, bool host_only)
    : capacity_(capacity), slots_(std::min(device_slots, capacity)), window_(window), row_bytes_(row_bytes), host_only_(host_only),
      lru_(std::max(std::min(device_slots, capacity), 1)) {
  if (capacity < 1 || device_slots < 1 || row_bytes < 16 || (row_bytes & 15) != 0 || window < 0)
    throw std::runtime_error("kv swap: capacity and slots must be positive, row_bytes a positive multiple of 16, window >= 0");
  const size_t host_bytes = (size_t)capacity_ * row_bytes_, bounce_bytes = (size_t)slots_ * row_bytes_;
  if (host_only_) {
    host_ = new uint8_t[host_bytes];
    bounce_ = new uint8_t[bounce_bytes];
    bounce_dev_ = new uint8_t[bounce_bytes];
    slot_ids_host_ = new int[slots_];
    slot_ids_dev_ = new int[slots_];
  } else {
    ck(cudaMallocHost((void**)&host_, host_bytes), "pinned store");
    ck(cudaMallocHost((void**)&bounce_, bounce_bytes), "pinned bounce");
    ck(cudaMallocHost((void**)&slot_ids_host_, (size_t)slots_ * sizeof(int)), "pinned slot ids");
    ck(cudaMalloc((void**)&bounce_dev_, bounce_bytes), "device bounce");
    ck(cudaMalloc((void**)&slot_ids_dev_, (size_t)slots_ * sizeof(int)), "device slot ids");
  }
  ready_.assign((size_t)capacity_, 0);
}

KvSwapTier::~KvSwapTier() {
  if (host_only_) {
    delete[] host_;
    delete[] bounce_;
    delete[] bounce_dev_;
    delete[] slot_ids_host_;
    delete[] slot_ids_dev_;
    delete[] ids_host_;
  } else {
    if (host_) cudaFreeHost(host_);
    if (bounce_) cudaFreeHost(bounce_);
    if (slot_ids_host_) cudaFreeHost(slot_ids_host_);
    if (ids_host_) cudaFreeHost(ids_host_);
    if (bounce_dev_) cudaFree(bounce_dev_);
    if (slot_ids_dev_) cudaFree(slot_ids_dev_);
  }
}

void KvSwapTier::ensure_ids(int n) {
  if (n <= ids_cap_) return;
  const int cap = std::max(n, 2 * ids_cap_);
  if (host_only_) {
    delete[] ids_host_;
    ids_host_ = new int[cap];
  } else {
    if (ids_host_) cudaFreeHost(ids_host_);
    ids_host_ = nullptr;
    ck(cudaMallocHost((void**)&ids_host_, (size_t)cap * sizeof(int)), "pinned ids");
  }
  ids_cap_ = cap;
}

void KvSwapTier::reset() {
  std::fill(ready_.begin(), ready_.end(), 0);
  stored_ = 0;
  lru_ = LruSlotMap(slots_);
  stats_ = KvSwapStats();
}

void KvSwapTier::store(int first, int count, const void* rows_device, cudaStream_t stream) {
  if (count < 1) return;
  if (first < 0 || (long long)first + count > capacity_) throw std::runtime_error("kv swap: row outside the host store");
  // A device slot keeps a row's contents from the time it was loaded, so a resident row must not change underneath it.
  // Compressed rows are append-only; rewriting one that is resident is a caller error.
  for (int i = 0; i < count; ++i)
    if (lru_.contains(first + i)) throw std::runtime_error("kv swap: row " + std::to_string(first + i) + " is resident and cannot be rewritten");
  const size_t bytes = (size_t)count * row_bytes_;
  uint8_t* dst = host_ + (size_t)first * row_bytes_;
  if (host_only_) {
    memcpy(dst, rows_device, bytes);
  } else {
    ck(cudaMemcpyAsync(dst, rows_device, bytes, cudaMemcpyDeviceToHost, stream), "store");
    ck(cudaStreamSynchronize(stream), "store sync");
  }
  for (int i = 0; i < count; ++i) {
    if (!ready_[(size_t)first + i]) ++stored_;
    ready_[(size_t)first + i] = 1;
  }
  stats_.d2h_bytes += bytes;
}

void KvSwapTier::swap_in(const int* selected_device, int n, void* pool_device, int* physical_device, cudaStream_t stream) {
  if (n < 1) return;
  ensure_ids(n);
  if (host_only_) {
    memcpy(ids_host_, selected_device, (size_t)n * sizeof(int));
  } else {
    ck(cudaMemcpyAsync(ids_host_, selected_device, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, stream), "selection");
    ck(cudaStreamSynchronize(stream), "selection sync");
  }
  std::vector<long long> needed;
  needed.reserve((size_t)n);
  for (int i = 0; i < n; ++i) {
    const int id = ids_host_[i];
    if (id < 0) continue;
    if (id >= capacity_ || !ready_[(size_t)id]) throw std::runtime_error("kv swap: selected row " + std::to_string(id) + " was never stored");
    needed.push_back(id);
  }
  std::vector<std::pair<long long, int>> loads;
  const long long ev0 = lru_.evictions, hit0 = lru_.hits, miss0 = lru_.misses;
  const std::vector<int> slots = lru_.assign(needed, &loads);   // throws when the distinct rows outnumber the slots
  stats_.evictions += (uint64_t)(lru_.evictions - ev0);
  stats_.hits += (uint64_t)(lru_.hits - hit0);
  stats_.misses += (uint64_t)(lru_.misses - miss0);
  ++stats_.steps;
  const int m = (int)loads.size();
  for (int j = 0; j < m; ++j) {
    memcpy(bounce_ + (size_t)j * row_bytes_, host_ + (size_t)loads[j].first * row_bytes_, row_bytes_);
    slot_ids_host_[j] = loads[j].second;
  }
  size_t k = 0;
  for (int i = 0; i < n; ++i) ids_host_[i] = ids_host_[i] < 0 ? -1 : window_ + slots[k++];
  if (host_only_) {
    for (int j = 0; j < m; ++j) memcpy((uint8_t*)pool_device + (size_t)slot_ids_host_[j] * row_bytes_, bounce_ + (size_t)j * row_bytes_, row_bytes_);
    memcpy(physical_device, ids_host_, (size_t)n * sizeof(int));
  } else {
    if (m > 0) {
      ck(cudaMemcpyAsync(bounce_dev_, bounce_, (size_t)m * row_bytes_, cudaMemcpyHostToDevice, stream), "misses");
      ck(cudaMemcpyAsync(slot_ids_dev_, slot_ids_host_, (size_t)m * sizeof(int), cudaMemcpyHostToDevice, stream), "slot ids");
      if (pk_scatter_rows(bounce_dev_, slot_ids_dev_, m, (int)row_bytes_, pool_device, stream) != 0) throw std::runtime_error("kv swap: scatter kernel failed");
    }
    ck(cudaMemcpyAsync(physical_device, ids_host_, (size_t)n * sizeof(int), cudaMemcpyHostToDevice, stream), "physical rows");
    // the pinned buffers are reused by the next call
    ck(cudaStreamSynchronize(stream), "swap-in sync");
  }
  stats_.h2d_bytes += (size_t)m * row_bytes_;
}

}  // namespace pk

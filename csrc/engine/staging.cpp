#include "staging.hpp"

#include <unordered_set>

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>

namespace pk {

namespace {
void ck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
}  // namespace

// ---- LruSlotMap ----

LruSlotMap::LruSlotMap(int slots) : n_(slots) {
  if (slots < 1) throw std::runtime_error("LruSlotMap: at least one slot");
  for (int s = slots - 1; s >= 0; --s) free_.push_back(s);
}

std::vector<int> LruSlotMap::assign(const std::vector<long long>& needed, std::vector<std::pair<long long, int>>* loads) {
  std::vector<long long> uniq;
  std::unordered_set<long long> in_step;
  for (long long k : needed)
    if (in_step.insert(k).second) uniq.push_back(k);
  if ((int)uniq.size() > n_)
    throw std::runtime_error(std::to_string(uniq.size()) + " distinct keys do not fit in " + std::to_string(n_) + " slots; split the step into waves");
  // touch the residents first so that none of them is the eviction victim of another key of this step
  for (long long k : uniq) {
    auto it = where_.find(k);
    if (it == where_.end()) continue;
    order_.erase(it->second.second);
    order_.push_back(k);
    it->second.second = std::prev(order_.end());
    ++hits;
  }
  for (long long k : uniq) {
    if (where_.count(k)) continue;
    ++misses;
    int slot;
    if (!free_.empty()) {
      slot = free_.back();
      free_.pop_back();
    } else {
      auto victim = order_.begin();
      while (victim != order_.end() && in_step.count(*victim) != 0) ++victim;
      if (victim == order_.end()) throw std::runtime_error("LruSlotMap: no evictable slot");
      slot = where_[*victim].first;
      where_.erase(*victim);
      order_.erase(victim);
      ++evictions;
    }
    order_.push_back(k);
    where_[k] = {slot, std::prev(order_.end())};
    if (loads) loads->push_back({k, slot});
  }
  std::vector<int> out;
  out.reserve(needed.size());
  for (long long k : needed) out.push_back(where_[k].first);
  return out;
}

// ---- PinnedStagingRing ----

PinnedStagingRing::PinnedStagingRing(int slots, size_t slot_bytes) : slot_bytes_(slot_bytes) {
  if (slots < 1 || slot_bytes == 0) throw std::runtime_error("PinnedStagingRing: slots and slot_bytes must be positive");
  for (int i = 0; i < slots; ++i) {
    void* p = nullptr;
    ck(cudaHostAlloc(&p, slot_bytes, cudaHostAllocDefault), "cudaHostAlloc");
    host_.push_back(p);
    cudaEvent_t e;
    ck(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    done_.push_back(e);
    used_.push_back(false);
  }
}

PinnedStagingRing::~PinnedStagingRing() {
  for (size_t i = 0; i < host_.size(); ++i) {
    if (used_[i]) cudaEventSynchronize(done_[i]);
    cudaEventDestroy(done_[i]);
    cudaFreeHost(host_[i]);
  }
}

int PinnedStagingRing::stage(const void* src_host, size_t bytes, void* dst_device, cudaStream_t stream) {
  if (bytes > slot_bytes_) throw std::runtime_error("PinnedStagingRing: request larger than a slot");
  const int s = next_;
  next_ = (next_ + 1) % (int)host_.size();
  if (used_[s]) {
    if (cudaEventQuery(done_[s]) == cudaErrorNotReady) ++waits;
    ck(cudaEventSynchronize(done_[s]), "staging slot wait");
  }
  std::memcpy(host_[s], src_host, bytes);
  ck(cudaMemcpyAsync(dst_device, host_[s], bytes, cudaMemcpyHostToDevice, stream), "staging copy");
  ck(cudaEventRecord(done_[s], stream), "staging event");
  used_[s] = true;
  return s;
}

void PinnedStagingRing::drain() {
  for (size_t i = 0; i < host_.size(); ++i)
    if (used_[i]) ck(cudaEventSynchronize(done_[i]), "staging drain");
}

// ---- ExpertSlotArena ----

ExpertSlotArena::ExpertSlotArena(int device_slots, size_t expert_bytes, int ring_slots)
    : expert_bytes_(expert_bytes), map_(device_slots), ring_(ring_slots, expert_bytes) {
  ck(cudaMalloc(&device_, (size_t)device_slots * expert_bytes), "expert arena");
}

ExpertSlotArena::~ExpertSlotArena() {
  ring_.drain();
  cudaFree(device_);
}

void ExpertSlotArena::set_host_store(const void* base, long long n_experts) {
  host_base_ = (const uint8_t*)base;
  n_experts_ = n_experts;
}

void ExpertSlotArena::ensure(const long long* keys, int n, void** out_ptrs, cudaStream_t stream) {
  if (host_base_ == nullptr) throw std::runtime_error("ExpertSlotArena: no host store");
  std::vector<long long> needed(keys, keys + n);
  for (long long k : needed)
    if (k < 0 || k >= n_experts_) throw std::runtime_error("ExpertSlotArena: expert " + std::to_string(k) + " out of range");
  std::vector<std::pair<long long, int>> loads;
  const std::vector<int> slots = map_.assign(needed, &loads);
  for (const auto& l : loads) {
    ring_.stage(host_base_ + (size_t)l.first * expert_bytes_, expert_bytes_, (uint8_t*)device_ + (size_t)l.second * expert_bytes_, stream);
    bytes_copied += (long long)expert_bytes_;
  }
  for (int i = 0; i < n; ++i) out_ptrs[i] = (uint8_t*)device_ + (size_t)slots[i] * expert_bytes_;
}

}  // namespace pk

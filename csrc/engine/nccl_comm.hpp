// NCCL as the baseline / fallback collective path of the native side: one communicator per (world, rank, device, id
// path), created from a unique id that rank 0 publishes through the file rendezvous. The library is opened at run time
// (dlopen of libnccl.so.2), so the engine keeps no link-time dependency on it and shares the copy a host process has
// already loaded. Counterpart of the reference's cpp_engine/src/tp_comm.cpp:40-269 (id rendezvous, communicator cache,
// all-reduce fp32 / fp16 / bf16, int32 broadcast, all-gather, global top-1), with the collectives on the caller's
// stream instead of the NULL stream.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace pk {

class NcclComm {
 public:
  enum class Dtype { F32, F16, BF16, I32 };
  static bool available();   // the library and its entry points were found
  // Blocks until all `world` ranks have joined (file rendezvous under id_path; timeout_ms bounds the wait).
  NcclComm(const std::string& id_path, int rank, int world, int device, int timeout_ms = 600000);
  ~NcclComm();
  NcclComm(const NcclComm&) = delete;
  NcclComm& operator=(const NcclComm&) = delete;

  void all_reduce_sum(void* buf, size_t count, Dtype dt, cudaStream_t stream);            // in place
  void broadcast(void* buf, size_t count, Dtype dt, int root, cudaStream_t stream);       // in place
  void all_gather(const void* send, void* recv, size_t count_per_rank, Dtype dt, cudaStream_t stream);
  // Greedy pick over vocabulary shards: every rank passes its best {logit, token}; returns the winner (lowest token on ties).
  // Synchronises the stream.
  int global_top1(float local_logit, int local_token, cudaStream_t stream, float* best_logit = nullptr);
  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
  int rank_, world_;
};

}  // namespace pk

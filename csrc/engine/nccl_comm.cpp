#include "nccl_comm.hpp"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <stdexcept>

#include "control_plane.hpp"

namespace pk {

namespace {

struct Api {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      a.lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (a.lib) break;
    }
    if (!a.lib) return;
    auto sym = [&](const char* n) { return dlsym(a.lib, n); };
    a.GetUniqueId = (decltype(a.GetUniqueId))sym("ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))sym("ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))sym("ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))sym("ncclAllReduce");
    a.Broadcast = (decltype(a.Broadcast))sym("ncclBroadcast");
    a.AllGather = (decltype(a.AllGather))sym("ncclAllGather");
    a.GetErrorString = (decltype(a.GetErrorString))sym("ncclGetErrorString");
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.Broadcast && a.AllGather && a.GetErrorString;
  });
  return a;
}

void check(ncclResult_t r, const char* what) {
  if (r != ncclSuccess) throw std::runtime_error(std::string(what) + ": " + api().GetErrorString(r));
}

ncclDataType_t nccl_type(NcclComm::Dtype dt) {
  switch (dt) {
    case NcclComm::Dtype::F32: return ncclFloat32;
    case NcclComm::Dtype::F16: return ncclFloat16;
    case NcclComm::Dtype::BF16: return ncclBfloat16;
    default: return ncclInt32;
  }
}

}  // namespace

struct NcclComm::Impl {
  ncclComm_t comm = nullptr;
  int device = 0;
  float* pair_send = nullptr;   // {logit, token as float bits} for global_top1
  float* pair_recv = nullptr;
};

bool NcclComm::available() { return api().ok; }

NcclComm::NcclComm(const std::string& id_path, int rank, int world, int device, int timeout_ms) : impl_(new Impl), rank_(rank), world_(world) {
  if (!api().ok) throw std::runtime_error("NCCL library not found (libnccl.so.2)");
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("NcclComm: bad rank / world");
  impl_->device = device;
  if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("NcclComm: cudaSetDevice failed");
  ncclUniqueId id;
  std::memset(&id, 0, sizeof id);
  std::vector<uint8_t> blob;
  if (rank == 0) {
    check(api().GetUniqueId(&id), "ncclGetUniqueId");
    blob.assign((const uint8_t*)&id, (const uint8_t*)&id + sizeof id);
  }
  if (world > 1) {
    // every rank publishes a blob of the same size; only rank 0's carries the id
    blob.resize(sizeof id, 0);
    const auto all = file_rendezvous(id_path + ".ncclid", rank, world, blob, timeout_ms);
    std::memcpy(&id, all[0].data(), sizeof id);
  }
  check(api().CommInitRank(&impl_->comm, world, id, rank), "ncclCommInitRank");
  if (world > 1) file_rendezvous_cleanup(id_path + ".ncclid", rank);
  cudaMalloc((void**)&impl_->pair_send, 2 * sizeof(float));
  cudaMalloc((void**)&impl_->pair_recv, (size_t)2 * world * sizeof(float));
}

NcclComm::~NcclComm() {
  if (impl_->comm) api().CommDestroy(impl_->comm);
  cudaFree(impl_->pair_send);
  cudaFree(impl_->pair_recv);
}

void NcclComm::all_reduce_sum(void* buf, size_t count, Dtype dt, cudaStream_t stream) {
  check(api().AllReduce(buf, buf, count, nccl_type(dt), ncclSum, impl_->comm, stream), "ncclAllReduce");
}

void NcclComm::broadcast(void* buf, size_t count, Dtype dt, int root, cudaStream_t stream) {
  check(api().Broadcast(buf, buf, count, nccl_type(dt), root, impl_->comm, stream), "ncclBroadcast");
}

void NcclComm::all_gather(const void* send, void* recv, size_t count_per_rank, Dtype dt, cudaStream_t stream) {
  check(api().AllGather(send, recv, count_per_rank, nccl_type(dt), impl_->comm, stream), "ncclAllGather");
}

int NcclComm::global_top1(float local_logit, int local_token, cudaStream_t stream, float* best_logit) {
  float pair[2];
  pair[0] = local_logit;
  std::memcpy(&pair[1], &local_token, sizeof(int));
  if (cudaMemcpyAsync(impl_->pair_send, pair, sizeof pair, cudaMemcpyHostToDevice, stream) != cudaSuccess) throw std::runtime_error("global_top1: h2d");
  all_gather(impl_->pair_send, impl_->pair_recv, 2, Dtype::F32, stream);
  std::vector<float> all((size_t)2 * world_);
  if (cudaMemcpyAsync(all.data(), impl_->pair_recv, all.size() * sizeof(float), cudaMemcpyDeviceToHost, stream) != cudaSuccess) throw std::runtime_error("global_top1: d2h");
  if (cudaStreamSynchronize(stream) != cudaSuccess) throw std::runtime_error("global_top1: sync");
  float best = all[0];
  int tok;
  std::memcpy(&tok, &all[1], sizeof(int));
  for (int r = 1; r < world_; ++r) {
    int t;
    std::memcpy(&t, &all[2 * r + 1], sizeof(int));
    if (all[2 * r] > best || (all[2 * r] == best && t < tok)) {
      best = all[2 * r];
      tok = t;
    }
  }
  if (best_logit) *best_logit = best;
  return tok;
}

}  // namespace pk

// Host control plane of the native engine: a file rendezvous that exchanges small blobs
// (CUDA IPC handles of the peer-memory arenas) between the rank processes, and a
// Unix-domain command channel on which rank 0 drives idle workers.
//
// Same roles as the reference's NCCL-id file poll (cpp_engine/src/tp_comm.cpp:40-73) and
// CmdChannel (cpp_engine/include/cmd_channel.hpp:10-40, src/cmd_channel.cpp:72-173), but
// nothing here touches a GPU: the collectives themselves run inside the kernels.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace pk {

// Every rank publishes `blob` under `base_path` and collects the blobs of all ranks.
// Files are written atomically (temp + rename). Throws std::runtime_error when a peer's
// file does not appear within `timeout_ms`, or has the wrong size.
std::vector<std::vector<uint8_t>> file_rendezvous(const std::string& base_path, int rank, int world,
                                                  const std::vector<uint8_t>& blob, int timeout_ms = 600000,
                                                  int poll_ms = 50);
void file_rendezvous_cleanup(const std::string& base_path, int rank);

// Rank 0 binds `path` and accepts world-1 workers; workers connect with retries. Messages
// are an int32 opcode, an int32 payload length and the payload.
class CmdChannel {
 public:
  struct Message {
    int32_t op = 0;
    std::vector<int32_t> payload;
  };
  CmdChannel(const std::string& path, int rank, int world, int connect_retries = 400, int retry_ms = 50);
  ~CmdChannel();
  CmdChannel(const CmdChannel&) = delete;
  CmdChannel& operator=(const CmdChannel&) = delete;
  // rank 0: send to every worker. Throws when a worker hung up.
  void broadcast(const Message& m);
  // workers: block (no GPU or CPU use) until the next command. Returns false on EOF.
  bool receive(Message& m);
  int rank() const { return rank_; }
  int world() const { return world_; }

 private:
  std::string path_;
  int rank_, world_;
  int listen_fd_ = -1;
  std::vector<int> peers_;  // rank 0: worker sockets; worker: one socket to rank 0
};

}  // namespace pk

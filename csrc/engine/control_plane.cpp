#include "control_plane.hpp"

#include <fcntl.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <thread>

namespace pk {

namespace {

std::string rank_file(const std::string& base, int r) { return base + ".rank" + std::to_string(r); }

bool read_whole(const std::string& path, std::vector<uint8_t>& out) {
  int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return false;
  struct stat st;
  if (fstat(fd, &st) != 0) {
    ::close(fd);
    return false;
  }
  out.resize((size_t)st.st_size);
  size_t got = 0;
  while (got < out.size()) {
    ssize_t n = ::read(fd, out.data() + got, out.size() - got);
    if (n <= 0) break;
    got += (size_t)n;
  }
  ::close(fd);
  return got == out.size();
}

void write_all(int fd, const void* data, size_t n) {
  const char* p = (const char*)data;
  while (n > 0) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      throw std::runtime_error(std::string("command channel send: ") + strerror(errno));
    }
    p += w;
    n -= (size_t)w;
  }
}

bool read_all(int fd, void* data, size_t n) {
  char* p = (char*)data;
  while (n > 0) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      throw std::runtime_error(std::string("command channel recv: ") + strerror(errno));
    }
    p += r;
    n -= (size_t)r;
  }
  return true;
}

}  // namespace

std::vector<std::vector<uint8_t>> file_rendezvous(const std::string& base_path, int rank, int world,
                                                  const std::vector<uint8_t>& blob, int timeout_ms, int poll_ms) {
  if (rank < 0 || rank >= world) throw std::runtime_error("rendezvous: bad rank");
  const std::string mine = rank_file(base_path, rank), tmp = mine + ".tmp" + std::to_string((long)getpid());
  {
    int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0600);
    if (fd < 0) throw std::runtime_error("rendezvous: cannot write " + tmp);
    size_t off = 0;
    while (off < blob.size()) {
      ssize_t w = ::write(fd, blob.data() + off, blob.size() - off);
      if (w <= 0) {
        ::close(fd);
        throw std::runtime_error("rendezvous: short write " + tmp);
      }
      off += (size_t)w;
    }
    ::close(fd);
    if (::rename(tmp.c_str(), mine.c_str()) != 0) throw std::runtime_error("rendezvous: cannot publish " + mine);
  }
  std::vector<std::vector<uint8_t>> all(world);
  all[rank] = blob;
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    while (true) {
      std::vector<uint8_t> got;
      if (read_whole(rank_file(base_path, r), got)) {
        if (got.size() != blob.size())
          throw std::runtime_error("rendezvous: rank " + std::to_string(r) + " published " + std::to_string(got.size()) +
                                   " bytes, expected " + std::to_string(blob.size()));
        all[r] = std::move(got);
        break;
      }
      const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
      if (ms > timeout_ms) throw std::runtime_error("rendezvous: rank " + std::to_string(r) + " never published " + rank_file(base_path, r));
      std::this_thread::sleep_for(std::chrono::milliseconds(poll_ms));
    }
  }
  return all;
}

void file_rendezvous_cleanup(const std::string& base_path, int rank) { ::unlink(rank_file(base_path, rank).c_str()); }

CmdChannel::CmdChannel(const std::string& path, int rank, int world, int connect_retries, int retry_ms)
    : path_(path), rank_(rank), world_(world) {
  if (world <= 1) return;
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  if (path.size() >= sizeof(addr.sun_path)) throw std::runtime_error("command channel: socket path too long");
  strncpy(addr.sun_path, path.c_str(), sizeof(addr.sun_path) - 1);
  if (rank == 0) {
    ::unlink(path.c_str());
    listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (listen_fd_ < 0) throw std::runtime_error("command channel: socket()");
    if (::bind(listen_fd_, (sockaddr*)&addr, sizeof addr) != 0 || ::listen(listen_fd_, world) != 0)
      throw std::runtime_error(std::string("command channel: bind/listen: ") + strerror(errno));
    peers_.assign(world, -1);
    for (int i = 1; i < world; ++i) {
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) throw std::runtime_error("command channel: accept()");
      int32_t who = -1;
      if (!read_all(fd, &who, 4) || who <= 0 || who >= world || peers_[who] != -1) {
        ::close(fd);
        throw std::runtime_error("command channel: bad hello from worker");
      }
      peers_[who] = fd;
    }
  } else {
    int fd = -1;
    for (int attempt = 0; attempt < connect_retries; ++attempt) {
      fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
      if (fd < 0) throw std::runtime_error("command channel: socket()");
      if (::connect(fd, (sockaddr*)&addr, sizeof addr) == 0) break;
      ::close(fd);
      fd = -1;
      std::this_thread::sleep_for(std::chrono::milliseconds(retry_ms));
    }
    if (fd < 0) throw std::runtime_error("command channel: rank 0 never listened on " + path);
    int32_t who = rank;
    write_all(fd, &who, 4);
    peers_.push_back(fd);
  }
}

CmdChannel::~CmdChannel() {
  for (int fd : peers_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) {
    ::close(listen_fd_);
    ::unlink(path_.c_str());
  }
}

void CmdChannel::broadcast(const Message& m) {
  if (world_ <= 1) return;
  if (rank_ != 0) throw std::runtime_error("command channel: only rank 0 broadcasts");
  const int32_t hdr[2] = {m.op, (int32_t)m.payload.size()};
  for (int r = 1; r < world_; ++r) {
    write_all(peers_[r], hdr, sizeof hdr);
    if (!m.payload.empty()) write_all(peers_[r], m.payload.data(), m.payload.size() * 4);
  }
}

bool CmdChannel::receive(Message& m) {
  if (rank_ == 0 || peers_.empty()) throw std::runtime_error("command channel: rank 0 does not receive");
  int32_t hdr[2];
  if (!read_all(peers_[0], hdr, sizeof hdr)) return false;
  if (hdr[1] < 0 || hdr[1] > (1 << 26)) throw std::runtime_error("command channel: bad payload length");
  m.op = hdr[0];
  m.payload.resize((size_t)hdr[1]);
  if (hdr[1] > 0 && !read_all(peers_[0], m.payload.data(), (size_t)hdr[1] * 4)) return false;
  return true;
}

}  // namespace pk

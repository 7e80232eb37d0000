#include "mem_guard.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <stdexcept>

namespace pk {

std::string headroom_verdict(size_t free_bytes, size_t total_bytes, size_t request_bytes, size_t min_free_bytes, const char* what) {
  if (min_free_bytes == 0) return "";
  if (request_bytes <= free_bytes && free_bytes - request_bytes >= min_free_bytes) return "";
  char buf[320];
  std::snprintf(buf, sizeof buf,
                "%s: allocating %.1f MiB would leave %.1f MiB free of %.1f MiB, below the floor of %.1f MiB (POCKET_MIN_FREE_MIB)",
                what, request_bytes / 1048576.0, request_bytes <= free_bytes ? (free_bytes - request_bytes) / 1048576.0 : 0.0,
                total_bytes / 1048576.0, min_free_bytes / 1048576.0);
  return buf;
}

size_t min_free_bytes_from_env() {
  const char* v = std::getenv("POCKET_MIN_FREE_MIB");
  if (v == nullptr || *v == 0) return 0;
  const long long mib = std::atoll(v);
  return mib > 0 ? (size_t)mib << 20 : 0;
}

bool mem_log_enabled() {
  const char* v = std::getenv("POCKET_LOG_MEM");
  return v != nullptr && v[0] == '1';
}

void require_headroom(size_t request_bytes, const char* what) {
  const size_t floor_bytes = min_free_bytes_from_env();
  if (floor_bytes == 0) return;
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return;   // no answer: the allocation itself will tell
  const std::string msg = headroom_verdict(free_b, total_b, request_bytes, floor_bytes, what);
  if (!msg.empty()) throw std::runtime_error(msg);
}

void log_device_memory(const char* tag, size_t engine_bytes) {
  if (!mem_log_enabled()) return;
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return;
  std::fprintf(stderr, "mem tag=%s free_mib=%zu total_mib=%zu engine_mib=%zu\n", tag, free_b >> 20, total_b >> 20, engine_bytes >> 20);
}

}  // namespace pk

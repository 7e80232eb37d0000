// Device-memory guard and log for long-lived engines: refuse an allocation that would leave less than
// POCKET_MIN_FREE_MIB of the GPU free (other tenants, fragmentation headroom, CUDA graphs), and print one line per
// allocation phase when POCKET_LOG_MEM=1. Counterpart of the reference's gguf_log_mem / DSV4_GGUF_MIN_FREE_MIB
// (cpp_engine/src/dsv4_engine.cpp:1406,1417-1430).
#pragma once

#include <cstddef>
#include <string>

namespace pk {

// Pure decision: empty string when `request` may be allocated, else the message to fail with.
std::string headroom_verdict(size_t free_bytes, size_t total_bytes, size_t request_bytes, size_t min_free_bytes, const char* what);

size_t min_free_bytes_from_env();   // POCKET_MIN_FREE_MIB (0 when unset)
bool mem_log_enabled();             // POCKET_LOG_MEM=1

// Queries the current device; throws std::runtime_error when the request does not fit above the floor.
void require_headroom(size_t request_bytes, const char* what);
// "mem tag=<tag> free_mib=<n> total_mib=<n> engine_mib=<n>" on stderr when logging is on.
void log_device_memory(const char* tag, size_t engine_bytes);

}  // namespace pk

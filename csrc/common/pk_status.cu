#include <cstdlib>

#include "pk_common.cuh"

static int g_last_cuda_error = 0;

PK_API void pk_set_last_cuda_error(int code) { g_last_cuda_error = code; }
PK_API int pk_last_cuda_error() { return g_last_cuda_error; }

// Library identity, so that callers can check that the in-tree build is the one loaded.
PK_API const char* pk_build_arch() { return "sm_100a"; }

PK_API int pk_pdl_enabled() {
  static const int on = [] {
    const char* v = getenv("POCKET_PDL");
    return (v != nullptr && v[0] == '0') ? 0 : 1;
  }();
  return on;
}

// ---- debug build: index checks (pk_common.cuh) ----
#include <utility>
#include <vector>

namespace {
std::vector<std::pair<int (*)(unsigned*), int (*)()>>& debug_units() {
  static std::vector<std::pair<int (*)(unsigned*), int (*)()>> v;
  return v;
}
}  // namespace

// Called by every translation unit of the debug library while it is loaded.
PK_API void pk_debug_register(int (*read)(unsigned*), int (*clear)()) { debug_units().push_back({read, clear}); }

PK_API int pk_debug_bounds_enabled() { return PK_DEBUG_BUILD; }

// out[0] code (0 = nothing recorded), out[1] the bad index, out[2] its limit, out[3] how many accesses were skipped.
// Synchronises the device.
PK_API int pk_debug_bounds_read(unsigned* out) {
  out[0] = out[1] = out[2] = out[3] = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return PK_ERR_CUDA;
  for (auto& u : debug_units()) {
    unsigned w[4] = {0, 0, 0, 0};
    if (u.first(w) != 0) return PK_ERR_CUDA;
    if (w[0] != 0 && out[0] == 0) {
      out[0] = w[0];
      out[1] = w[1];
      out[2] = w[2];
    }
    out[3] += w[3];
  }
  return PK_OK;
}

PK_API int pk_debug_bounds_clear() {
  for (auto& u : debug_units())
    if (u.second() != 0) return PK_ERR_CUDA;
  return PK_OK;
}

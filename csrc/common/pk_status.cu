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

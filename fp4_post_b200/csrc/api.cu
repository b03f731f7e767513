// Status plumbing and queries of the C ABI.
#include "common.cuh"

#include <atomic>
#include <stdlib.h>

namespace metis {

static thread_local char g_last_error[512] = "";

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace metis

extern "C" const char* metis_last_error_string(void) { return metis::g_last_error; }

namespace metis {
// SMs a launch of the persistent GEMM kernels may take on the current device: all, or the caller's limit
int gemm_sm_budget(int32_t limit) {
  const int n = device_sm_count();
  return (limit > 0 && limit < n) ? (int)limit : n;
}
// METIS_LAUNCH_OVERLAP in the environment: a mask of the LaunchClass bits that get programmatic-serialization launches
bool launch_overlap_enabled(int launch_class) {
  static const int mask = [] {
    const char* v = getenv("METIS_LAUNCH_OVERLAP");
    return v ? atoi(v) : (kLaunchShort | kLaunchGemm | kLaunchStream);
  }();
  return (mask & launch_class) != 0;
}
}  // namespace metis

extern "C" int32_t metis_query(int32_t* abi_version, int32_t* compiled_sm, int32_t* device_sm_count) {
  if (abi_version) *abi_version = METIS_NVFP4_ABI_VERSION;
  if (compiled_sm) *compiled_sm = 100;
  if (device_sm_count) {
    int n = 0, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess)
      *device_sm_count = n;
    else
      *device_sm_count = 0;
  }
  return METIS_OK;
}

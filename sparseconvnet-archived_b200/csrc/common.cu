// Error reporting, device queries and status strings of libscn_b200.so.
#include <cstdlib>
#include "scn_common.cuh"
#include <atomic>
#include <cstdarg>
#include <cstring>

namespace scn {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
void clear_error() { g_err[0] = 0; }

static std::atomic<long long> g_launches{0};
bool dependent_launch_enabled() {
  static const bool on = [] { const char *e = std::getenv("SCN_DEPENDENT_LAUNCH"); return !(e && e[0] == '0'); }();
  return on;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

} // namespace scn

extern "C" const char *scn_status_string(int status) {
  switch (status) {
  case SCN_OK: return "ok";
  case SCN_ERR_INVALID: return "invalid argument";
  case SCN_ERR_CUDA: return "CUDA error";
  case SCN_ERR_WORKSPACE: return "workspace too small";
  case SCN_ERR_UNSUPPORTED: return "unsupported configuration";
  default: return "unknown status";
  }
}

extern "C" const char *scn_last_error(void) { return scn::g_err; }
extern "C" long long scn_kernel_launch_count(void) { return scn::g_launches.load(std::memory_order_relaxed); }

extern "C" int scn_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
  return major == 10;
}

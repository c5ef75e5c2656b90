// Library-wide plumbing of the C ABI: version, error string, launch counter, device info.
#include <stdarg.h>

#include <atomic>

#include "common.cuh"

namespace dlb {
namespace {
thread_local char g_err[512] = "";
thread_local int64_t g_launches = 0;
// process-wide policy of the bounded barrier waits (dlb_set_wait_policy)
std::atomic<unsigned long long> g_wait_limit{0};
std::atomic<int> g_withhold_loads{0};
}  // namespace

unsigned long long wait_limit_cycles(unsigned long long fallback) {
  const unsigned long long v = g_wait_limit.load(std::memory_order_relaxed);
  return v ? v : fallback;
}
bool withhold_loads() { return g_withhold_loads.load(std::memory_order_relaxed) != 0; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch() { ++g_launches; }

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace dlb

extern "C" int dlb_version(void) { return 100; }

extern "C" const char* dlb_last_error_string(void) { return dlb::g_err; }

extern "C" int64_t dlb_launch_count(int reset) {
  int64_t v = dlb::g_launches;
  if (reset) dlb::g_launches = 0;
  return v;
}

extern "C" int dlb_set_wait_policy(uint64_t limit_cycles, int withhold_loads) {
  dlb::g_wait_limit.store(limit_cycles, std::memory_order_relaxed);
  dlb::g_withhold_loads.store(withhold_loads ? 1 : 0, std::memory_order_relaxed);
  return DLB_OK;
}

// Error reporting and launch accounting shared by every entry point.
#include "common.cuh"
#include <atomic>
#include <cstdarg>
#include <cstdio>

namespace {
thread_local char g_error[512] = "";
std::atomic<unsigned long long> g_launches{0};
}  // namespace

namespace mb {

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int num_sms() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return 148;
  }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 148;
  }
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

int after_launch(const char* kernel_name) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(MB_ERR_LAUNCH, "%s: launch failed: %s", kernel_name, cudaGetErrorString(e));
  return MB_OK;
}

}  // namespace mb

extern "C" {
const char* mb_last_error(void) { return g_error; }
int mb_abi_version(void) { return 1; }
unsigned long long mb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
}

// Error reporting and version of the C ABI.
#include <stdarg.h>

#include <atomic>

#include "tab_common.cuh"

namespace tab {

static thread_local char g_last_error[512] = "";
static std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what, int kernels) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TAB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(kernels, std::memory_order_relaxed);
  return TAB_OK;
}

}  // namespace tab

extern "C" int tab_version(void) { return 100; }

extern "C" const char* tab_last_error(void) { return tab::g_last_error; }

extern "C" long long tab_launch_count(void) { return tab::g_launches.load(std::memory_order_relaxed); }

// Status reporting, launch accounting and small host utilities of the pariskv_b200 library.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace pk {
static thread_local char g_err[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what, int n_kernels) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  g_launches.fetch_add(n_kernels, std::memory_order_relaxed);
  return PK_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace pk

extern "C" {
int pk_version(void) { return 1; }
const char* pk_last_error(void) { return pk::g_err; }
int64_t pk_launch_count(void) { return pk::g_launches.load(std::memory_order_relaxed); }
}

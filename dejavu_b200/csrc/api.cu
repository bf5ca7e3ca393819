// Library-wide plumbing of the C ABI: error strings, launch counter, device properties.
#include <atomic>
#include <cstdarg>
#include <cstring>

#include "common.cuh"

namespace djv {

static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
    return DJV_ERR_CUDA;
  }
  return DJV_OK;
}

static thread_local int g_early_prefetch = 0;
bool early_prefetch() { return g_early_prefetch != 0 && pdl_enabled(); }

static thread_local int g_programmatic_launch = 1;
bool pdl_enabled() {
  static const bool on = env_int("DJV_PDL", 1) != 0;
  return on && g_programmatic_launch != 0;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace djv

extern "C" int djv_version(void) { return 100; }

extern "C" void djv_set_early_weight_prefetch(int enabled) { djv::g_early_prefetch = enabled; }

extern "C" void djv_set_programmatic_launch(int enabled) { djv::g_programmatic_launch = enabled; }

extern "C" const char *djv_last_error(void) { return djv::g_err; }

extern "C" const char *djv_status_string(int status) {
  switch (status) {
    case DJV_OK: return "ok";
    case DJV_ERR_INVALID: return "invalid argument";
    case DJV_ERR_UNSUPPORTED: return "unsupported configuration";
    case DJV_ERR_CUDA: return "CUDA error";
    case DJV_ERR_SCRATCH: return "scratch buffer too small or misaligned";
    case DJV_ERR_TIMEOUT: return "bounded device-side wait ran out";
    default: return "unknown status";
  }
}

extern "C" unsigned long long djv_launch_count(void) {
  return djv::g_launches.load(std::memory_order_relaxed);
}

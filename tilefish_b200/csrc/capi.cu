// Library identity and the thread-local last error.
#include <atomic>
#include <string>

#include "common.cuh"

namespace tf {

static thread_local std::string g_last_error;

tf_status fail(tf_status code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

void clear_error() { g_last_error.clear(); }

int sm_count() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

static std::atomic<int> g_programmatic_launch{0};  // process-wide (tf_set_programmatic_launch)
bool programmatic_launch_enabled() { return g_programmatic_launch.load(std::memory_order_relaxed) != 0; }
void set_programmatic_launch(bool on) { g_programmatic_launch.store(on ? 1 : 0, std::memory_order_relaxed); }

}  // namespace tf

using namespace tf;

extern "C" {

tf_status tf_set_programmatic_launch(int32_t enabled) {
  tf::clear_error();
  tf::set_programmatic_launch(enabled != 0);
  return TF_OK;
}

const char* tf_version(void) { return "tilefish_b200 0.2.0 (sm_100a)"; }
const char* tf_last_error(void) { return g_last_error.c_str(); }

}  // extern "C"

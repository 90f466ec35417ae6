// Library identity, the thread-local last error and the device status word.
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

// Written by kernels whose bounded waits ran out: [0] = status, [1] = detail (which wait, which block).
__device__ int g_device_status[2];

}  // namespace tf

using namespace tf;

extern "C" {

const char* tf_version(void) { return "tilefish_b200 0.1.0 (sm_100a)"; }
const char* tf_last_error(void) { return g_last_error.c_str(); }

tf_status tf_device_status(int32_t* status, int32_t* detail) {
  clear_error();
  TF_CHECK_ARG(status != nullptr, "%s: null pointer", __func__);
  int host[2] = {0, 0};
  TF_CUDA(cudaDeviceSynchronize());
  TF_CUDA(cudaMemcpyFromSymbol(host, g_device_status, sizeof(host)));
  if (host[0] != 0) {
    const int zero[2] = {0, 0};
    TF_CUDA(cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero)));
  }
  *status = host[0];
  if (detail) *detail = host[1];
  return TF_OK;
}

}  // extern "C"

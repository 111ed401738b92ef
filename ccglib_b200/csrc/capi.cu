// Status handling and small utilities of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace ccglib_b200 {

namespace {
thread_local char g_last_error[512] = "";
}

void set_last_error(const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
  va_end(args);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_last_error("cudaGetDevice failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    set_last_error("cudaDeviceGetAttribute failed: %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (dev >= 0 && dev < 64) cached[dev] = sms;
  return sms;
}

} // namespace ccglib_b200

using namespace ccglib_b200;

extern "C" const char *ccglib_b200_status_string(int status) {
  switch (status) {
  case CCGLIB_B200_OK:
    return "success";
  case CCGLIB_B200_INVALID_ARGUMENT:
    return "invalid argument";
  case CCGLIB_B200_UNSUPPORTED:
    return "unsupported combination";
  case CCGLIB_B200_CUDA_ERROR:
    return "CUDA error";
  case CCGLIB_B200_DEVICE_TIMEOUT:
    return "device-side wait timed out";
  case CCGLIB_B200_OUT_OF_MEMORY:
    return "out of memory";
  default:
    return "unknown status";
  }
}

extern "C" const char *ccglib_b200_last_error(void) { return g_last_error; }

// Error plumbing and device queries of the C ABI.
#include "common.cuh"

namespace sb {

char *error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
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

}  // namespace sb

extern "C" int spira_b200_version(void) { return 100; }

extern "C" const char *spira_b200_last_error(void) { return sb::error_buffer(); }

extern "C" int spira_b200_reset_error(void) {
  cudaGetLastError();
  sb::error_buffer()[0] = 0;
  return SPIRA_B200_OK;
}

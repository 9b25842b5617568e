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

static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void set_pdl_enabled(bool on) { g_pdl = on; }

}  // namespace sb

extern "C" int spira_b200_version(void) { return 100; }

extern "C" const char *spira_b200_last_error(void) { return sb::error_buffer(); }

extern "C" int spira_b200_reset_error(void) {
  cudaGetLastError();
  sb::error_buffer()[0] = 0;
  return SPIRA_B200_OK;
}

// Stream-ordered read-back that does not wait for work enqueued later on `stream`: an event marks the current end
// of `stream`, `copy_stream` waits for it and copies, `done_event` (recorded on `copy_stream`) tells the host when
// the bytes have arrived.  One library-owned event per device serves as the marker.
extern "C" int spira_b200_read_back(const void *device_src, void *pinned_dst, size_t bytes, void *stream, void *copy_stream,
                                    void *done_event) {
  SB_CHECK_ARG(device_src && pinned_dst && copy_stream && done_event, "read_back: null pointer");
  SB_CHECK_ARG(copy_stream != stream, "read_back: copy_stream must differ from stream");
  static cudaEvent_t marker[64] = {nullptr};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64, "read_back: device %d out of range", dev);
  if (marker[dev] == nullptr) SB_CHECK_CUDA(cudaEventCreateWithFlags(&marker[dev], cudaEventDisableTiming));
  SB_CHECK_CUDA(cudaEventRecord(marker[dev], sb::as_stream(stream)));
  SB_CHECK_CUDA(cudaStreamWaitEvent(sb::as_stream(copy_stream), marker[dev], 0));
  SB_CHECK_CUDA(cudaMemcpyAsync(pinned_dst, device_src, bytes, cudaMemcpyDeviceToHost, sb::as_stream(copy_stream)));
  SB_CHECK_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(done_event), sb::as_stream(copy_stream)));
  return SPIRA_B200_OK;
}

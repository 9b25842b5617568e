// Shared helpers of the spira_b200 native library (error reporting, key layout, launch checks).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "spira_b200.h"

namespace sb {

// Thread-local message returned by spira_b200_last_error().
char *error_buffer();
int fail(int code, const char *fmt, ...);

#define SB_CHECK_ARG(cond, ...)                                  \
  do {                                                           \
    if (!(cond)) return sb::fail(SPIRA_B200_ERR_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define SB_CHECK_CUDA(expr)                                                                     \
  do {                                                                                          \
    cudaError_t e_ = (expr);                                                                    \
    if (e_ != cudaSuccess)                                                                      \
      return sb::fail(SPIRA_B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                      __FILE__, __LINE__);                                                      \
  } while (0)

#define SB_CHECK_LAUNCH() SB_CHECK_CUDA(cudaGetLastError())

// Bit layout of packed voxel keys: z in the low bits, then y, then x.
template <typename KeyT>
struct KeyLayout;
template <>
struct KeyLayout<uint32_t> {
  static constexpr int ZB = 8, YB = 12, XB = 12;
};
template <>
struct KeyLayout<uint64_t> {
  static constexpr int ZB = 16, YB = 24, XB = 24;
};
template <typename KeyT>
struct KeyShift {
  static constexpr int Y = KeyLayout<KeyT>::ZB;
  static constexpr int X = KeyLayout<KeyT>::ZB + KeyLayout<KeyT>::YB;
};

inline int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align128(int64_t n) { return div_up(n, 128) * 128; }

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of SMs of the current device (cached per device).
int sm_count();

// One convolution from its descriptor (the body of spira_b200_conv; the tape executor calls it per operator).
int conv_run(const spira_b200_conv_desc &desc, int32_t *status, void *stream);

}  // namespace sb

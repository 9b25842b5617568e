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

// Programmatic dependent launch.  A kernel launched through launch_dependent() may be scheduled while its predecessor on
// the stream is still draining: its CTAs take the SMs the predecessor's CTAs leave, run their set-up, and block in
// pdl_wait() (device side, ptx.cuh) until the predecessor grid has completed and its writes are visible.  That hides the
// 2-3 us between two dependent launches of one-CTA-per-SM kernels (measured: 3.1 -> 0.7 us).  Rules for a kernel launched
// this way: every thread executes pdl_wait() before its FIRST access to global memory -- also to weights and other
// constants, which a kernel enqueued just before may have written -- and nothing is written before it.  `pdl_enabled()` is the "pdl" option (default on).
bool pdl_enabled();
void set_pdl_enabled(bool on);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Device side of the programmatic dependent launch: pdl_trigger() lets the next kernel on the stream be scheduled as this
// grid's CTAs leave, pdl_wait() blocks until the previous grid has completed and its writes are visible.  Both are no-ops
// for a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// One convolution from its descriptor (the body of spira_b200_conv; the tape executor calls it per operator).
int conv_run(const spira_b200_conv_desc &desc, int32_t *status, void *stream);

// 1x1x1 layers (identity map) as dense tiles moved by TMA (dense.cu).  dense_applies: channel counts in whole 32-channel
// boxes (c_a = channels of the first source, c_in - c_a of the second), c_out a multiple of 16 up to 256, 16-byte aligned
// tensors, and a driver that encodes tensor maps.  `packed` is the K = 1 image of spira_b200_pack_weights.
bool dense_applies(int64_t n, int c_in, int c_a, int c_out, const void *feats, const void *feats_b, const void *packed);
int dense_run(const void *feats, const void *feats_b, int c_a, const void *packed, const spira_b200_epilogue *epilogue, int64_t n,
              int c_in, int c_out, void *out, int32_t *status, unsigned long long wait_ns, cudaStream_t st);

}  // namespace sb

// 1x1x1 layers with few output channels (classification heads): out[n][c_out] = feats[n][c_in] . W[c_in][c_out] + bias.
//
// The reference sends every 1x1x1 layer to torch.mm (spira/nn/conv.py:312-316).  For a head with e.g. 19 classes the
// library GEMM cannot use its aligned kernels (c_out is not a multiple of 8) and a separate element-wise kernel adds
// the bias.  The layer reads n*c_in*2 bytes and writes n*c_out*2: it is bound by HBM, not by arithmetic, so plain
// fp32 FMAs are enough.  One thread per voxel: the row arrives with 16-byte loads, the weights sit in shared memory
// as fp32 (every lane reads the same address: a broadcast), the c_out sums stay in registers, and the rows of a block
// leave through shared memory so that the stores are contiguous.  fp32 accumulation, one rounding to fp16.
#include "common.cuh"

namespace sb {

constexpr int kPwThreads = 256;

template <int CO>   // c_out rounded up to a multiple of 8
__global__ void __launch_bounds__(kPwThreads) pointwise_kernel(const __half *__restrict__ feats, const __half *__restrict__ w,
                                                                const __half *__restrict__ bias, int64_t n, int c_in, int c_out,
                                                                __half *__restrict__ out) {
  extern __shared__ __align__(16) unsigned char pw_smem[];
  float *s_w = reinterpret_cast<float *>(pw_smem);                         // [c_in][CO]
  float *s_bias = s_w + c_in * CO;                                          // [CO]
  __half *s_out = reinterpret_cast<__half *>(s_bias + CO);                  // [256][c_out]
  const int tid = threadIdx.x;
  for (int i = tid; i < c_in * CO; i += kPwThreads) {
    const int k = i / CO, c = i - k * CO;
    s_w[i] = c < c_out ? __half2float(w[k * c_out + c]) : 0.f;
  }
  if (tid < CO) s_bias[tid] = (bias != nullptr && tid < c_out) ? __half2float(bias[tid]) : 0.f;
  __syncthreads();
  const int k8_end = c_in / 8;
  for (int64_t row0 = static_cast<int64_t>(blockIdx.x) * kPwThreads; row0 < n; row0 += static_cast<int64_t>(gridDim.x) * kPwThreads) {
    const int64_t row = row0 + tid;
    float acc[CO];
#pragma unroll
    for (int c = 0; c < CO; ++c) acc[c] = s_bias[c];
    if (row < n) {
      const uint4 *p = reinterpret_cast<const uint4 *>(feats + row * c_in);
#pragma unroll 2
      for (int k8 = 0; k8 < k8_end; ++k8) {
        const uint4 v = __ldg(p + k8);
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          const float4 *w0 = reinterpret_cast<const float4 *>(s_w + (k8 * 8 + 2 * j) * CO);
#pragma unroll
          for (int c4 = 0; c4 < CO / 4; ++c4) {
            const float4 a = w0[c4], b = w0[CO / 4 + c4];
            acc[4 * c4 + 0] = fmaf(f.x, a.x, acc[4 * c4 + 0]);
            acc[4 * c4 + 1] = fmaf(f.x, a.y, acc[4 * c4 + 1]);
            acc[4 * c4 + 2] = fmaf(f.x, a.z, acc[4 * c4 + 2]);
            acc[4 * c4 + 3] = fmaf(f.x, a.w, acc[4 * c4 + 3]);
            acc[4 * c4 + 0] = fmaf(f.y, b.x, acc[4 * c4 + 0]);
            acc[4 * c4 + 1] = fmaf(f.y, b.y, acc[4 * c4 + 1]);
            acc[4 * c4 + 2] = fmaf(f.y, b.z, acc[4 * c4 + 2]);
            acc[4 * c4 + 3] = fmaf(f.y, b.w, acc[4 * c4 + 3]);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < CO; ++c)
      if (c < c_out) s_out[tid * c_out + c] = __float2half_rn(acc[c]);
    __syncthreads();
    const int64_t rows_here = (n - row0 < kPwThreads) ? (n - row0) : kPwThreads;
    const int total = static_cast<int>(rows_here) * c_out;
    __half *dst = out + row0 * c_out;
    for (int i = tid; i < total; i += kPwThreads) dst[i] = s_out[i];
    __syncthreads();
  }
}

template <int CO>
static int launch_pointwise(const __half *feats, const __half *w, const __half *bias, int64_t n, int c_in, int c_out, __half *out,
                            cudaStream_t st) {
  const size_t smem = static_cast<size_t>(c_in) * CO * 4 + CO * 4 + static_cast<size_t>(kPwThreads) * c_out * 2;
  if (smem > 48 * 1024) return fail(SPIRA_B200_ERR_UNSUPPORTED, "pointwise: c_in=%d, c_out=%d need %zu bytes of shared memory", c_in, c_out, smem);
  int64_t blocks = div_up(n, kPwThreads);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  pointwise_kernel<CO><<<static_cast<unsigned>(blocks), kPwThreads, smem, st>>>(feats, w, bias, n, c_in, c_out, out);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

}  // namespace sb

using namespace sb;

extern "C" int spira_b200_pointwise(const void *feats, const void *weights, const void *bias, int64_t n, int c_in, int c_out,
                                    void *out, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "pointwise: n=%lld out of range", (long long)n);
  if (c_in < 8 || c_in % 8 != 0 || c_out < 1 || c_out > 32)
    return fail(SPIRA_B200_ERR_UNSUPPORTED, "pointwise: c_in=%d must be a multiple of 8 and c_out=%d at most 32", c_in, c_out);
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(feats && weights && out, "pointwise: null pointer");
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(feats) % 16 == 0, "pointwise: feature rows must be 16-byte aligned");
  const __half *f = static_cast<const __half *>(feats), *w = static_cast<const __half *>(weights), *b = static_cast<const __half *>(bias);
  __half *o = static_cast<__half *>(out);
  cudaStream_t st = as_stream(stream);
  if (c_out <= 8) return launch_pointwise<8>(f, w, b, n, c_in, c_out, o, st);
  if (c_out <= 16) return launch_pointwise<16>(f, w, b, n, c_in, c_out, o, st);
  if (c_out <= 24) return launch_pointwise<24>(f, w, b, n, c_in, c_out, o, st);
  return launch_pointwise<32>(f, w, b, n, c_in, c_out, o, st);
}

// 1x1x1 layers with few output channels (classification heads): out[n][c_out] = feats[n][c_in] . W[c_in][c_out] + bias.
//
// The reference sends every 1x1x1 layer to torch.mm (spira/nn/conv.py:312-316).  For a head with e.g. 19 classes the
// library GEMM cannot use its aligned kernels (c_out is not a multiple of 8) and a separate element-wise kernel adds
// the bias.  The layer reads n*c_in*2 bytes and writes n*c_out*2: it is bound by HBM.  A reduction of 96 and 24
// (padded) output columns is far too small for a tcgen05 pipeline (one 128-row MMA tile would wait longer for its
// barriers than it computes), so each warp multiplies 16 voxels at a time with warp-level m16n8k16 MMAs: the A
// fragments come straight from global memory (the four lanes of a quad read 16 contiguous bytes of a row), the
// transposed weights sit in shared memory with a padded stride (conflict-free fragment loads), accumulation is fp32
// with the bias as the initial value, and the 16 x c_out results leave through shared memory as one contiguous run.
#include "common.cuh"

namespace sb {

constexpr int kPwThreads = 256;
constexpr int kPwWarps = kPwThreads / 32;
constexpr int kPwKGroup = 6;     // k-steps (of 16) whose row loads are issued together

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NT>   // 8-column tiles of the output: c_out <= 8 * NT
__global__ void __launch_bounds__(kPwThreads) pointwise_kernel(const __half *__restrict__ feats, const __half *__restrict__ w,
                                                                const __half *__restrict__ bias, int64_t n, int c_in, int c_out,
                                                                __half *__restrict__ out) {
  extern __shared__ __align__(16) unsigned char pw_smem[];
  const int k_pad = (c_in + 15) / 16 * 16;          // reduction length in whole k-steps (c_in is a multiple of 8)
  const int ldw = k_pad + 8;                        // halfs per weight column: 4 * (odd number) words, no bank conflicts
  __half *s_wt = reinterpret_cast<__half *>(pw_smem);                                  // [8 * NT][ldw]: W transposed
  float *s_bias = reinterpret_cast<float *>(pw_smem + static_cast<size_t>(8 * NT) * ldw * 2);   // [8 * NT]
  __half *s_out = reinterpret_cast<__half *>(s_bias + 8 * NT);                         // [warps][16 * c_out]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  pdl_trigger();
  pdl_wait();      // (before the first global read: also the weights may have been written by the kernel before this one)
  for (int i = tid; i < 8 * NT * ldw; i += kPwThreads) {
    const int col = i / ldw, k = i - col * ldw;
    s_wt[i] = (col < c_out && k < c_in) ? w[k * c_out + col] : __float2half(0.f);
  }
  if (tid < 8 * NT) s_bias[tid] = (bias != nullptr && tid < c_out) ? __half2float(bias[tid]) : 0.f;
  __syncthreads();

  const int k_steps = k_pad / 16;
  const uint32_t *wt32 = reinterpret_cast<const uint32_t *>(s_wt);
  __half *my_out = s_out + warp * 16 * c_out;
  const int64_t n_tiles = (n + 15) / 16;
  for (int64_t tile = static_cast<int64_t>(blockIdx.x) * kPwWarps + warp; tile < n_tiles;
       tile += static_cast<int64_t>(gridDim.x) * kPwWarps) {
    const int64_t r0 = tile * 16 + g, r1 = r0 + 8;
    const uint32_t *p0 = reinterpret_cast<const uint32_t *>(feats + (r0 < n ? r0 : 0) * c_in);
    const uint32_t *p1 = reinterpret_cast<const uint32_t *>(feats + (r1 < n ? r1 : 0) * c_in);
    const bool ok0 = r0 < n, ok1 = r1 < n;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc[nt][0] = acc[nt][2] = s_bias[8 * nt + 2 * t];
      acc[nt][1] = acc[nt][3] = s_bias[8 * nt + 2 * t + 1];
    }
    for (int kb = 0; kb < k_steps; kb += kPwKGroup) {
      uint32_t a[kPwKGroup][4];
#pragma unroll
      for (int j = 0; j < kPwKGroup; ++j) {
        // words of a row: k-step (kb + j) covers halfs [16 (kb + j), +16); this lane takes halfs 2t, 2t+1 and 2t+8, 2t+9
        const int w_lo = 8 * (kb + j) + t, w_hi = w_lo + 4;
        const bool in_lo = kb + j < k_steps, in_hi = in_lo && 2 * w_hi < c_in;   // (c_in % 16 == 8: the last half step is padding)
        a[j][0] = (in_lo && ok0) ? __ldg(p0 + w_lo) : 0u;
        a[j][1] = (in_lo && ok1) ? __ldg(p1 + w_lo) : 0u;
        a[j][2] = (in_hi && ok0) ? __ldg(p0 + w_hi) : 0u;
        a[j][3] = (in_hi && ok1) ? __ldg(p1 + w_hi) : 0u;
      }
#pragma unroll
      for (int j = 0; j < kPwKGroup; ++j) {
        if (kb + j >= k_steps) break;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t *col = wt32 + (8 * nt + g) * (ldw / 2) + 8 * (kb + j) + t;
          mma_m16n8k16(acc[nt], a[j], col[0], col[4]);
        }
      }
    }
    // accumulator layout: [0], [1] = row g, columns 2t, 2t+1 of the tile; [2], [3] = row g + 8
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = 8 * nt + 2 * t + (e & 1), row = g + 8 * (e >> 1);
        if (col < c_out) my_out[row * c_out + col] = __float2half_rn(acc[nt][e]);
      }
    }
    __syncwarp();
    const int64_t rows_here = n - tile * 16 < 16 ? n - tile * 16 : 16;
    const int total = static_cast<int>(rows_here) * c_out;
    __half *dst = out + tile * 16 * c_out;
    for (int i = lane; i < total; i += 32) dst[i] = my_out[i];
    __syncwarp();
  }
}

template <int NT>
static int launch_pointwise(const __half *feats, const __half *w, const __half *bias, int64_t n, int c_in, int c_out, __half *out,
                            cudaStream_t st) {
  const int k_pad = (c_in + 15) / 16 * 16;
  const size_t smem = static_cast<size_t>(8 * NT) * (k_pad + 8) * 2 + 8 * NT * 4 + static_cast<size_t>(kPwWarps) * 16 * c_out * 2;
  if (smem > 48 * 1024) return fail(SPIRA_B200_ERR_UNSUPPORTED, "pointwise: c_in=%d, c_out=%d need %zu bytes of shared memory", c_in, c_out, smem);
  int64_t blocks = div_up(div_up(n, 16), kPwWarps);
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  SB_CHECK_CUDA(launch_dependent(pointwise_kernel<NT>, dim3(static_cast<unsigned>(blocks)), dim3(kPwThreads), smem, st, feats, w, bias, n,
                                 c_in, c_out, out));
  return SPIRA_B200_OK;
}

}  // namespace sb

using namespace sb;

extern "C" int spira_b200_pointwise(const void *feats, const void *weights, const void *bias, int64_t n, int c_in, int c_out,
                                    void *out, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "pointwise: n=%lld out of range", (long long)n);
  if (c_in < 8 || c_in % 8 != 0 || c_in > 512 || c_out < 1 || c_out > 32)
    return fail(SPIRA_B200_ERR_UNSUPPORTED, "pointwise: c_in=%d must be a multiple of 8 up to 512 and c_out=%d at most 32", c_in, c_out);
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(feats && weights && out, "pointwise: null pointer");
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(feats) % 16 == 0, "pointwise: feature rows must be 16-byte aligned");
  const __half *f = static_cast<const __half *>(feats), *w = static_cast<const __half *>(weights), *b = static_cast<const __half *>(bias);
  __half *o = static_cast<__half *>(out);
  cudaStream_t st = as_stream(stream);
  if (c_out <= 8) return launch_pointwise<1>(f, w, b, n, c_in, c_out, o, st);
  if (c_out <= 16) return launch_pointwise<2>(f, w, b, n, c_in, c_out, o, st);
  if (c_out <= 24) return launch_pointwise<3>(f, w, b, n, c_in, c_out, o, st);
  return launch_pointwise<4>(f, w, b, n, c_in, c_out, o, st);
}

// Scene ingest in two cooperative launches: (1) pack + sort the voxel keys with their permutation, (2) all down-sampled
// levels of the network.
//
// Both steps are a handful of dependent passes over ~10^5 keys, a megabyte or so: the work of a pass takes a few
// microseconds, so a chain of library kernels (a radix sort is ~7 launches, a stream compaction 2, per level and per
// sort) spends its time on launch latencies.  Here every chain is ONE kernel whose CTAs meet at grid barriers between
// the passes (cooperative launch, bounded waits).
//
// Sort (replaces the Compress + FillRange + radix SortPairs sequence of
// csrc/spira/cuda/functions/arg_sort_coodrinates.cu:35-88): least-significant-digit radix sort with 8-bit digits,
// stable, so equal keys keep their input order like the reference's.  A first pass over the input packs the keys and
// finds which bits differ between keys at all (AND / OR of all keys): digits whose bits are constant are skipped, which
// removes e.g. five of the eight passes of a 64-bit key in a 512^3 grid.  A pass is: every CTA sums the per-CTA digit
// histograms of the CTAs before it (its base position per digit) and scatters its contiguous chunk in order, ranking
// equal digits inside a warp with match_any and across warps with a per-warp count table, and counts the NEXT digit of
// every key it moves for the chunk the key lands in -> grid barrier (one per pass).
//
// Down-sampling of sorted keys (csrc/spira/torch/cuda_arg_sort_coordinates.cu:107-200 sorts every level from scratch):
// flooring the coordinates to a stride twice as coarse disturbs the order only inside a coarse cell, so the final
// position of a coarse key = the number of input keys with a smaller coarse key = a sum of lengths of contiguous ranges
// of the sorted input, found by binary searches inside the x' block of the element.  All inputs with the same coarse key
// land on the same slot; compacting the written slots (per-CTA counts -> grid barrier -> scatter) yields
// unique(sort(keys & mask)).  Level l + 1 is computed from the output of level l inside the same launch.
#include "common.cuh"
#include "grid_sync.cuh"
#include "radix_sort.cuh"

namespace sb {

// key of voxel i from its coordinates (csrc/spira/cuda/kernels/compress.cuh:18-22)
template <typename KeyT>
struct CoordsGen {
  const int32_t *coords;      // [n][3]
  __device__ __forceinline__ KeyT operator()(int i) const {
    const KeyT x = static_cast<KeyT>(coords[3 * i + 0]), y = static_cast<KeyT>(coords[3 * i + 1]),
               z = static_cast<KeyT>(coords[3 * i + 2]);
    return (x << KeyShift<KeyT>::X) | (y << KeyShift<KeyT>::Y) | z;
  }
};

// ---- all down-sampled levels of sorted keys ----------------------------------------------------------------------------
template <typename KeyT>
struct CoarsenParams {
  const KeyT *keys;                                 // level 0, sorted
  KeyT *out[SPIRA_B200_MAX_LEVELS];                 // level l + 1, n keys of room each
  int32_t stride[SPIRA_B200_MAX_LEVELS][3];         // target stride of level l + 1
  int32_t *counts;                                  // [n_levels]
  KeyT *vals;                                       // [n] scratch
  uint32_t *flags;                                  // [n_levels][flags_pitch] words, zero on entry: bit i = slot i written
  unsigned *barrier;
  int32_t *status;                                  // may be null; 2 = the input is not sorted
  unsigned long long limit_ns;
  int64_t flags_pitch;
  int32_t n, n_levels;
};

// (The input of a level is never written while the level is being read, and an SM has not read it before it was
// written: plain, L1-cached loads are safe and keep the block-local searches out of L2.)
template <typename KeyT>
__device__ __forceinline__ int lower_bound_range(const KeyT *__restrict__ a, int lo, int hi, KeyT v) {
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// lower_bound over [0, n) by a whole warp: 32 probes per round (4 dependent loads for 10^5 keys instead of 17)
template <typename KeyT>
__device__ __forceinline__ int warp_lower_bound_range(const KeyT *__restrict__ a, int n, KeyT q, int lane) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int len = hi - lo;
    const int step = (len + 31) >> 5;
    const int pos = lo + lane * step;
    const bool less = (pos < hi) && (a[pos] < q);
    const int c = __popc(__ballot_sync(0xffffffffu, less));
    if (c == 0) {
      hi = lo;
    } else {
      const int nhi = lo + c * step;
      lo = lo + (c - 1) * step + 1;
      hi = nhi < hi ? nhi : hi;
    }
  }
  return lo;
}

template <typename KeyT>
__global__ void __launch_bounds__(kIngestThreads) coarsen_levels_kernel(const __grid_constant__ CoarsenParams<KeyT> P) {
  using L = KeyLayout<KeyT>;
  constexpr KeyT XM = (KeyT(1) << L::XB) - 1, YM = (KeyT(1) << L::YB) - 1, ZM = (KeyT(1) << L::ZB) - 1;
  __shared__ uint32_t s_warp[kIngestWarps];
  __shared__ uint32_t s_red2[kIngestWarps];
  __shared__ uint32_t s_run;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, b = blockIdx.x;
  GridBarrier gb{P.barrier, P.limit_ns, P.status, 0u};
  auto pack3 = [](KeyT a, KeyT bb, KeyT c) { return (a << KeyShift<KeyT>::X) | (bb << KeyShift<KeyT>::Y) | c; };

  const KeyT *in = P.keys;
  int n = P.n;
  int prev[3] = {1, 1, 1};
  for (int l = 0; l < P.n_levels; ++l) {
    const int sx = prev[0], sy = prev[1], sz = prev[2];
    const int rx = P.stride[l][0] / sx, ry = P.stride[l][1] / sy, rz = P.stride[l][2] / sz;      // 1 or 2 per axis
    uint32_t *flags = P.flags + l * P.flags_pitch;
    // ---- every input key writes its coarse key to the slot of its final rank among the inputs ----------------------------
    for (int i0 = (b * kIngestThreads + tid) & ~31; i0 < n; i0 += G * kIngestThreads) {        // (whole warps enter together)
      const int i = i0 + lane;
      const bool valid = i < n;
      const KeyT key = valid ? in[i] : KeyT(0);
      if (l == 0 && valid && i > 0 && in[i - 1] > key && P.status) atomicExch(P.status, 2);     // not sorted: report, do not guess
      const KeyT x = (key >> KeyShift<KeyT>::X) & XM, y = (key >> KeyShift<KeyT>::Y) & YM, z = key & ZM;
      const KeyT X0 = x & ~static_cast<KeyT>(sx * rx - 1), Y0 = y & ~static_cast<KeyT>(sy * ry - 1),
                 Z0 = z & ~static_cast<KeyT>(sz * rz - 1);
      const KeyT x_end = X0 + static_cast<KeyT>(sx * rx);
      // The x' block [lo, hi) of this element.  The 32 consecutive elements of a warp mostly share it: then the warp finds
      // its two ends together; else every lane searches for itself.
      const KeyT X0_first = __shfl_sync(0xffffffffu, X0, 0);
      const bool uniform = __all_sync(0xffffffffu, !valid || X0 == X0_first);
      int lo, hi;
      if (uniform) {
        const KeyT xe = X0_first + static_cast<KeyT>(sx * rx);
        lo = warp_lower_bound_range(in, n, pack3(X0_first, 0, 0), lane);
        hi = xe <= XM ? warp_lower_bound_range(in, n, pack3(xe, 0, 0), lane) : n;
      } else {
        lo = valid ? lower_bound_range(in, 0, i + 1, pack3(X0, 0, 0)) : 0;
        hi = !valid ? 0 : (x_end <= XM ? lower_bound_range(in, i, n, pack3(x_end, 0, 0)) : n);
      }
      if (!valid) continue;
      // pos = lo + sum over the x values xc of the cell of [ #{xc, y < Y0} + sum over its y values yc of #{xc, yc, z < Z0} ].
      // With LB(.) the lower bound of a key inside [lo, hi), the term of one xc is
      //     LB(xc,Y0,0) - LB(xc,0,0)  +  LB(xc,Y0,Z0) - LB(xc,Y0,0)  +  LB(xc,Y0+sy,Z0) - LB(xc,Y0+sy,0)
      //   = - LB(xc,0,0) + LB(xc,Y0,Z0) - LB(xc,Y0+sy,0) + LB(xc,Y0+sy,Z0)          (the last two only if y is halved).
      // The eight lower bounds do not depend on one another, so they advance in lockstep: one round of eight loads per
      // halving of the block instead of eight searches one after the other.
      KeyT q[8];
      int sign[8];
#pragma unroll
      for (int jx = 0; jx < 2; ++jx) {
        const KeyT xc = X0 + static_cast<KeyT>(jx * sx), y1 = Y0 + static_cast<KeyT>(sy);
        const bool on_x = jx < rx, on_y = on_x && ry > 1;
        q[4 * jx + 0] = pack3(xc, 0, 0);   sign[4 * jx + 0] = on_x ? -1 : 0;
        q[4 * jx + 1] = pack3(xc, Y0, Z0); sign[4 * jx + 1] = on_x ? 1 : 0;
        q[4 * jx + 2] = pack3(xc, y1, 0);  sign[4 * jx + 2] = on_y ? -1 : 0;
        q[4 * jx + 3] = pack3(xc, y1, Z0); sign[4 * jx + 3] = on_y ? 1 : 0;
      }
      int at[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) at[e] = lo;
      for (int len = hi - lo; len > 0;) {                     // branch-free lower bounds, all eight at once
        const int half = len >> 1;
        if (half == 0) {
#pragma unroll
          for (int e = 0; e < 8; ++e) at[e] += (sign[e] != 0 && in[at[e]] < q[e]) ? 1 : 0;
          break;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (sign[e] != 0) at[e] = (in[at[e] + half - 1] < q[e]) ? at[e] + half : at[e];
        len -= half;
      }
      int pos = lo;
#pragma unroll
      for (int e = 0; e < 8; ++e) pos += sign[e] * at[e];
      if (pos < n) {       // (always, for sorted input)
        P.vals[pos] = pack3(X0, Y0, Z0);
        atomicOr(&flags[pos >> 5], 1u << (pos & 31));
      }
    }
    if (!grid_sync(gb)) return;
    // ---- compaction of the written slots.  The CTA takes a contiguous run of flag words; the number of slots written
    // before its run is the popcount of all words before it, which every CTA adds up for itself (a few KB from L2).
    const int n_words = (n + 31) >> 5;
    const int chunk = (n_words + G - 1) / G;
    const int w0 = min(n_words, b * chunk), w1 = min(n_words, w0 + chunk);
    uint32_t before = 0, total = 0;
    for (int w = tid; w < n_words; w += kIngestThreads) {
      const uint32_t c = __popc(__ldcg(flags + w));
      total += c;
      before += w < w0 ? c : 0u;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      total += __shfl_xor_sync(0xffffffffu, total, d);
      before += __shfl_xor_sync(0xffffffffu, before, d);
    }
    if (lane == 0) { s_warp[warp] = total; s_red2[warp] = before; }
    __syncthreads();
    if (tid == 0) {
      uint32_t t = 0, bf = 0;
      for (int w = 0; w < kIngestWarps; ++w) { t += s_warp[w]; bf += s_red2[w]; }
      s_run = bf;
      if (b == 0) P.counts[l] = static_cast<int32_t>(t);
    }
    __syncthreads();
    KeyT *out = P.out[l];
    for (int wb = w0; wb < w1; wb += kIngestWarps) {          // one flag word per warp, one slot per lane
      const int w = wb + warp;
      const uint32_t bits = w < w1 ? __ldcg(flags + w) : 0u;
      if (lane == 0) s_warp[warp] = __popc(bits);
      __syncthreads();
      uint32_t pos = s_run + __popc(bits & ((1u << lane) - 1u));
      for (int j = 0; j < warp; ++j) pos += s_warp[j];
      if ((bits >> lane) & 1u) out[pos] = __ldcg(P.vals + w * 32 + lane);
      __syncthreads();
      if (tid == 0) {
        uint32_t t = 0;
        for (int j = 0; j < kIngestWarps; ++j) t += s_warp[j];
        s_run += t;
      }
      __syncthreads();
    }
    // the next level reads this level's output and count, and reuses vals
    if (l + 1 < P.n_levels) {
      if (!grid_sync(gb)) return;
      n = __ldcg(&P.counts[l]);
      in = out;
      prev[0] = P.stride[l][0]; prev[1] = P.stride[l][1]; prev[2] = P.stride[l][2];
    }
  }
}

inline size_t round256i(size_t b) { return (b + 255) / 256 * 256; }

// CTAs of the cooperative down-sampling launch: as many as can be resident at once (at most four per SM).
template <typename KeyT>
static int coarsen_grid() {
  static int per_sm[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count();
  if (per_sm[dev] == 0) {
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, coarsen_levels_kernel<KeyT>, kIngestThreads, 0) != cudaSuccess || nb < 1) nb = 1;
    per_sm[dev] = nb > 4 ? 4 : nb;
  }
  return sm_count() * per_sm[dev];
}

static unsigned long long ingest_wait_ns() {
  const int us = spira_b200_get_option("wait_limit_us");
  return static_cast<unsigned long long>(us > 0 ? us : 1500000) * 1000ull;
}

template <typename KeyT>
int sort_impl(const int32_t *coords, int64_t n, KeyT *sorted_keys, int32_t *perm, void *ws, size_t ws_bytes, int32_t *status,
              cudaStream_t stream) {
  return radix_sort_generated<KeyT>(CoordsGen<KeyT>{coords}, n, sorted_keys, perm, ws, ws_bytes, status, ingest_wait_ns(), stream,
                                    "flatten_sort");
}

template <typename KeyT>
size_t coarsen_workspace_bytes(int64_t n) {
  // [control 256][vals n][flag bits MAX_LEVELS * pitch]
  return 256 + round256i(n * sizeof(KeyT)) + SPIRA_B200_MAX_LEVELS * round256i((n + 31) / 32 * 4);
}

template <typename KeyT>
int coarsen_impl(const KeyT *keys, int64_t n, int n_levels, const int32_t *strides, void *const *out_keys, int32_t *counts,
                 void *ws, size_t ws_bytes, int32_t *status, cudaStream_t stream) {
  const size_t need = coarsen_workspace_bytes<KeyT>(n);
  if (ws_bytes < need) return fail(SPIRA_B200_ERR_WORKSPACE, "downsample_sorted: workspace %zu < %zu bytes", ws_bytes, need);
  if (n == 0) {
    SB_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_levels, stream));
    return SPIRA_B200_OK;
  }
  char *p = static_cast<char *>(ws);
  CoarsenParams<KeyT> P{};
  P.keys = keys;
  for (int l = 0; l < n_levels; ++l) {
    P.out[l] = static_cast<KeyT *>(out_keys[l]);
    for (int a = 0; a < 3; ++a) P.stride[l][a] = strides[3 * l + a];
  }
  P.counts = counts;
  P.barrier = reinterpret_cast<unsigned *>(p);
  char *q = p + 256;
  P.vals = reinterpret_cast<KeyT *>(q);
  P.flags = reinterpret_cast<uint32_t *>(q + round256i(n * sizeof(KeyT)));
  P.flags_pitch = static_cast<int64_t>(round256i((n + 31) / 32 * 4) / 4);
  P.status = status;
  P.limit_ns = ingest_wait_ns();
  P.n = static_cast<int32_t>(n);
  P.n_levels = n_levels;
  if (status) SB_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  SB_CHECK_CUDA(cudaMemsetAsync(p, 0, 256, stream));
  SB_CHECK_CUDA(cudaMemsetAsync(P.flags, 0, n_levels * round256i((n + 31) / 32 * 4), stream));
  void *args[] = {&P};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&coarsen_levels_kernel<KeyT>), dim3(coarsen_grid<KeyT>()),
                                              dim3(kIngestThreads), args, 0, stream);
  if (e != cudaSuccess) return fail(SPIRA_B200_ERR_CUDA, "downsample_sorted: cooperative launch failed: %s", cudaGetErrorString(e));
  return SPIRA_B200_OK;
}

size_t ingest_sort_workspace(int64_t n, int key_bytes) {
  return key_bytes == 4 ? sort_workspace_bytes<uint32_t>(n) : sort_workspace_bytes<uint64_t>(n);
}

int ingest_sort(const int32_t *coords, int64_t n, int key_bytes, void *sorted_keys, int32_t *perm, void *ws, size_t ws_bytes,
                int32_t *status, cudaStream_t stream) {
  if (key_bytes == 4) return sort_impl<uint32_t>(coords, n, static_cast<uint32_t *>(sorted_keys), perm, ws, ws_bytes, status, stream);
  return sort_impl<uint64_t>(coords, n, static_cast<uint64_t *>(sorted_keys), perm, ws, ws_bytes, status, stream);
}

size_t ingest_coarsen_workspace(int64_t n, int key_bytes) {
  return key_bytes == 4 ? coarsen_workspace_bytes<uint32_t>(n) : coarsen_workspace_bytes<uint64_t>(n);
}

int ingest_coarsen(const void *keys, int64_t n, int key_bytes, int n_levels, const int32_t *strides, void *const *out_keys,
                   int32_t *counts, void *ws, size_t ws_bytes, int32_t *status, cudaStream_t stream) {
  if (key_bytes == 4)
    return coarsen_impl<uint32_t>(static_cast<const uint32_t *>(keys), n, n_levels, strides, out_keys, counts, ws, ws_bytes, status, stream);
  return coarsen_impl<uint64_t>(static_cast<const uint64_t *>(keys), n, n_levels, strides, out_keys, counts, ws, ws_bytes, status, stream);
}

}  // namespace sb

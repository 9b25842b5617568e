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
// removes e.g. five of the eight passes of a 64-bit key in a 512^3 grid.  A pass is: per-CTA digit histogram of the
// CTA's contiguous chunk -> grid barrier -> every CTA sums the histogram columns of the CTAs before it (its base
// position per digit) and scatters its chunk in order, ranking equal digits inside a warp with match_any and across
// warps with a per-warp count table -> grid barrier.
//
// Down-sampling of sorted keys (csrc/spira/torch/cuda_arg_sort_coordinates.cu:107-200 sorts every level from scratch):
// flooring the coordinates to a stride twice as coarse disturbs the order only inside a coarse cell, so the final
// position of a coarse key = the number of input keys with a smaller coarse key = a sum of lengths of contiguous ranges
// of the sorted input, found by binary searches inside the x' block of the element.  All inputs with the same coarse key
// land on the same slot; compacting the written slots (per-CTA counts -> grid barrier -> scatter) yields
// unique(sort(keys & mask)).  Level l + 1 is computed from the output of level l inside the same launch.
#include "common.cuh"
#include "grid_sync.cuh"

namespace sb {

constexpr int kIngestThreads = 1024;
constexpr int kIngestWarps = kIngestThreads / 32;

template <typename KeyT>
struct SortParams {
  const int32_t *coords;      // [n][3]
  KeyT *keys_a;               // result (sorted keys)
  int32_t *vals_a;            // result (permutation)
  KeyT *keys_b;               // scratch
  int32_t *vals_b;
  uint32_t *ghist;            // [gridDim.x][256]
  KeyT *bits;                 // [2]: AND and OR of all keys (initialised to ~0 and 0)
  unsigned *barrier;
  int32_t *status;
  unsigned long long limit_ns;
  int32_t n;
};

__device__ __forceinline__ void atomic_and_or(uint32_t *bits, uint32_t a, uint32_t o) {
  atomicAnd(&bits[0], a);
  atomicOr(&bits[1], o);
}
__device__ __forceinline__ void atomic_and_or(uint64_t *bits, uint64_t a, uint64_t o) {
  atomicAnd(reinterpret_cast<unsigned long long *>(&bits[0]), static_cast<unsigned long long>(a));
  atomicOr(reinterpret_cast<unsigned long long *>(&bits[1]), static_cast<unsigned long long>(o));
}

template <typename KeyT>
__global__ void __launch_bounds__(kIngestThreads) sort_keys_kernel(const __grid_constant__ SortParams<KeyT> P) {
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_base[256];
  __shared__ uint32_t s_wcount[kIngestWarps][256];
  __shared__ uint32_t s_part[3][2][256];
  __shared__ KeyT s_red[2 * kIngestWarps];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, b = blockIdx.x, n = P.n;
  const int chunk = (n + G - 1) / G;
  const int c0 = min(n, b * chunk), c1 = min(n, c0 + chunk);
  GridBarrier gb{P.barrier, P.limit_ns, P.status, 0u};

  // ---- pack the chunk, identity permutation, AND / OR of all keys --------------------------------------------------------
  if (tid < 256) s_hist[tid] = 0;
  __syncthreads();
  KeyT k_and = ~KeyT(0), k_or = KeyT(0);
  for (int i = c0 + tid; i < c1; i += kIngestThreads) {
    const KeyT x = static_cast<KeyT>(P.coords[3 * i + 0]), y = static_cast<KeyT>(P.coords[3 * i + 1]),
               z = static_cast<KeyT>(P.coords[3 * i + 2]);
    const KeyT key = (x << KeyShift<KeyT>::X) | (y << KeyShift<KeyT>::Y) | z;
    P.keys_a[i] = key;
    P.vals_a[i] = i;
    k_and &= key;
    k_or |= key;
    atomicAdd(&s_hist[static_cast<uint32_t>(key) & 0xffu], 1u);      // histogram of the first pass (the lowest digit)
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    k_and &= __shfl_xor_sync(0xffffffffu, k_and, d);
    k_or |= __shfl_xor_sync(0xffffffffu, k_or, d);
  }
  if (lane == 0) { s_red[warp] = k_and; s_red[kIngestWarps + warp] = k_or; }
  for (int i = tid; i < kIngestWarps * 256; i += kIngestThreads) (&s_wcount[0][0])[i] = 0;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kIngestWarps; ++w) { k_and &= s_red[w]; k_or |= s_red[kIngestWarps + w]; }
    atomic_and_or(P.bits, k_and, k_or);
  }
  if (tid < 256) P.ghist[b * 256 + tid] = s_hist[tid];
  if (!grid_sync(gb)) return;
  // bits in which at least two keys differ; the lowest digit always gets its pass (its histogram is on its way already:
  // a pass over a constant digit moves nothing)
  const KeyT varying = (__ldcg(&P.bits[0]) ^ __ldcg(&P.bits[1])) | KeyT(0xff);

  const KeyT *k_in = P.keys_a;
  const int32_t *v_in = P.vals_a;
  KeyT *k_out = P.keys_b;
  int32_t *v_out = P.vals_b;
  for (int shift = 0; shift < static_cast<int>(sizeof(KeyT)) * 8; shift += 8) {
    if (((varying >> shift) & KeyT(0xff)) == 0) continue;            // every key has the same digit here: nothing moves
    // ---- histogram of the chunk (the first pass got its histogram while packing) -------------------------------------------
    if (shift > 0) {
      if (tid < 256) s_hist[tid] = 0;
      __syncthreads();
      // (keys written by other CTAs in the pass before: read them past the L1, which is not coherent across SMs)
      for (int i = c0 + tid; i < c1; i += kIngestThreads) atomicAdd(&s_hist[static_cast<uint32_t>(__ldcg(k_in + i) >> shift) & 0xffu], 1u);
      __syncthreads();
      if (tid < 256) P.ghist[b * 256 + tid] = s_hist[tid];
      if (!grid_sync(gb)) return;
    }
    // ---- base position of every digit for this CTA: digits before it, and the same digit in the CTAs before it ---------------
    {
      // four threads per digit, each over a quarter of the CTAs, sixteen loads in flight: the sums are latency, not work
      const int d = tid & 255, part = tid >> 8;
      const int per = (G + 3) / 4;
      const int cb = min(G, part * per), ce = min(G, cb + per);
      uint32_t total = 0, before = 0;
      int c = cb;
      for (; c + 16 <= ce; c += 16) {
        uint32_t v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __ldcg(&P.ghist[(c + e) * 256 + d]);
#pragma unroll
        for (int e = 0; e < 16; ++e) { total += v[e]; before += (c + e) < b ? v[e] : 0u; }
      }
      for (; c < ce; ++c) {
        const uint32_t v = __ldcg(&P.ghist[c * 256 + d]);
        total += v;
        before += c < b ? v : 0u;
      }
      if (part > 0) { s_part[part - 1][0][d] = total; s_part[part - 1][1][d] = before; }
      __syncthreads();
      if (part == 0) {
        s_hist[d] = total + s_part[0][0][d] + s_part[1][0][d] + s_part[2][0][d];
        s_base[d] = before + s_part[0][1][d] + s_part[1][1][d] + s_part[2][1][d];
      }
    }
    __syncthreads();
    if (warp == 0) {                     // exclusive scan of the 256 totals: 8 per lane
      uint32_t t[8], sum = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) { t[e] = s_hist[lane * 8 + e]; sum += t[e]; }
      uint32_t incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += y;
      }
      uint32_t run = incl - sum;
#pragma unroll
      for (int e = 0; e < 8; ++e) { s_base[lane * 8 + e] += run; run += t[e]; }
    }
    __syncthreads();
    // ---- scatter the chunk in order: 512 keys per step, equal digits ranked inside a warp and across the warps -----------------
    for (int i0 = c0; i0 < c1; i0 += kIngestThreads) {
      const int i = i0 + tid;
      const bool valid = i < c1;
      KeyT key = KeyT(0);
      int32_t val = 0;
      if (valid) { key = __ldcg(k_in + i); val = __ldcg(v_in + i); }
      const uint32_t digit = valid ? (static_cast<uint32_t>(key >> shift) & 0xffu) : 0x100u + lane;   // idle lanes match nobody
      const unsigned peers = __match_any_sync(0xffffffffu, digit);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const bool leader = valid && rank == 0;
      if (leader) s_wcount[warp][digit] = __popc(peers);
      __syncthreads();
      if (tid < 256) {                   // digit `tid`: positions of the warps' groups, and the running base
        uint32_t acc = s_base[tid];
#pragma unroll
        for (int w = 0; w < kIngestWarps; ++w) {
          const uint32_t c = s_wcount[w][tid];
          s_wcount[w][tid] = acc;
          acc += c;
        }
        s_base[tid] = acc;
      }
      __syncthreads();
      if (valid) {
        const uint32_t pos = s_wcount[warp][digit] + rank;
        k_out[pos] = key;
        v_out[pos] = val;
      }
      __syncthreads();
      if (tid < 256) {
#pragma unroll
        for (int w = 0; w < kIngestWarps; ++w) s_wcount[w][tid] = 0;
      }
      __syncthreads();
    }
    if (!grid_sync(gb)) return;
    const KeyT *tk = k_in; k_in = k_out; k_out = const_cast<KeyT *>(tk);
    const int32_t *tv = v_in; v_in = v_out; v_out = const_cast<int32_t *>(tv);
  }
  // an odd number of passes leaves the result in the scratch buffers
  if (k_in != P.keys_a) {
    for (int i = c0 + tid; i < c1; i += kIngestThreads) { P.keys_a[i] = __ldcg(k_in + i); P.vals_a[i] = __ldcg(v_in + i); }
  }
}

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

// CTAs of a cooperative ingest launch: they all have to be resident at once.  The sort uses one per SM (every CTA sums
// a histogram column per CTA and pass); the down-sampling, whose rank pass is a chain of dependent loads per key, takes
// as many as fit.
static int ingest_grid() { return sm_count(); }

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
size_t sort_workspace_bytes(int64_t n) {
  // [control 256][ghist G*256*4][alt keys][alt perm]
  return 256 + round256i(static_cast<size_t>(ingest_grid()) * 256 * 4) + round256i(n * sizeof(KeyT)) + round256i(n * sizeof(int32_t));
}

template <typename KeyT>
int sort_impl(const int32_t *coords, int64_t n, KeyT *sorted_keys, int32_t *perm, void *ws, size_t ws_bytes, int32_t *status,
              cudaStream_t stream) {
  const size_t need = sort_workspace_bytes<KeyT>(n);
  if (ws_bytes < need) return fail(SPIRA_B200_ERR_WORKSPACE, "flatten_sort: workspace %zu < %zu bytes", ws_bytes, need);
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(ws) % 16 == 0, "flatten_sort: workspace must be 16-byte aligned");
  char *p = static_cast<char *>(ws);
  // control block: [0] barrier counter, [16..] AND / OR words
  SB_CHECK_CUDA(cudaMemsetAsync(p, 0, 256, stream));
  SB_CHECK_CUDA(cudaMemsetAsync(p + 16, 0xFF, sizeof(KeyT), stream));
  SortParams<KeyT> P{};
  P.coords = coords;
  P.keys_a = sorted_keys;
  P.vals_a = perm;
  P.barrier = reinterpret_cast<unsigned *>(p);
  P.bits = reinterpret_cast<KeyT *>(p + 16);
  P.ghist = reinterpret_cast<uint32_t *>(p + 256);
  char *q = p + 256 + round256i(static_cast<size_t>(ingest_grid()) * 256 * 4);
  P.keys_b = reinterpret_cast<KeyT *>(q);
  P.vals_b = reinterpret_cast<int32_t *>(q + round256i(n * sizeof(KeyT)));
  P.status = status;
  P.limit_ns = ingest_wait_ns();
  P.n = static_cast<int32_t>(n);
  void *args[] = {&P};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&sort_keys_kernel<KeyT>), dim3(ingest_grid()),
                                              dim3(kIngestThreads), args, 0, stream);
  if (e != cudaSuccess) return fail(SPIRA_B200_ERR_CUDA, "flatten_sort: cooperative launch failed: %s", cudaGetErrorString(e));
  return SPIRA_B200_OK;
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

// Cooperative radix sort of (key, index) pairs whose keys are produced on the fly by a generator.
//
// Least-significant-digit radix sort with 8-bit digits, stable (equal keys keep their input order).  ONE kernel, launched
// cooperatively with one CTA per SM; the passes are separated by grid barriers instead of kernel boundaries, because a
// pass over ~10^5 keys is a few microseconds of work and a chain of launches would spend its time on launch latencies.
// A first phase generates the keys of the CTA's contiguous chunk (gen(i) for element i), writes the identity
// permutation, builds the histogram of the lowest digit and finds which bits differ between keys at all (AND / OR of all
// keys): digits whose bits are the same in every key are skipped.  A pass is: every CTA sums the histogram columns of the
// CTAs before it (its base position per digit) and scatters its chunk in order, ranking equal digits inside a warp with
// match_any and across warps with a per-warp count table -> grid barrier.  The per-CTA histograms of the NEXT pass are
// built during the scatter: the thread that moves a key knows the chunk it lands in and adds one to that chunk's count
// of the key's next digit (a global reduction), so a pass needs ONE grid barrier and no histogram phase of its own.
// Three histogram tables rotate: pass p reads table p % 3, adds into table (p + 1) % 3 and clears its own row of table
// (p + 2) % 3, which every CTA finished reading before the barrier of pass p - 1.
#pragma once

#include "common.cuh"
#include "grid_sync.cuh"

namespace sb {

constexpr int kIngestThreads = 1024;
constexpr int kIngestWarps = kIngestThreads / 32;

template <typename KeyT, typename Gen>
struct SortParams {
  Gen gen;                    // gen(i) = key of element i
  KeyT *keys_a;               // result (sorted keys)
  int32_t *vals_a;            // result (permutation)
  KeyT *keys_b;               // scratch
  int32_t *vals_b;
  uint32_t *ghist;            // [3][gridDim.x][256]
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

template <typename KeyT, typename Gen>
__global__ void __launch_bounds__(kIngestThreads) sort_keys_kernel(const __grid_constant__ SortParams<KeyT, Gen> P) {
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

  // ---- keys of the chunk, identity permutation, AND / OR of all keys ---------------------------------------------------------
  if (tid < 256) s_hist[tid] = 0;
  __syncthreads();
  KeyT k_and = ~KeyT(0), k_or = KeyT(0);
  for (int i = c0 + tid; i < c1; i += kIngestThreads) {
    const KeyT key = P.gen(i);
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
  if (tid < 256) {
    P.ghist[b * 256 + tid] = s_hist[tid];
    P.ghist[(G + b) * 256 + tid] = 0u;      // this CTA's row of the table the first pass adds into
  }
  if (!grid_sync(gb)) return;
  // bits in which at least two keys differ; the lowest digit always gets its pass (its histogram is on its way already:
  // a pass over a constant digit moves nothing)
  const KeyT varying = (__ldcg(&P.bits[0]) ^ __ldcg(&P.bits[1])) | KeyT(0xff);

  const KeyT *k_in = P.keys_a;
  const int32_t *v_in = P.vals_a;
  KeyT *k_out = P.keys_b;
  int32_t *v_out = P.vals_b;
  constexpr int kKeyBits = static_cast<int>(sizeof(KeyT)) * 8;
  int pass = 0;
  for (int shift = 0; shift < kKeyBits; shift += 8) {
    if (((varying >> shift) & KeyT(0xff)) == 0) continue;            // every key has the same digit here: nothing moves
    int next_shift = shift + 8;                                      // the digit of the next pass, if there is one
    while (next_shift < kKeyBits && ((varying >> next_shift) & KeyT(0xff)) == 0) next_shift += 8;
    const bool more = next_shift < kKeyBits;
    const uint32_t *hist_cur = P.ghist + static_cast<size_t>(pass % 3) * G * 256;
    uint32_t *hist_next = P.ghist + static_cast<size_t>((pass + 1) % 3) * G * 256;
    if (tid < 256) P.ghist[(static_cast<size_t>((pass + 2) % 3) * G + b) * 256 + tid] = 0u;
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
        for (int e = 0; e < 16; ++e) v[e] = __ldcg(&hist_cur[(c + e) * 256 + d]);
#pragma unroll
        for (int e = 0; e < 16; ++e) { total += v[e]; before += (c + e) < b ? v[e] : 0u; }
      }
      for (; c < ce; ++c) {
        const uint32_t v = __ldcg(&hist_cur[c * 256 + d]);
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
        // the key lands in chunk pos / chunk: that CTA's histogram of the next digit
        if (more) atomicAdd(&hist_next[(pos / static_cast<uint32_t>(chunk)) * 256 + (static_cast<uint32_t>(key >> next_shift) & 0xffu)], 1u);
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
    ++pass;
  }
  // an odd number of passes leaves the result in the scratch buffers
  if (k_in != P.keys_a) {
    for (int i = c0 + tid; i < c1; i += kIngestThreads) { P.keys_a[i] = __ldcg(k_in + i); P.vals_a[i] = __ldcg(v_in + i); }
  }
}


inline size_t sort_round256(size_t b) { return (b + 255) / 256 * 256; }

// CTAs of the cooperative sort: one per SM (they all have to be resident at once, and every CTA sums one histogram
// column per CTA and pass).
inline int sort_grid() { return sm_count(); }

template <typename KeyT>
size_t sort_workspace_bytes(int64_t n) {
  // [control 256][ghist 3*G*256*4][alt keys][alt values]
  return 256 + sort_round256(static_cast<size_t>(sort_grid()) * 3 * 256 * 4) + sort_round256(n * sizeof(KeyT)) + sort_round256(n * sizeof(int32_t));
}

// Sorts n generated keys into sorted_keys / order (order[i] = element of sorted position i).  The 16-byte aligned
// workspace is cleared in stream order by the call.
template <typename KeyT, typename Gen>
int radix_sort_generated(const Gen &gen, int64_t n, KeyT *sorted_keys, int32_t *order, void *ws, size_t ws_bytes, int32_t *status,
                         unsigned long long limit_ns, cudaStream_t stream, const char *what) {
  const size_t need = sort_workspace_bytes<KeyT>(n);
  if (ws_bytes < need) return fail(SPIRA_B200_ERR_WORKSPACE, "%s: workspace %zu < %zu bytes", what, ws_bytes, need);
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(ws) % 16 == 0, "%s: workspace must be 16-byte aligned", what);
  char *p = static_cast<char *>(ws);
  // control block: [0] barrier counter, [16..] AND / OR words
  SB_CHECK_CUDA(cudaMemsetAsync(p, 0, 256, stream));
  SB_CHECK_CUDA(cudaMemsetAsync(p + 16, 0xFF, sizeof(KeyT), stream));
  SortParams<KeyT, Gen> P{};
  P.gen = gen;
  P.keys_a = sorted_keys;
  P.vals_a = order;
  P.barrier = reinterpret_cast<unsigned *>(p);
  P.bits = reinterpret_cast<KeyT *>(p + 16);
  P.ghist = reinterpret_cast<uint32_t *>(p + 256);
  char *q = p + 256 + sort_round256(static_cast<size_t>(sort_grid()) * 3 * 256 * 4);
  P.keys_b = reinterpret_cast<KeyT *>(q);
  P.vals_b = reinterpret_cast<int32_t *>(q + sort_round256(n * sizeof(KeyT)));
  P.status = status;
  P.limit_ns = limit_ns;
  P.n = static_cast<int32_t>(n);
  void *args[] = {&P};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&sort_keys_kernel<KeyT, Gen>), dim3(sort_grid()),
                                              dim3(kIngestThreads), args, 0, stream);
  if (e != cudaSuccess) return fail(SPIRA_B200_ERR_CUDA, "%s: cooperative launch failed: %s", what, cudaGetErrorString(e));
  return SPIRA_B200_OK;
}

}  // namespace sb

// Kernel-map construction: one launch builds the (input, output, weight-offset) maps of every
// sparse-convolution layer of a network.
//
// Work decomposition: one CTA of 256 threads per tile of 128 consecutive sorted targets of one map; a thread resolves
// one (target, xy offset) column at a time: a lower bound for the lowest z, then a walk over the kz consecutive z
// values (keys are z-fastest, so the kz answers are neighbours in the sorted source array).
// The lower bound does not search the whole source array.  For a fixed x offset the queries tgt[t] + off(ix, iy) of a
// tile grow with t and with iy, so all of them fall into ONE window of the sorted sources, whose two ends the CTA
// finds first with warp-cooperative 32-ary searches (4 dependent loads for 120k keys instead of 17).  The per-thread
// binary searches then run inside that window (typically a few hundred keys: ~9 steps, and the window stays in L1).
// No shared-memory staging: the kernel keeps next to nothing per CTA, so every SM holds its full complement of warps
// and the dependent loads of one search hide behind the others.
// Results are
//   - written as a dense int32 map, [K][T_al] (consecutive threads = consecutive targets of one offset: coalesced
//     rows) or [T_al][K] (consecutive threads = consecutive xy offsets of one target: runs of nxy entries), and
//   - counted per (offset, 128-target tile), which is what the compaction into weight-stationary pair lists, the mask
//     format and the dataflow selector consume.
// A query equals an exact lookup of the wrapped packed key; offsets whose queries wrap inside the tile search the
// whole array, every z on its own.
#include "common.cuh"

namespace sb {

constexpr int kTile = 128;          // targets per CTA
constexpr int kSearchThreads = 256;
constexpr int kMaxXY = 64;          // kx*ky
constexpr int kMaxK = 512;          // kx*ky*kz

template <typename KeyT>
struct MapDesc {
  const KeyT *src;
  const KeyT *tgt;
  int32_t *map;
  int32_t *tile_counts;
  const int32_t *row_perm;   // weight-stationary layout: natural row k is stored as row row_perm[k] (null: identity)
  int32_t S, T, T_al, n_tiles;
  int32_t kx, ky, kz, nxy, K;
  int32_t x0, y0, z0;  // lowest offset per axis, in units of the source stride
  int32_t sx, sy, sz;
  int32_t layout;
  int32_t tile_begin;
};

template <typename KeyT>
struct SearchParams {
  MapDesc<KeyT> m[SPIRA_B200_MAX_MAPS];
  int32_t n_maps;
};

template <typename KeyT>
__device__ __forceinline__ KeyT xy_offset(const MapDesc<KeyT> &D, int ix, int iy) {
  // wrapping arithmetic on purpose: identical to adding signed multiples of the field units
  return static_cast<KeyT>(static_cast<int64_t>(ix + D.x0) * D.sx) * (KeyT(1) << KeyShift<KeyT>::X) +
         static_cast<KeyT>(static_cast<int64_t>(iy + D.y0) * D.sy) * (KeyT(1) << KeyShift<KeyT>::Y) +
         static_cast<KeyT>(static_cast<int64_t>(D.z0) * D.sz);
}

// lower_bound over global memory by a whole warp: 32 probes per round.
template <typename KeyT>
__device__ __forceinline__ int warp_lower_bound(const KeyT *__restrict__ a, int n, KeyT q, int lane) {
  int lo = 0, hi = n;
  while (lo < hi) {
    int len = hi - lo;
    int step = (len + 31) >> 5;
    int pos = lo + lane * step;
    bool less = (pos < hi) && (a[pos] < q);
    int c = __popc(__ballot_sync(0xffffffffu, less));
    if (c == 0) {
      hi = lo;
    } else {
      int nhi = lo + c * step;
      lo = lo + (c - 1) * step + 1;
      hi = nhi < hi ? nhi : hi;
    }
  }
  return lo;
}

// Branch-free lower bound in a[lo, hi): the trip count depends on the window length only, so the lanes of a warp that
// share a window stay converged.
template <typename KeyT>
__device__ __forceinline__ int lower_bound(const KeyT *__restrict__ a, int lo, int hi, KeyT q) {
  int len = hi - lo;
  if (len <= 0) return lo;
  while (len > 1) {
    const int half = len >> 1;
    lo = (__ldg(a + lo + half - 1) < q) ? lo + half : lo;
    len -= half;
  }
  return lo + (__ldg(a + lo) < q ? 1 : 0);
}

template <typename KeyT>
__global__ void __launch_bounds__(kSearchThreads) kmap_search_kernel(const __grid_constant__ SearchParams<KeyT> P) {
  __shared__ KeyT s_tgt[kTile];
  __shared__ int s_lo[8], s_hi[8], s_irregular[8];      // per x offset (kx <= 8)
  __shared__ int s_cnt[kMaxK];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_trigger();
  pdl_wait();
  int mi = 0;
  while (mi + 1 < P.n_maps && static_cast<int>(blockIdx.x) >= P.m[mi + 1].tile_begin) ++mi;
  const MapDesc<KeyT> &D = P.m[mi];
  const int lt = blockIdx.x - D.tile_begin;
  const int t0 = lt * kTile;
  const int nvalid = min(kTile, D.T - t0);
  const KeyT *__restrict__ src = D.src;
  const KeyT first = D.tgt[t0], last = D.tgt[t0 + nvalid - 1];
  const KeyT sz = static_cast<KeyT>(D.sz);
  const int K = D.K, nxy = D.nxy, kz = D.kz, kx = D.kx, ky = D.ky, S = D.S;
  const bool count = D.tile_counts != nullptr;
  const bool ws = D.layout == SPIRA_B200_LAYOUT_WS;

  if (tid < kTile) s_tgt[tid] = tid < nvalid ? D.tgt[t0 + tid] : KeyT(0);
  for (int k = tid; k < K; k += kSearchThreads) s_cnt[k] = 0;

  // ---- one source window per x offset: 2 * kx warp-cooperative searches ----------------------------------------------
  for (int b = warp; b < 2 * kx; b += kSearchThreads / 32) {
    const int ix = b >> 1;
    const KeyT off_lo = xy_offset(D, ix, 0), off_hi = xy_offset(D, ix, ky - 1);
    const KeyT qf = first + off_lo, ql = last + off_lo, qh = last + off_hi;
    const KeyT qmax = qh + static_cast<KeyT>(kz - 1) * sz;
    // the queries of this x offset are ordered like (t, iy, iz) unless one of them wraps around the key range
    const bool irregular = !(qf <= ql && ql <= qh && qh <= qmax) || S == 0;
    int r;
    if (irregular) {
      r = (b & 1) ? S : 0;
    } else if (b & 1) {
      r = (qmax == ~KeyT(0)) ? S : warp_lower_bound(src, S, static_cast<KeyT>(qmax + 1), lane);
    } else {
      r = warp_lower_bound(src, S, qf, lane);
    }
    if (lane == 0) {
      if (b & 1) s_hi[ix] = r; else { s_lo[ix] = r; s_irregular[ix] = irregular; }
    }
  }
  __syncthreads();

  // ---- one (target, xy offset) column per thread and turn --------------------------------------------------------------
  // One column: a lower bound for the lowest z inside the window of the column's x offset, then the kz answers by
  // walking on (z is the fastest key field).  `row` points at the first entry of the column in the map, `step` is the
  // distance between its z entries; hits are counted per map row.
  auto column = [&](int tl, int o, int ix, KeyT off, int32_t *__restrict__ out, int step, int k_first, int k_step) {
    const bool valid = tl < nvalid;
    const int lo = s_lo[ix], hi = s_hi[ix];
    KeyT q = s_tgt[tl] + off;
    if (s_irregular[ix] == 0) {
      int i = valid ? lower_bound(src, lo, hi, q) : hi;
#pragma unroll 1
      for (int iz = 0; iz < kz; ++iz) {
        int r = -1;
        KeyT v = KeyT(0);
        while (i < hi && (v = __ldg(src + i)) < q) ++i;
        if (i < hi && v == q) r = i;
        out[iz * step] = r;
        if (count) {
          if (ws) {
            const unsigned m = __ballot_sync(0xffffffffu, r >= 0);  // (the 32 columns of a warp share the offset)
            if (lane == 0 && m) atomicAdd(&s_cnt[k_first + iz * k_step], __popc(m));
          } else if (r >= 0) {
            atomicAdd(&s_cnt[k_first + iz * k_step], 1);
          }
        }
        q += sz;
      }
    } else {
      // some query of this x offset wraps around the key range: every z is an exact lookup in the whole array
#pragma unroll 1
      for (int iz = 0; iz < kz; ++iz) {
        int r = -1;
        if (valid) {
          const int i = lower_bound(src, 0, S, q);
          if (i < S && __ldg(src + i) == q) r = i;
        }
        out[iz * step] = r;
        if (count) {
          if (ws) {
            const unsigned m = __ballot_sync(0xffffffffu, r >= 0);
            if (lane == 0 && m) atomicAdd(&s_cnt[k_first + iz * k_step], __popc(m));
          } else if (r >= 0) {
            atomicAdd(&s_cnt[k_first + iz * k_step], 1);
          }
        }
        q += sz;
      }
    }
  };

  if (ws) {
    // [K][T_al]: thread = target tid % 128 of offsets tid / 128, tid / 128 + 2, ...: consecutive threads write consecutive
    // entries of one map row.  Natural row k = kz*o + iz may be stored elsewhere (row_perm).
    const int tl = tid & (kTile - 1);
    int32_t *const base = D.map + t0 + tl;
    for (int o = tid >> 7; o < nxy; o += kSearchThreads / kTile) {
      const int ix = o / ky, iy = o - ix * ky;
      const KeyT off = xy_offset(D, ix, iy);
      if (D.row_perm == nullptr) {
        column(tl, o, ix, off, base + static_cast<int64_t>(kz * o) * D.T_al, D.T_al, kz * o, 1);
      } else {
        // permuted rows are not equidistant: one z at a time
        const bool valid = tl < nvalid;
        const int lo = s_lo[ix], hi = s_hi[ix];
        const bool irregular = s_irregular[ix] != 0;
        KeyT q = s_tgt[tl] + off;
        int i = (valid && !irregular) ? lower_bound(src, lo, hi, q) : hi;
#pragma unroll 1
        for (int iz = 0; iz < kz; ++iz) {
          int r = -1;
          if (valid && irregular) {
            const int j = lower_bound(src, 0, S, q);
            if (j < S && __ldg(src + j) == q) r = j;
          } else {
            KeyT v = KeyT(0);
            while (i < hi && (v = __ldg(src + i)) < q) ++i;
            if (i < hi && v == q) r = i;
          }
          const int k_ws = D.row_perm[kz * o + iz];
          base[static_cast<int64_t>(k_ws) * D.T_al] = r;
          if (count) {
            const unsigned m = __ballot_sync(0xffffffffu, r >= 0);
            if (lane == 0 && m) atomicAdd(&s_cnt[k_ws], __popc(m));
          }
          q += sz;
        }
      }
    }
  } else {
    // [T_al][K]: thread = xy offset tid % nxy of targets tid / nxy, + 256 / nxy, ...: consecutive threads write runs of nxy
    // consecutive entries (column iz*nxy + o of a row).  Offset, window and x offset are fixed per thread.
    const int per_turn = kSearchThreads / nxy;
    if (tid < per_turn * nxy) {
      const int o = tid % nxy, sub = tid / nxy;
      const int ix = o / ky, iy = o - ix * ky;
      const KeyT off = xy_offset(D, ix, iy);
      for (int tl = sub; tl < kTile; tl += per_turn)
        column(tl, o, ix, off, D.map + static_cast<int64_t>(t0 + tl) * K + o, nxy, kz * o, 1);
    }
  }
  __syncthreads();
  if (count)
    for (int k = tid; k < K; k += kSearchThreads) D.tile_counts[static_cast<int64_t>(k) * D.n_tiles + lt] = s_cnt[k];
}

// ---- weight-stationary post-processing ------------------------------------------------------

// One CTA per map row: exclusive scan of the row's per-tile counts.
__device__ __forceinline__ void ws_row_scan_body(const int32_t *__restrict__ tile_counts, int64_t n_tiles,
                                                 int32_t *__restrict__ tile_base, int32_t *__restrict__ nbsizes, int k) {
  __shared__ int s_warp[8];
  __shared__ int s_carry;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_carry = 0;
  __syncthreads();
  for (int64_t b = 0; b < n_tiles; b += 256) {
    int64_t i = b + tid;
    int v = i < n_tiles ? tile_counts[k * n_tiles + i] : 0;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    int wp = 0;
    for (int w = 0; w < warp; ++w) wp += s_warp[w];
    int carry = s_carry;
    if (i < n_tiles) tile_base[k * n_tiles + i] = carry + wp + x - v;
    __syncthreads();
    if (tid == 255) s_carry = carry + wp + x;
    __syncthreads();
  }
  if (tid == 0) nbsizes[k] = s_carry;
}

__global__ void __launch_bounds__(256) ws_row_scan_kernel(const int32_t *__restrict__ tile_counts, int64_t n_tiles,
                                                           int32_t *__restrict__ tile_base,
                                                           int32_t *__restrict__ nbsizes) {
  ws_row_scan_body(tile_counts, n_tiles, tile_base, nbsizes, blockIdx.x);
}

__device__ __forceinline__ void ws_addr_body(const int32_t *__restrict__ nbsizes, int rows, int32_t *__restrict__ naddrs,
                                             int32_t *__restrict__ qnaddrs, int32_t *__restrict__ sizes) {
  int acc = 0, qacc = 0;
  for (int k = 0; k < rows; ++k) {
    naddrs[k] = acc;
    qnaddrs[k] = qacc;
    int v = nbsizes[k];
    acc += v;
    qacc += (v + 127) / 128 * 128;
  }
  naddrs[rows] = acc;
  qnaddrs[rows] = qacc;
  sizes[0] = acc;
  sizes[1] = qacc;
}

__global__ void ws_addr_kernel(const int32_t *__restrict__ nbsizes, int rows, int32_t *__restrict__ naddrs,
                               int32_t *__restrict__ qnaddrs, int32_t *__restrict__ sizes) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  ws_addr_body(nbsizes, rows, naddrs, qnaddrs, sizes);
}

// compaction of one 128-target tile of one row, order preserved.
__device__ __forceinline__ void ws_pairs_body(const int32_t *__restrict__ map_ws, int64_t T_al, int64_t n_tiles,
                                              const int32_t *__restrict__ naddrs, const int32_t *__restrict__ tile_base,
                                              int32_t *__restrict__ in_idx, int32_t *__restrict__ out_idx, int tile, int k) {
  __shared__ int s_warp[kTile / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = static_cast<int64_t>(tile) * kTile + tid;
  const int v = map_ws[k * T_al + t];
  const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
  if (lane == 0) s_warp[warp] = __popc(m);
  __syncthreads();
  if (v < 0) return;
  int rank = __popc(m & ((1u << lane) - 1));
  for (int w = 0; w < warp; ++w) rank += s_warp[w];
  const int64_t pos = static_cast<int64_t>(naddrs[k]) + tile_base[k * n_tiles + tile] + rank;
  in_idx[pos] = v;
  out_idx[pos] = static_cast<int32_t>(t);
}

// grid (n_tiles, rows)
__global__ void __launch_bounds__(kTile) ws_pairs_kernel(const int32_t *__restrict__ map_ws, int64_t T_al,
                                                          int64_t n_tiles, const int32_t *__restrict__ naddrs,
                                                          const int32_t *__restrict__ tile_base,
                                                          int32_t *__restrict__ in_idx, int32_t *__restrict__ out_idx) {
  ws_pairs_body(map_ws, T_al, n_tiles, naddrs, tile_base, in_idx, out_idx, blockIdx.x, blockIdx.y);
}

// ---- the same three steps for up to SPIRA_B200_MAX_MAPS maps per launch ---------------------------------------------
struct WsBatch {
  const int32_t *map_ws[SPIRA_B200_MAX_MAPS];
  const int32_t *tile_counts[SPIRA_B200_MAX_MAPS];
  int32_t *nbsizes[SPIRA_B200_MAX_MAPS], *naddrs[SPIRA_B200_MAX_MAPS], *qnaddrs[SPIRA_B200_MAX_MAPS];
  int32_t *tile_base[SPIRA_B200_MAX_MAPS], *sizes[SPIRA_B200_MAX_MAPS];
  int32_t *in_idx[SPIRA_B200_MAX_MAPS], *out_idx[SPIRA_B200_MAX_MAPS];
  int32_t T_al[SPIRA_B200_MAX_MAPS], K[SPIRA_B200_MAX_MAPS], rows[SPIRA_B200_MAX_MAPS];
  int32_t scan_base[SPIRA_B200_MAX_MAPS + 1];    // first CTA of map m in the row-scan launch (one CTA per map row)
  int32_t pairs_base[SPIRA_B200_MAX_MAPS + 1];   // first CTA of map m in the compaction launch (tiles x listed rows)
  int32_t n_maps;
};

__global__ void __launch_bounds__(256) ws_row_scan_batched_kernel(const __grid_constant__ WsBatch B) {
  pdl_trigger();
  pdl_wait();
  int m = 0;
  while (m + 1 < B.n_maps && static_cast<int>(blockIdx.x) >= B.scan_base[m + 1]) ++m;
  ws_row_scan_body(B.tile_counts[m], B.T_al[m] / kTile, B.tile_base[m], B.nbsizes[m], blockIdx.x - B.scan_base[m]);
}

__global__ void ws_addr_batched_kernel(const __grid_constant__ WsBatch B) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  if (threadIdx.x == 0) ws_addr_body(B.nbsizes[m], B.rows[m], B.naddrs[m], B.qnaddrs[m], B.sizes[m]);
}

__global__ void __launch_bounds__(kTile) ws_pairs_batched_kernel(const __grid_constant__ WsBatch B) {
  pdl_trigger();
  pdl_wait();
  int m = 0;
  while (m + 1 < B.n_maps && static_cast<int>(blockIdx.x) >= B.pairs_base[m + 1]) ++m;
  const int local = blockIdx.x - B.pairs_base[m];
  const int n_tiles = B.T_al[m] / kTile;
  ws_pairs_body(B.map_ws[m], B.T_al[m], n_tiles, B.naddrs[m], B.tile_base[m], B.in_idx[m], B.out_idx[m], local % n_tiles,
                local / n_tiles);
}

__global__ void __launch_bounds__(kTile) masks_kernel(const int32_t *__restrict__ map_ws, int64_t S, int64_t T,
                                                       int64_t T_al, int64_t n_tiles,
                                                       const int32_t *__restrict__ tile_base,
                                                       int32_t *__restrict__ source_masks,
                                                       int32_t *__restrict__ target_masks) {
  __shared__ int s_warp[kTile / 32];
  const int tile = blockIdx.x, k = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = static_cast<int64_t>(tile) * kTile + tid;
  const int v = map_ws[k * T_al + t];
  const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
  if (lane == 0) s_warp[warp] = __popc(m);
  __syncthreads();
  if (v < 0) return;
  int rank = __popc(m & ((1u << lane) - 1)) + tile_base[k * n_tiles + tile];
  for (int w = 0; w < warp; ++w) rank += s_warp[w];
  source_masks[k * S + v] = rank;
  target_masks[k * T + t] = rank;
}

// Mask format of a mirrored map (csrc/spira/cuda/kernels/generate_masks_from_kernel_map.cuh:36-62): only the first
// `rows_listed` rows of the `rows_masks` mask rows are ranked; the pair (s, t) of listed row o with rank r also enters the
// mirrored row rows_masks - 1 - o with the roles exchanged (source t, target s), unless o is its own mirror image.
__global__ void __launch_bounds__(kTile) masks_half_kernel(const int32_t *__restrict__ map_rows, int rows_masks, int64_t S,
                                                            int64_t T, int64_t T_al, int64_t n_tiles,
                                                            const int32_t *__restrict__ tile_base,
                                                            int32_t *__restrict__ source_masks,
                                                            int32_t *__restrict__ target_masks) {
  __shared__ int s_warp[kTile / 32];
  const int tile = blockIdx.x, k = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = static_cast<int64_t>(tile) * kTile + tid;
  const int v = map_rows[k * T_al + t];
  const unsigned m = __ballot_sync(0xffffffffu, v >= 0);
  if (lane == 0) s_warp[warp] = __popc(m);
  __syncthreads();
  if (v < 0) return;
  int rank = __popc(m & ((1u << lane) - 1)) + tile_base[k * n_tiles + tile];
  for (int w = 0; w < warp; ++w) rank += s_warp[w];
  source_masks[k * S + v] = rank;
  target_masks[k * T + t] = rank;
  const int km = rows_masks - 1 - k;
  if (km != k) {
    source_masks[km * S + t] = rank;
    target_masks[km * T + v] = rank;
  }
}

// Pair lists from the mask format alone (the inverse of the kernels above): sizes[k] for all `rows` mask rows from
// nbsizes[n_sizes] (n_sizes == rows, or a mirrored half whose missing rows repeat the listed ones back to front), prefix
// sums naddrs / qnaddrs, then in_idx[naddrs[k] + r] = s for source_masks[k][s] = r and likewise out_idx from the targets.
__global__ void masks_addr_kernel(const int32_t *__restrict__ nbsizes, int n_sizes, int rows, int32_t *__restrict__ naddrs,
                                  int32_t *__restrict__ qnaddrs) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int acc = 0, qacc = 0;
  for (int k = 0; k < rows; ++k) {
    naddrs[k] = acc;
    qnaddrs[k] = qacc;
    const int v = nbsizes[k < n_sizes ? k : rows - 1 - k];
    acc += v;
    qacc += (v + 127) / 128 * 128;
  }
  naddrs[rows] = acc;
  qnaddrs[rows] = qacc;
}

__global__ void __launch_bounds__(256) lists_from_masks_kernel(const int32_t *__restrict__ masks, int64_t n,
                                                                const int32_t *__restrict__ naddrs,
                                                                int32_t *__restrict__ idx) {
  const int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int k = blockIdx.y;
  if (i >= n) return;
  const int r = masks[k * n + i];
  if (r >= 0) idx[naddrs[k] + r] = static_cast<int32_t>(i);
}

__global__ void __launch_bounds__(256) invert_os_kernel(const int32_t *__restrict__ map_os, int64_t n, int K,
                                                         int32_t *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  int v = map_os[i];
  if (v < 0) return;
  out[static_cast<int64_t>(v) * K + (i % K)] = static_cast<int32_t>(i / K);
}

__global__ void __launch_bounds__(256) transpose_kernel(const int32_t *__restrict__ in, int64_t rows, int64_t cols,
                                                         int32_t *__restrict__ out) {
  __shared__ int32_t tile[32][33];
  int64_t c0 = blockIdx.x * 32ll, r0 = blockIdx.y * 32ll;
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    int64_t r = r0 + j, c = c0 + tx;
    if (r < rows && c < cols) tile[j][tx] = in[r * cols + c];
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    int64_t c = c0 + j, r = r0 + tx;
    if (r < rows && c < cols) out[c * rows + r] = tile[tx][j];
  }
}

template <typename KeyT>
int search_impl(const spira_b200_kmap_desc *descs, int n_maps, cudaStream_t stream) {
  SearchParams<KeyT> P;
  P.n_maps = 0;
  int tiles = 0;
  for (int i = 0; i < n_maps; ++i) {
    const spira_b200_kmap_desc &d = descs[i];
    SB_CHECK_ARG(d.num_sources >= 0 && d.num_sources < (int64_t(1) << 31) && d.num_targets >= 0 &&
                     d.num_targets < (int64_t(1) << 31) - 128,
                 "kmap_search: map %d has sizes out of range", i);
    const int kx = d.kernel_size[0], ky = d.kernel_size[1], kz = d.kernel_size[2];
    SB_CHECK_ARG(kx >= 1 && ky >= 1 && kz >= 1, "kmap_search: map %d has a non-positive kernel size", i);
    SB_CHECK_ARG(kx <= 8 && kx * ky <= kMaxXY && kx * ky * kz <= kMaxK,
                 "kmap_search: map %d kernel %dx%dx%d exceeds 8 in x / %d xy / %d total offsets", i, kx, ky, kz, kMaxXY, kMaxK);
    SB_CHECK_ARG(d.source_stride[0] >= 1 && d.source_stride[1] >= 1 && d.source_stride[2] >= 1,
                 "kmap_search: map %d has a non-positive stride", i);
    SB_CHECK_ARG(d.layout == SPIRA_B200_LAYOUT_OS || d.layout == SPIRA_B200_LAYOUT_WS, "kmap_search: map %d layout %d", i,
                 d.layout);
    if (d.num_targets == 0) continue;
    SB_CHECK_ARG(d.targets && d.map && (d.sources || d.num_sources == 0), "kmap_search: map %d has a null pointer", i);
    MapDesc<KeyT> &m = P.m[P.n_maps++];
    m.src = static_cast<const KeyT *>(d.sources);
    m.tgt = static_cast<const KeyT *>(d.targets);
    m.map = d.map;
    m.tile_counts = d.tile_counts;
    m.row_perm = d.layout == SPIRA_B200_LAYOUT_WS ? d.row_perm : nullptr;
    m.S = static_cast<int32_t>(d.num_sources);
    m.T = static_cast<int32_t>(d.num_targets);
    m.T_al = static_cast<int32_t>(align128(d.num_targets));
    m.n_tiles = m.T_al / kTile;
    m.kx = kx; m.ky = ky; m.kz = kz; m.nxy = kx * ky; m.K = kx * ky * kz;
    m.x0 = (kx % 2 == 1) ? -(kx / 2) : -(kx / 2) + 1;
    m.y0 = (ky % 2 == 1) ? -(ky / 2) : -(ky / 2) + 1;
    m.z0 = (kz % 2 == 1) ? -(kz / 2) : -(kz / 2) + 1;
    m.sx = d.source_stride[0]; m.sy = d.source_stride[1]; m.sz = d.source_stride[2];
    m.layout = d.layout;
    m.tile_begin = tiles;
    tiles += m.n_tiles;
  }
  if (tiles == 0) return SPIRA_B200_OK;
  SB_CHECK_CUDA(launch_dependent(kmap_search_kernel<KeyT>, dim3(tiles), dim3(kSearchThreads), 0, stream, P));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

}  // namespace sb

using namespace sb;

extern "C" int spira_b200_kmap_search(const spira_b200_kmap_desc *host_descs, int n_maps, int key_bytes,
                                      void *stream) {
  SB_CHECK_ARG(n_maps >= 0 && n_maps <= SPIRA_B200_MAX_MAPS, "kmap_search: n_maps=%d not in [0,%d]", n_maps,
               SPIRA_B200_MAX_MAPS);
  if (n_maps == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(host_descs != nullptr, "kmap_search: null descriptor array");
  if (key_bytes == 4) return search_impl<uint32_t>(host_descs, n_maps, as_stream(stream));
  if (key_bytes == 8) return search_impl<uint64_t>(host_descs, n_maps, as_stream(stream));
  return fail(SPIRA_B200_ERR_ARGUMENT, "key_bytes must be 4 or 8, got %d", key_bytes);
}

extern "C" int spira_b200_kmap_ws_sizes(const int32_t *tile_counts, int rows, int64_t n_tiles, int32_t *nbsizes,
                                        int32_t *naddrs, int32_t *qnaddrs, int32_t *tile_base, int32_t *sizes,
                                        void *stream) {
  SB_CHECK_ARG(rows >= 1 && rows <= kMaxK && n_tiles >= 0, "kmap_ws_sizes: rows=%d n_tiles=%lld", rows, (long long)n_tiles);
  SB_CHECK_ARG(nbsizes && naddrs && qnaddrs && sizes && (n_tiles == 0 || (tile_counts && tile_base)),
               "kmap_ws_sizes: null pointer");
  ws_row_scan_kernel<<<rows, 256, 0, as_stream(stream)>>>(tile_counts, n_tiles, tile_base, nbsizes);
  SB_CHECK_LAUNCH();
  ws_addr_kernel<<<1, 32, 0, as_stream(stream)>>>(nbsizes, rows, naddrs, qnaddrs, sizes);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_ws_pairs(const int32_t *map_ws, int rows, int64_t aligned_targets,
                                        const int32_t *naddrs, const int32_t *tile_base, int32_t *in_idx,
                                        int32_t *out_idx, void *stream) {
  SB_CHECK_ARG(rows >= 1 && rows <= kMaxK && aligned_targets >= 0 && aligned_targets % 128 == 0,
               "kmap_ws_pairs: rows=%d aligned_targets=%lld", rows, (long long)aligned_targets);
  if (aligned_targets == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(map_ws && naddrs && tile_base && in_idx && out_idx, "kmap_ws_pairs: null pointer");
  int64_t n_tiles = aligned_targets / kTile;
  dim3 grid(static_cast<unsigned>(n_tiles), static_cast<unsigned>(rows));
  ws_pairs_kernel<<<grid, kTile, 0, as_stream(stream)>>>(map_ws, aligned_targets, n_tiles, naddrs, tile_base, in_idx,
                                                         out_idx);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_ws_lists(const spira_b200_ws_desc *descs, int n_maps, void *stream) {
  SB_CHECK_ARG(n_maps >= 0 && n_maps <= SPIRA_B200_MAX_MAPS, "kmap_ws_lists: n_maps=%d (at most %d per call)", n_maps,
               SPIRA_B200_MAX_MAPS);
  if (n_maps == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(descs != nullptr, "kmap_ws_lists: null descriptor array");
  WsBatch B{};
  int64_t scan = 0, pairs = 0;
  for (int m = 0; m < n_maps; ++m) {
    const spira_b200_ws_desc &d = descs[m];
    SB_CHECK_ARG(d.K >= 1 && d.K <= kMaxK && d.rows >= 1 && d.rows <= d.K, "kmap_ws_lists: map %d: K=%d rows=%d", m, d.K, d.rows);
    SB_CHECK_ARG(d.aligned_targets > 0 && d.aligned_targets % 128 == 0 && d.aligned_targets < (int64_t(1) << 31),
                 "kmap_ws_lists: map %d: aligned_targets=%lld", m, (long long)d.aligned_targets);
    SB_CHECK_ARG(d.map_ws && d.tile_counts && d.nbsizes && d.naddrs && d.qnaddrs && d.tile_base && d.sizes && d.in_idx && d.out_idx,
                 "kmap_ws_lists: map %d: null pointer", m);
    B.map_ws[m] = d.map_ws; B.tile_counts[m] = d.tile_counts; B.nbsizes[m] = d.nbsizes; B.naddrs[m] = d.naddrs;
    B.qnaddrs[m] = d.qnaddrs; B.tile_base[m] = d.tile_base; B.sizes[m] = d.sizes; B.in_idx[m] = d.in_idx; B.out_idx[m] = d.out_idx;
    B.T_al[m] = static_cast<int32_t>(d.aligned_targets); B.K[m] = d.K; B.rows[m] = d.rows;
    B.scan_base[m] = static_cast<int32_t>(scan); B.pairs_base[m] = static_cast<int32_t>(pairs);
    scan += d.K;
    pairs += (d.aligned_targets / kTile) * d.rows;
  }
  SB_CHECK_ARG(pairs < (int64_t(1) << 31), "kmap_ws_lists: too many tiles in one call");
  B.scan_base[n_maps] = static_cast<int32_t>(scan); B.pairs_base[n_maps] = static_cast<int32_t>(pairs);
  B.n_maps = n_maps;
  cudaStream_t st = as_stream(stream);
  SB_CHECK_CUDA(launch_dependent(ws_row_scan_batched_kernel, dim3(static_cast<unsigned>(scan)), dim3(256), 0, st, B));
  SB_CHECK_LAUNCH();
  SB_CHECK_CUDA(launch_dependent(ws_addr_batched_kernel, dim3(n_maps), dim3(32), 0, st, B));
  SB_CHECK_LAUNCH();
  SB_CHECK_CUDA(launch_dependent(ws_pairs_batched_kernel, dim3(static_cast<unsigned>(pairs)), dim3(kTile), 0, st, B));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_masks(const int32_t *map_ws, int rows_total, int64_t num_sources, int64_t num_targets,
                                     int64_t aligned_targets, const int32_t *tile_base, int32_t *source_masks,
                                     int32_t *target_masks, void *stream) {
  SB_CHECK_ARG(rows_total >= 1 && rows_total <= kMaxK && aligned_targets % 128 == 0 && num_targets <= aligned_targets,
               "kmap_masks: bad sizes");
  SB_CHECK_ARG(source_masks && target_masks, "kmap_masks: null pointer");
  SB_CHECK_CUDA(cudaMemsetAsync(source_masks, 0xFF, sizeof(int32_t) * rows_total * num_sources, as_stream(stream)));
  SB_CHECK_CUDA(cudaMemsetAsync(target_masks, 0xFF, sizeof(int32_t) * rows_total * num_targets, as_stream(stream)));
  if (aligned_targets == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(map_ws && tile_base, "kmap_masks: null pointer");
  int64_t n_tiles = aligned_targets / kTile;
  dim3 grid(static_cast<unsigned>(n_tiles), static_cast<unsigned>(rows_total));
  masks_kernel<<<grid, kTile, 0, as_stream(stream)>>>(map_ws, num_sources, num_targets, aligned_targets, n_tiles,
                                                      tile_base, source_masks, target_masks);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_masks_half(const int32_t *map_rows, const int32_t *tile_base_rows, int rows_listed,
                                          int rows_masks, int64_t num_sources, int64_t num_targets, int64_t aligned_targets,
                                          int32_t *source_masks, int32_t *target_masks, void *stream) {
  SB_CHECK_ARG(rows_masks >= 1 && rows_masks <= kMaxK && rows_listed >= 0 && 2 * rows_listed <= rows_masks + 1 &&
                   2 * rows_listed >= rows_masks && aligned_targets % 128 == 0 && num_targets <= aligned_targets,
               "kmap_masks_half: bad sizes (rows_listed must be rows_masks / 2, rounded up)");
  SB_CHECK_ARG(num_sources == num_targets, "kmap_masks_half: a mirrored map has as many sources as targets");
  SB_CHECK_ARG(source_masks && target_masks, "kmap_masks_half: null pointer");
  SB_CHECK_CUDA(cudaMemsetAsync(source_masks, 0xFF, sizeof(int32_t) * rows_masks * num_sources, as_stream(stream)));
  SB_CHECK_CUDA(cudaMemsetAsync(target_masks, 0xFF, sizeof(int32_t) * rows_masks * num_targets, as_stream(stream)));
  if (aligned_targets == 0 || rows_listed == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(map_rows && tile_base_rows, "kmap_masks_half: null pointer");
  const int64_t n_tiles = aligned_targets / kTile;
  dim3 grid(static_cast<unsigned>(n_tiles), static_cast<unsigned>(rows_listed));
  masks_half_kernel<<<grid, kTile, 0, as_stream(stream)>>>(map_rows, rows_masks, num_sources, num_targets, aligned_targets, n_tiles,
                                                           tile_base_rows, source_masks, target_masks);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_lists_from_masks(const int32_t *source_masks, const int32_t *target_masks, const int32_t *nbsizes,
                                                int n_sizes, int rows, int64_t num_sources, int64_t num_targets, int32_t *naddrs,
                                                int32_t *qnaddrs, int32_t *in_idx, int32_t *out_idx, void *stream) {
  SB_CHECK_ARG(rows >= 1 && rows <= kMaxK && (n_sizes == rows || n_sizes == (rows + 1) / 2) && num_sources >= 0 && num_targets >= 0,
               "kmap_lists_from_masks: rows=%d n_sizes=%d (the sizes cover all mask rows or their first half)", rows, n_sizes);
  SB_CHECK_ARG(nbsizes && naddrs && qnaddrs, "kmap_lists_from_masks: null pointer");
  cudaStream_t st = as_stream(stream);
  masks_addr_kernel<<<1, 32, 0, st>>>(nbsizes, n_sizes, rows, naddrs, qnaddrs);
  SB_CHECK_LAUNCH();
  if (num_sources > 0 && num_targets > 0) {
    SB_CHECK_ARG(source_masks && target_masks && in_idx && out_idx, "kmap_lists_from_masks: null pointer");
    lists_from_masks_kernel<<<dim3(static_cast<unsigned>(div_up(num_sources, 256)), static_cast<unsigned>(rows)), 256, 0, st>>>(
        source_masks, num_sources, naddrs, in_idx);
    SB_CHECK_LAUNCH();
    lists_from_masks_kernel<<<dim3(static_cast<unsigned>(div_up(num_targets, 256)), static_cast<unsigned>(rows)), 256, 0, st>>>(
        target_masks, num_targets, naddrs, out_idx);
    SB_CHECK_LAUNCH();
  }
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_convert_transposed_os(const int32_t *map_os, int64_t aligned_targets, int K, int32_t *out,
                                                int64_t aligned_sources, void *stream) {
  SB_CHECK_ARG(K >= 1 && aligned_targets >= 0 && aligned_sources >= 0, "convert_transposed_os: bad sizes");
  if (aligned_sources > 0) {
    SB_CHECK_ARG(out != nullptr, "convert_transposed_os: null output");
    SB_CHECK_CUDA(cudaMemsetAsync(out, 0xFF, sizeof(int32_t) * aligned_sources * K, as_stream(stream)));
  }
  int64_t n = aligned_targets * K;
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(map_os != nullptr, "convert_transposed_os: null input");
  SB_CHECK_CUDA(launch_dependent(invert_os_kernel, dim3(static_cast<unsigned>(div_up(n, 256))), dim3(256), 0, as_stream(stream), map_os, n, K, out));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_transpose_map(const int32_t *in, int64_t rows, int64_t cols, int32_t *out, void *stream) {
  SB_CHECK_ARG(rows >= 0 && cols >= 0, "transpose_map: bad sizes");
  if (rows == 0 || cols == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(in && out, "transpose_map: null pointer");
  dim3 grid(static_cast<unsigned>(div_up(cols, 32)), static_cast<unsigned>(div_up(rows, 32)));
  transpose_kernel<<<grid, 256, 0, as_stream(stream)>>>(in, rows, cols, out);
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

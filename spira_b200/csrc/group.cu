// Grouping the targets of an output-stationary kernel map by neighbour pattern.
//
// The output-stationary convolution processes a tile of consecutive map rows per (weight offset, 64 input channels)
// chunk and skips a chunk only if NO row of the tile has a neighbour at that offset.  In spatial order nearly every
// (tile, offset) pair has some neighbour (97 % on LiDAR-like scenes) although only ~30 % of the individual rows do,
// so ~3.3x more rows are multiplied than there are pairs.  Rows with the same set of present offsets need exactly the
// same chunks: sorting the rows by their K-bit presence mask (fullest first) makes tiles homogeneous and the ratio of
// processed rows to pairs drops to ~1.2.  The convolution then runs over the re-ordered map and writes output row
// `row_of[i]` for grouped row i; per-tile presence masks tell it which chunks to visit without scanning the tile.
//
// The sort key keeps the 19 highest mask bits beside the 5-bit count of absent offsets: 24 bits are three radix passes
// instead of four, and on LiDAR-like scenes the processed rows per pair grow by less than 0.5 % against the full mask.
//
// The sort is the library's cooperative radix sort (radix_sort.cuh): the keys are generated from the map rows inside its
// first phase, and the digits that are the same for every row are skipped, so a network's maps take three or four 8-bit
// passes inside ONE launch.
//
// The reference has no counterpart: its output-stationary kernel walks the map in target order.
#include "common.cuh"
#include "radix_sort.cuh"

namespace sb {

constexpr int kGroupTile = 128;
constexpr int kGroupMaskBits = 19;    // mask bits kept in the sort key of a map with K <= 27

struct GroupBatch {
  const int32_t *map_os[SPIRA_B200_MAX_MAPS];
  int32_t *grouped_map[SPIRA_B200_MAX_MAPS];
  int32_t *row_of[SPIRA_B200_MAX_MAPS];
  uint32_t *tile_masks[SPIRA_B200_MAX_MAPS];
  int32_t *stats[SPIRA_B200_MAX_MAPS];
  int32_t T[SPIRA_B200_MAX_MAPS], K[SPIRA_B200_MAX_MAPS];
  int32_t row_base[SPIRA_B200_MAX_MAPS + 1];    // first row of map m among the concatenated rows of all maps
  int32_t tile_base[SPIRA_B200_MAX_MAPS + 1];   // first 128-row tile of map m among all tiles
  int32_t pair_base[SPIRA_B200_MAX_MAPS + 1];   // first pair of tiles (one CTA of group_rows_kernel) of map m
  int32_t n_maps;
  int32_t key_bits;                             // bits of a key below the map index: 24, or 32 if some map has K > 27
};

// Sort key of row t of map m: map index on top (the maps stay apart); below it, for K <= 27, K - popcount (fullest rows
// first) and the 19 highest bits of the mask (rows with similar masks adjacent); for larger K the complemented mask.
// Element g of the sort is row g - row_base[m] of map m.
struct GroupKeyGen {
  GroupBatch B;
  __device__ __forceinline__ uint64_t operator()(int g) const {
    int m = 0;
    while (m + 1 < B.n_maps && g >= B.row_base[m + 1]) ++m;
    const int64_t t = g - B.row_base[m];
    const int K = B.K[m];
    const int32_t *row = B.map_os[m] + t * K;
    uint32_t mask = 0;
    for (int k = 0; k < K; ++k) mask |= (row[k] >= 0 ? 1u : 0u) << k;
    const int drop = K > kGroupMaskBits ? K - kGroupMaskBits : 0;
    const uint32_t low = (K <= 27) ? ((static_cast<uint32_t>(K - __popc(mask)) << kGroupMaskBits) | (mask >> drop)) : ~mask;
    if (t == 0) { B.stats[m][0] = 0; B.stats[m][1] = 0; }      // counted by the kernel that follows on the stream
    return (static_cast<uint64_t>(m) << B.key_bits) | low;
  }
};

// One CTA per pair of 128-row tiles: gathers the rows of the map in the new order (through shared memory, so that the
// grouped map is written with coalesced stores), ORs the presence masks of each tile and counts the non-empty
// (tile, offset) pairs for 128-row tiles (stats[0]) and for 256-row tiles (stats[1]).
__global__ void __launch_bounds__(2 * kGroupTile) group_rows_kernel(const __grid_constant__ GroupBatch B,
                                                                     const int32_t *__restrict__ order) {
  extern __shared__ int32_t s_rows[];   // [256][K]
  __shared__ uint32_t s_mask[2];
  const int tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  int m = 0;
  while (m + 1 < B.n_maps && static_cast<int>(blockIdx.x) >= B.pair_base[m + 1]) ++m;
  const int tile0 = 2 * (blockIdx.x - B.pair_base[m]);
  const int n_tiles = B.tile_base[m + 1] - B.tile_base[m];
  const int K = B.K[m], T = B.T[m];
  const int rows_here = (tile0 + 1 < n_tiles ? 2 : 1) * kGroupTile;       // the last pair of a map may hold one tile
  const int64_t g = static_cast<int64_t>(tile0) * kGroupTile + tid;
  if (tid < 2) s_mask[tid] = 0;
  __syncthreads();
  // the sorted values are global row numbers; the rows of map m occupy [row_base[m], row_base[m] + T) of the order
  const int32_t src = g < T ? order[B.row_base[m] + g] - B.row_base[m] : -1;
  if (tid < rows_here) B.row_of[m][g] = src;
  const int32_t *map_os = B.map_os[m];
  // a warp copies its 32 rows one after the other: lane k reads entry k, so that a row costs one request
  const int lane = tid & 31, row0 = tid & ~31;
  uint32_t mask = 0;
  for (int r = 0; r < 32; ++r) {
    const int32_t s_r = __shfl_sync(0xffffffffu, src, r);
    const int32_t v = (s_r >= 0 && lane < K) ? map_os[static_cast<int64_t>(s_r) * K + lane] : -1;
    if (lane < K) s_rows[(row0 + r) * K + lane] = v;
    mask |= __ballot_sync(0xffffffffu, v >= 0);
  }
  if (lane == 0 && mask != 0) atomicOr(&s_mask[tid / kGroupTile], mask);
  __syncthreads();
  int32_t *dst = B.grouped_map[m] + static_cast<int64_t>(tile0) * kGroupTile * K;
  for (int i = tid; i < rows_here * K; i += 2 * kGroupTile) dst[i] = s_rows[i];
  if (tid == 0) {
    B.tile_masks[m][tile0] = s_mask[0];
    if (rows_here > kGroupTile) B.tile_masks[m][tile0 + 1] = s_mask[1];
    const int n128 = __popc(s_mask[0]) + __popc(s_mask[1]), n256 = __popc(s_mask[0] | s_mask[1]);
    if (n128 != 0) {
      atomicAdd(&B.stats[m][0], n128);
      atomicAdd(&B.stats[m][1], n256);
    }
  }
}

static size_t round256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace sb

using namespace sb;

extern "C" int spira_b200_kmap_group_workspace(int64_t total_targets, size_t *bytes) {
  SB_CHECK_ARG(bytes != nullptr, "kmap_group_workspace: null output");
  SB_CHECK_ARG(total_targets >= 0 && total_targets < (int64_t(1) << 31) - 128, "kmap_group: total_targets out of range");
  // [sorted keys][order][workspace of the sort]
  *bytes = round256(total_targets * 8) + round256(total_targets * 4) + sort_workspace_bytes<uint64_t>(total_targets) + 256;
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_kmap_group(const spira_b200_group_desc *descs, int n_maps, void *workspace,
                                     size_t workspace_bytes, void *stream) {
  SB_CHECK_ARG(n_maps >= 0 && n_maps <= SPIRA_B200_MAX_MAPS, "kmap_group: n_maps=%d (at most %d per call)", n_maps,
               SPIRA_B200_MAX_MAPS);
  if (n_maps == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(descs != nullptr, "kmap_group: null descriptor array");
  GroupBatch B{};
  int64_t rows = 0, tiles = 0, pairs = 0;
  int max_K = 1;
  for (int m = 0; m < n_maps; ++m) {
    const spira_b200_group_desc &d = descs[m];
    SB_CHECK_ARG(d.num_targets > 0 && d.num_targets < (int64_t(1) << 31) - 128, "kmap_group: map %d: num_targets out of range", m);
    SB_CHECK_ARG(d.K >= 1 && d.K <= 32, "kmap_group: map %d: K=%d, the presence mask of a row must fit 32 bits", m, d.K);
    SB_CHECK_ARG(d.map_os && d.grouped_map && d.row_of && d.tile_masks && d.stats, "kmap_group: map %d: null pointer", m);
    B.map_os[m] = d.map_os; B.grouped_map[m] = d.grouped_map; B.row_of[m] = d.row_of; B.tile_masks[m] = d.tile_masks;
    B.stats[m] = d.stats;
    B.T[m] = static_cast<int32_t>(d.num_targets); B.K[m] = d.K;
    B.row_base[m] = static_cast<int32_t>(rows); B.tile_base[m] = static_cast<int32_t>(tiles);
    B.pair_base[m] = static_cast<int32_t>(pairs);
    rows += d.num_targets;
    tiles += div_up(d.num_targets, kGroupTile);
    pairs += div_up(d.num_targets, 2 * kGroupTile);
    max_K = d.K > max_K ? d.K : max_K;
  }
  SB_CHECK_ARG(rows < (int64_t(1) << 31) - 128, "kmap_group: %lld rows in one call", (long long)rows);
  B.row_base[n_maps] = static_cast<int32_t>(rows);
  B.tile_base[n_maps] = static_cast<int32_t>(tiles);
  B.pair_base[n_maps] = static_cast<int32_t>(pairs);
  B.n_maps = n_maps;
  B.key_bits = max_K <= 27 ? 5 + kGroupMaskBits : 32;
  size_t need = 0;
  spira_b200_kmap_group_workspace(rows, &need);
  SB_CHECK_ARG(workspace != nullptr && workspace_bytes >= need, "kmap_group: workspace of %zu bytes, %zu needed", workspace_bytes, need);
  cudaStream_t st = as_stream(stream);
  unsigned char *w = static_cast<unsigned char *>(workspace);
  w += (256 - reinterpret_cast<uintptr_t>(w) % 256) % 256;
  const size_t col8 = round256(rows * 8), col4 = round256(rows * 4);
  uint64_t *keys_sorted = reinterpret_cast<uint64_t *>(w);
  int32_t *order = reinterpret_cast<int32_t *>(w + col8);
  const int wait_us = spira_b200_get_option("wait_limit_us");
  int rc = radix_sort_generated<uint64_t>(GroupKeyGen{B}, rows, keys_sorted, order, w + col8 + col4, sort_workspace_bytes<uint64_t>(rows),
                                          nullptr, static_cast<unsigned long long>(wait_us > 0 ? wait_us : 1500000) * 1000ull, st,
                                          "kmap_group");
  if (rc != SPIRA_B200_OK) return rc;
  SB_CHECK_CUDA(launch_dependent(group_rows_kernel, dim3(static_cast<unsigned>(pairs)), dim3(2 * kGroupTile),
                                 2 * kGroupTile * max_K * sizeof(int32_t), st, B, order));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

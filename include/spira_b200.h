/*
 * spira_b200 -- C ABI of the B200-native sparse-convolution hot path.
 *
 * Every entry point replaces one function of the reference's pybind module
 * `spira.nn.functional._C` (SPIN-Research-Group/Spira); the reference interface each one
 * stands in for is cited as  file:line  relative to the reference's `source/` directory.
 *
 * Conventions
 *   - plain pointers and sizes only; all data pointers are DEVICE pointers unless the name
 *     starts with `host_`;
 *   - every call is stream-ordered on `stream` (a cudaStream_t passed as void*) and never
 *     synchronises, allocates or frees device memory: outputs and scratch are caller-owned;
 *   - return value 0 = success, negative = error; spira_b200_last_error() returns the
 *     message of the last failing call made by the calling thread;
 *   - `key_bytes` is 4 (x12|y12|z8) or 8 (x24|y24|z16), z in the low bits
 *     (csrc/spira/compress_layout.h:12-44).
 */
#ifndef SPIRA_B200_H_
#define SPIRA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPIRA_B200_OK 0
#define SPIRA_B200_ERR_ARGUMENT (-1)
#define SPIRA_B200_ERR_CUDA (-2)
#define SPIRA_B200_ERR_UNSUPPORTED (-3)
#define SPIRA_B200_ERR_WORKSPACE (-4)

#define SPIRA_B200_LAYOUT_OS 0 /* map[T_al][K], column iz*nxy + o   (kernels/query_sorted.cuh:150,159) */
#define SPIRA_B200_LAYOUT_WS 1 /* map[K][T_al], row kz*o + iz       (kernels/query_sorted.cuh:42,52)   */

#define SPIRA_B200_MAX_MAPS 16   /* maps per batched search launch */
#define SPIRA_B200_MAX_LEVELS 8  /* levels per batched downsample  */

int spira_b200_version(void);
const char *spira_b200_last_error(void);
/* Clears the sticky CUDA error of the calling thread's device, like
 * cuda_reset_error (csrc/spira/torch/cuda_memory_buffer.cu:15-16). */
int spira_b200_reset_error(void);

/* Reads `bytes` from device memory into PINNED host memory without waiting for work that is enqueued on `stream`
 * after this call: `copy_stream` (a different stream) waits for the current end of `stream`, copies, and records
 * `done_event` (a cudaEvent_t of the caller); cudaEventSynchronize(done_event) then tells when the bytes are there.
 * Used for the one host read of a scene (the sizes of the down-sampled levels), so that the level-0 kernel map can be
 * enqueued behind it at once.  No reference counterpart (the reference synchronises the device here). */
int spira_b200_read_back(const void *device_src, void *pinned_dst, size_t bytes, void *stream, void *copy_stream,
                         void *done_event);

/* Run-time options of the calling process (not thread safe; set them before launching work):
 *   "gather_tma"        1: the tensor-core kernels fetch feature rows with TMA gather4, 0 (default): with 16-byte
 *                       cp.async
 *   "os_n256"           1 (default): output-stationary layers with 64 < c_out <= 128 and K <= 32 whose four-stage
 *                       pipeline fits in shared memory (c_out <= 96 for K = 27) run the kernel that puts 256 targets
 *                       on the MMA's N side and the weights on its M side; 0: always 128 targets as M
 *   "os_n256_min_targets" layers with fewer targets than this use the 128-target tiles even where the 256-target kernel
 *                       applies: with few tiles per SM the heaviest tile sets the time and smaller tiles balance better
 *   "wait_limit_us"     limit, in microseconds, of every wait inside the tensor-core kernels (mbarriers, the grid
 *                       barrier of spira_b200_conv_ws_fused); default 1500000.  A kernel whose wait runs out sets its
 *                       `status` word, lets its copies land, releases its tensor memory and returns
 *   "pdl"               1 (default): kernels are launched as programmatic dependents of their predecessor on the
 *                       stream -- their CTAs may be scheduled while the predecessor drains and block, before their first
 *                       access to global data, until it has completed and its writes are visible; what the caller
 *                       observes on the stream is unchanged.  0: ordinary launches
 *   "ws_cooperative_launch"  0 (default): spira_b200_conv_ws_fused is an ordinary dependent launch of at most one CTA per
 *                       SM (its grid barrier only waits for CTAs of its own grid, which become resident as earlier
 *                       kernels drain; the wait is bounded).  1: cudaLaunchCooperativeKernel, which guarantees the
 *                       residency -- for hosts that run other barrier kernels on other streams of the same GPU
 *   "identity_tma"      1 (default): a 1x1x1 layer through the identity map whose sources hold whole groups of 32 channels
 *                       (c_in_a and c_in - c_in_a multiples of 32) runs on the dense kernel: TMA moves 128-row boxes of
 *                       the feature tensors, no producer threads, no map.  0: every identity-map layer runs on the
 *                       output-stationary kernel (the results are equal)
 *   "ws_barrier_skew_once"  test aid: added to the grid-barrier target of the NEXT spira_b200_conv_ws_fused launch only,
 *                       so that its barrier cannot be met and the wait limit is exercised without any fault
 * get_option additionally answers "os_pack_mode": the SPIRA_B200_PACK_* image spira_b200_conv_os expects under
 * the current options.  Unknown names: set_option fails, get_option returns -1. */
int spira_b200_set_option(const char *name, int value);
int spira_b200_get_option(const char *name);

/* Recovery after a spira_b200_conv_ws_fused launch reported an expired wait, and the way to move the fused calls of
 * a device to another stream: synchronises the current device, sets the host's count of grid-barrier arrivals to the
 * device's, and forgets which stream the device's fused calls were bound to.  No reference counterpart. */
int spira_b200_ws_barrier_resync(void);

/* ---- packed keys ------------------------------------------------------------------------- */

/* coords[n][3] int32 -> keys[n]; replaces the Compress kernel (csrc/spira/cuda/kernels/compress.cuh:8-24). */
int spira_b200_pack(const int32_t *coords, int64_t n, int key_bytes, void *keys, void *stream);

/* keys[n] -> coords[n][3]; replaces cuda_unflatten (csrc/spira/torch/cuda_arg_sort_coordinates.cu:41-66). */
int spira_b200_unpack(const void *keys, int64_t n, int key_bytes, int32_t *coords, void *stream);

/* Scratch bytes needed by spira_b200_flatten_sort for n keys. */
int spira_b200_flatten_sort_workspace(int64_t n, int key_bytes, size_t *bytes);

/* pack + ascending unsigned sort + permutation; replaces cuda_flatten_sort
 * (csrc/spira/torch/cuda_arg_sort_coordinates.cu:11-39, cuda/functions/arg_sort_coodrinates.cu:35-88).
 * sorted_keys[n], perm[n] (int32, perm[i] = original row of sorted item i; equal keys keep their input order).
 * ONE cooperative launch: a stable 8-bit radix sort whose passes are separated by grid barriers and which skips the
 * digits that are the same in every key.  The 16-byte aligned workspace is cleared by the call.  `status` (device int32,
 * may be NULL) is set to 1 if a grid-barrier wait ran into the "wait_limit_us" option (the result is then undefined). */
int spira_b200_flatten_sort(const int32_t *coords, int64_t n, int key_bytes, void *sorted_keys, int32_t *perm,
                            void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/* rows_out[i][:] = rows_in[perm[i]][:], row_bytes a multiple of 2; the feature permutation of
 * SparseTensor.order (spira/tensors.py:55-65). */
int spira_b200_permute_rows(const void *rows_in, const int32_t *perm, int64_t n, int64_t row_bytes, void *rows_out,
                            void *stream);

/* 1x1x1 layer with few output channels (a classification head): out[n][c_out] = feats[n][c_in] . weights[c_in][c_out]
 * (+ bias[c_out], may be null), fp16 in and out, fp32 accumulation, one rounding.  The reference sends every 1x1x1
 * layer to torch.mm and adds the bias in a second pass (spira/nn/conv.py:312-316); a head whose c_out is not a
 * multiple of 8 misses the library's aligned kernels there.  c_in a multiple of 8 up to 512 and c_out <= 32, else
 * SPIRA_B200_ERR_UNSUPPORTED (use the library GEMM). */
int spira_b200_pointwise(const void *feats, const void *weights, const void *bias, int64_t n, int c_in, int c_out,
                         void *out, void *stream);

/* Scratch bytes for spira_b200_downsample with n input keys and n_levels levels. */
int spira_b200_downsample_workspace(int64_t n, int key_bytes, int n_levels, size_t *bytes);

/* For each level l: out_keys[l][0 .. counts[l]) = unique(sort(keys & mask(strides[l]))).
 * Replaces cuda_downsample and cuda_streamed_output_generate
 * (csrc/spira/torch/cuda_arg_sort_coordinates.cu:68-200).  host_strides is [n_levels][3]
 * (powers of two), host_out_keys holds n_levels device buffers of n keys each, counts is a
 * device int32[n_levels] written by the call (the caller copies it back to size its views). */
int spira_b200_downsample(const void *keys, int64_t n, int key_bytes, int n_levels, const int32_t *host_strides,
                          void *const *host_out_keys, int32_t *counts, void *workspace, size_t workspace_bytes,
                          void *stream);

/* The same result for keys that are ALREADY SORTED ascending (what spira_b200_flatten_sort returns) and strides
 * that, per axis, equal or double the stride of the level before (level 0 relative to stride 1), without any sort:
 * flooring to a coarser stride disturbs the order only inside a coarse cell, so the final position of every coarse
 * key is a sum of lengths of contiguous ranges of the sorted input, found by binary searches; level l+1 is computed
 * from the output of level l, whose size stays on the device.  The reference sorts every level from scratch
 * (csrc/spira/torch/cuda_arg_sort_coordinates.cu:107-200).  Other stride sequences: SPIRA_B200_ERR_UNSUPPORTED (use
 * spira_b200_downsample).  All levels are ONE cooperative launch (rank pass, grid barrier, compaction, per level).
 * `status` (device int32, may be NULL) is cleared by the call and set to 2 if the input turns out not to be sorted, to 1
 * if a grid-barrier wait ran into the "wait_limit_us" option. */
int spira_b200_downsample_sorted_workspace(int64_t n, int key_bytes, size_t *bytes);
int spira_b200_downsample_sorted(const void *sorted_keys, int64_t n, int key_bytes, int n_levels,
                                 const int32_t *host_strides, void *const *host_out_keys, int32_t *counts,
                                 void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/* ---- kernel-map search -------------------------------------------------------------------- */

typedef struct spira_b200_kmap_desc {
  const void *sources;     /* sorted unique keys [num_sources] */
  const void *targets;     /* sorted unique keys [num_targets] */
  int64_t num_sources;
  int64_t num_targets;
  int32_t kernel_size[3];  /* kx, ky, kz (odd: [-k/2, k/2], even: [-k/2+1, k/2]) */
  int32_t source_stride[3];
  int32_t layout;          /* SPIRA_B200_LAYOUT_OS / _WS */
  int32_t reserved;
  int32_t *map;            /* dense int32 map, T_al = ceil(T/128)*128 rows/columns, -1 = no neighbour */
  int32_t *tile_counts;    /* optional [K][T_al/128] (row order as LAYOUT_WS): hits per 128 targets, or NULL */
  const int32_t *row_perm; /* LAYOUT_WS only, device int32[K] or NULL: natural row k = kz*o + iz is stored as row
                              row_perm[k] of map and tile_counts -- the L1-norm order of the hybrid dataflows
                              (generate_indexes_L1, csrc/spira/torch/cuda_sparse_convolution_mapping.cu:159-209,
                              BinarySearch_kz_hybrid, csrc/spira/cuda/kernels/query_sorted.cuh:58-113) */
} spira_b200_kmap_desc;

/* Builds up to SPIRA_B200_MAX_MAPS kernel maps in ONE launch.  Replaces cuda_binary_search and
 * cuda_binary_search_streamed (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:211-892,
 * 894-1645) and the search kernels (csrc/spira/cuda/kernels/query_sorted.cuh:8-163).
 * Result: exact lookup of tgt[t] + offset (wrapping packed arithmetic) in sources. */
int spira_b200_kmap_search(const spira_b200_kmap_desc *host_descs, int n_maps, int key_bytes, void *stream);

/* Weight-stationary post-processing, phase 1 (sizes).  From tile_counts[K][n_tiles] of the first
 * `rows` rows: nbsizes[rows], naddrs[rows+1], qnaddrs[rows+1] (sizes rounded up to 128),
 * tile_base[rows][n_tiles] (exclusive position of each tile inside its row's list) and
 * sizes[2] = {mapsize, qmapsize}.  Replaces the ReduceByKey + prefix-sum part of
 * BinarySearch_Streamed_Ws[_Half] (csrc/spira/cuda/functions/query_sorted_index.cu:146-209,
 * csrc/spira/cuda/kernels/quantifier_wstat.cuh:8-44). */
int spira_b200_kmap_ws_sizes(const int32_t *tile_counts, int rows, int64_t n_tiles, int32_t *nbsizes,
                             int32_t *naddrs, int32_t *qnaddrs, int32_t *tile_base, int32_t *sizes, void *stream);

/* Phase 2 (pairs): compacts rows [0, rows) of a LAYOUT_WS map into in_idx / out_idx, ordered by
 * (row, target).  Replaces the DeviceSelect::If compaction (query_sorted_index.cu:170-188). */
int spira_b200_kmap_ws_pairs(const int32_t *map_ws, int rows, int64_t aligned_targets, const int32_t *naddrs,
                             const int32_t *tile_base, int32_t *in_idx, int32_t *out_idx, void *stream);

/* spira_b200_kmap_ws_sizes + spira_b200_kmap_ws_pairs for up to SPIRA_B200_MAX_MAPS maps with three launches in
 * total and no host read in between: the pair lists get a capacity the caller can bound without knowing nnz
 * (rows * num_targets entries each); sizes[0..1] = (nnz, nnz rounded per row to 128) stay on the device. */
typedef struct spira_b200_ws_desc {
  const int32_t *map_ws;      /* [K][aligned_targets] */
  const int32_t *tile_counts; /* [K][aligned_targets / 128] from spira_b200_kmap_search */
  int64_t aligned_targets;
  int32_t K;                  /* rows of the map: tile_base and nbsizes are produced for all of them */
  int32_t rows;               /* rows listed and covered by naddrs / qnaddrs: K, or (K + 1) / 2 for mirrored lists */
  int32_t *nbsizes;           /* [K] */
  int32_t *naddrs;            /* [rows + 1] */
  int32_t *qnaddrs;           /* [rows + 1] */
  int32_t *tile_base;         /* [K][aligned_targets / 128] */
  int32_t *sizes;             /* [2] */
  int32_t *in_idx;            /* capacity >= rows * num_targets */
  int32_t *out_idx;
} spira_b200_ws_desc;
int spira_b200_kmap_ws_lists(const spira_b200_ws_desc *descs, int n_maps, void *stream);

/* source_masks[K][S], target_masks[K][T] (rank of each pair inside its row, -1 elsewhere) from a
 * LAYOUT_WS map; both outputs are fully written.  Replaces GenerateMasksFromKernelMap
 * (csrc/spira/cuda/kernels/generate_masks_from_kernel_map.cuh:9-62). */
int spira_b200_kmap_masks(const int32_t *map_ws, int rows_total, int64_t num_sources, int64_t num_targets,
                          int64_t aligned_targets, const int32_t *tile_base, int32_t *source_masks,
                          int32_t *target_masks, void *stream);

/* Mask format of a MIRRORED map: map_rows / tile_base_rows point at the first of `rows_listed` consecutive rows of a
 * LAYOUT_WS map (and of its tile_base); the masks have rows_masks rows (rows_listed = rows_masks / 2, rounded up).  Row o
 * is ranked like spira_b200_kmap_masks does; the pair (s, t) with rank r also enters row rows_masks - 1 - o as
 * source_masks[..][t] = target_masks[..][s] = r.  num_sources must equal num_targets.  Replaces
 * GenerateMasksFromKernelMap_Half (csrc/spira/cuda/kernels/generate_masks_from_kernel_map.cuh:36-62) as used by the
 * submanifold mask dataflow and the hybrid dataflows (csrc/spira/cuda/functions/query_sorted_index.cu:516-640, 647-775). */
int spira_b200_kmap_masks_half(const int32_t *map_rows, const int32_t *tile_base_rows, int rows_listed, int rows_masks,
                               int64_t num_sources, int64_t num_targets, int64_t aligned_targets, int32_t *source_masks,
                               int32_t *target_masks, void *stream);

/* Pair lists from the mask format alone, so that masks built by ANY producer (the reference's own builder included) can
 * feed spira_b200_conv_ws: for all `rows` mask rows, in_idx[naddrs[k] + r] = s where source_masks[k][s] = r >= 0 and
 * out_idx[naddrs[k] + r] = t where target_masks[k][t] = r.  nbsizes holds the list sizes of all rows (n_sizes == rows) or
 * of the first half of a mirrored map (n_sizes == (rows + 1) / 2: row k >= n_sizes has the size of row rows - 1 - k).
 * naddrs / qnaddrs [rows + 1] are written by the call; in_idx / out_idx need room for every pair (at most
 * rows * min(num_sources, num_targets)).  This is what the gather and scatter stages of the reference's mask-format call
 * read the masks for (csrc/spira/cuda/functions/sparse_convolution.cu:1002-1124). */
int spira_b200_kmap_lists_from_masks(const int32_t *source_masks, const int32_t *target_masks, const int32_t *nbsizes,
                                     int n_sizes, int rows, int64_t num_sources, int64_t num_targets, int32_t *naddrs,
                                     int32_t *qnaddrs, int32_t *in_idx, int32_t *out_idx, void *stream);

/* out[S_al][K] (fully written) = inverse of map_os[T_al][K] per column; replaces
 * cuda_convert_transposed_os (csrc/spira/torch/cuda_sparse_convolution_mapping.cu:1809-1830). */
int spira_b200_convert_transposed_os(const int32_t *map_os, int64_t aligned_targets, int K, int32_t *out,
                                     int64_t aligned_sources, void *stream);

/* in-place [rows][cols] -> [cols][rows] transpose of an int32 map into `out` (the
 * `.T.contiguous()` of KernelMapCache.get_kernel_map, spira/nn/conv.py:80-83). */
int spira_b200_transpose_map(const int32_t *in, int64_t rows, int64_t cols, int32_t *out, void *stream);

/* ---- feature compute (fp16 in/out, fp32 accumulate) ---------------------------------------- */

/* Optional per-channel affine + residual + ReLU applied to the fp32 accumulator before the single
 * rounding to fp16:  y = relu?( (acc + bias) * scale + shift + residual ).  Any pointer may be NULL.
 * (The reference applies bias, BatchNorm, the residual add and ReLU as separate passes:
 * spira/nn/conv.py:415-416, spira/nn/normalizations.py:8-10, spira/nn/activations.py:8-18.) */
typedef struct spira_b200_epilogue {
  const void *bias;      /* fp16 [c_out] */
  const float *scale;    /* fp32 [c_out] */
  const float *shift;    /* fp32 [c_out] */
  const void *residual;  /* fp16 [num_targets][c_out] */
  int32_t relu;
  int32_t reserved;
} spira_b200_epilogue;

#define SPIRA_B200_PACK_OS 0 /* reduction index r = k*c_in + c, 64-wide chunks over the whole r range */
#define SPIRA_B200_PACK_WS 1 /* every offset padded to ceil(c_in/64) chunks of its own */

/* 1 if (c_in, c_out, K) can run on the tcgen05 tensor-core kernels, else 0 (SIMT kernels are used). */
int spira_b200_tensor_core_eligible(int K, int c_in, int c_out);

/* Which kernel a layer of this shape runs on under the current options (the dispatch rule of spira_b200_conv_os* /
 * spira_b200_conv_ws* given a packed weight image where one exists); -1 for invalid sizes.  No reference counterpart;
 * the benchmark uses it to attribute measured times to kernels. */
#define SPIRA_B200_KERNEL_SIMT_OS 0 /* conv_os_simt_kernel */
#define SPIRA_B200_KERNEL_STEM_OS 1 /* conv_os_stem_kernel: c_in <= 8, c_out in {16, 32, 64} */
#define SPIRA_B200_KERNEL_TC_OS 2   /* conv_tc_kernel<output-stationary>: 128 targets as the MMA's M operand */
#define SPIRA_B200_KERNEL_N256_OS 3 /* conv_os_n256_kernel: 256 targets as the MMA's N operand */
#define SPIRA_B200_KERNEL_TC_WS 4   /* conv_tc_kernel<weight-stationary> */
#define SPIRA_B200_KERNEL_SIMT_WS 5 /* conv_ws_simt_kernel */
int spira_b200_conv_kernel_choice(int weight_stationary, int K, int c_in, int c_out, int64_t num_targets);

/* Bytes of the pre-packed weight image for spira_b200_conv_*. */
int spira_b200_packed_weight_bytes(int K, int c_in, int c_out, int pack_mode, size_t *bytes);

/* weights[K][c_in][c_out] fp16 -> tensor-core operand image: per 64-wide reduction chunk one
 * 128-byte-swizzled K-major tile of c_out rows, so that one bulk copy lands a ready MMA operand
 * in shared memory.  Done once per layer (weights are constant at inference). */
int spira_b200_pack_weights(const void *weights, int K, int c_in, int c_out, int pack_mode, void *packed,
                            void *stream);

/* Output-stationary implicit GEMM: out[t][:] = sum_c feats[map[t][c]][:] @ W[c], map is
 * LAYOUT_OS [T_al][K].  Replaces cuda_sparse_convolution_forward_os
 * (csrc/spira/torch/cuda_sparse_convolution_forward.cu:11-80, cuda/kernels/output_stat.cuh:20-644).
 * `packed` (PACK_OS image) selects the tensor-core kernel; with packed == NULL the SIMT kernel
 * reads `weights` directly.  `epilogue` may be NULL.  `status` is a device int32 the kernel sets
 * non-zero if one of its bounded internal waits expired (it never spins forever). */
int spira_b200_conv_os(const void *feats, const void *weights, const void *packed,
                       const spira_b200_epilogue *epilogue, const int32_t *map_os, int64_t num_sources,
                       int64_t num_targets, int K, int c_in, int c_out, void *out, int32_t *status, void *stream);

/* Grouped output-stationary maps (K <= 32).  No reference counterpart: the reference's output-stationary kernel
 * (cuda/kernels/output_stat.cuh) walks the map in target order, where almost every (tile of targets, offset) pair
 * has SOME neighbour although only ~30 % of the rows do, so most of the multiplied rows are zeros.
 * spira_b200_kmap_group sorts the rows of up to SPIRA_B200_MAX_MAPS [T_al][K] maps by their K-bit presence mask
 * (fullest first, stable; key for K <= 27: (K - popcount) << 19 | mask >> max(0, K - 19), else ~mask) with ONE radix
 * sort over all of them, and writes per map:
 *   grouped_map [T_al][K]   row i = map row row_of[i] (rows >= num_targets: -1)
 *   row_of      [T_al]      target (output row) of grouped row i, -1 for padding rows
 *   tile_masks  [T_al/128]  bit k = some row of the 128-row tile has a neighbour at offset k
 *   stats       [2]         number of non-empty (128-row tile, offset) and (256-row tile, offset) pairs
 * The workspace size depends on the number of rows of all maps of the call together.
 * spira_b200_conv_os_grouped computes the same result as spira_b200_conv_os on the original map, bit for bit (a
 * skipped chunk only contributes zeros), and visits only the chunks named by the tile masks.  `weights` and `packed`
 * as for spira_b200_conv_os; without a packed image (a layer outside the tensor-core kernels) only the narrow-input
 * case c_in <= 8, c_out in {16, 32, 64} is covered (one thread per row: grouped rows let the lanes of a warp skip the
 * same offsets), anything else is SPIRA_B200_ERR_ARGUMENT. */
typedef struct spira_b200_group_desc {
  const int32_t *map_os; /* [T_al][K], T_al = num_targets rounded up to 128 */
  int64_t num_targets;   /* > 0 */
  int32_t K;             /* 1..32 */
  int32_t *grouped_map;
  int32_t *row_of;
  uint32_t *tile_masks;
  int32_t *stats;
} spira_b200_group_desc;
int spira_b200_kmap_group_workspace(int64_t total_targets, size_t *bytes);
int spira_b200_kmap_group(const spira_b200_group_desc *descs, int n_maps, void *workspace, size_t workspace_bytes,
                          void *stream);
int spira_b200_conv_os_grouped(const void *feats, const void *weights, const void *packed,
                               const spira_b200_epilogue *epilogue, const int32_t *grouped_map, const int32_t *row_of,
                               const uint32_t *tile_masks, int64_t num_sources, int64_t num_targets, int K, int c_in,
                               int c_out, void *out, int32_t *status, void *stream);

/* Output-stationary convolution of a SMALL layer with the reduction of every 128-target tile shared among `splits`
 * CTAs (2, 4 or 8), so that a deep network level of a few thousand voxels occupies all SMs instead of one SM per tile.
 * No reference counterpart: the reference runs such layers through its ordinary output-stationary kernel
 * (csrc/spira/cuda/kernels/output_stat.cuh:19-189).  CTA i of a tile takes the tile's non-empty 64-wide reduction chunks
 * i, i + splits, ...; the fp32 partial sums meet in `scratch`, each CTA then adds the partials of c_out / splits columns
 * in the fixed order 0 .. splits-1 (deterministic; rounds differently from spira_b200_conv_os, whose single CTA adds all
 * chunks in TMEM), applies the epilogue and writes fp16.  The kernel is launched cooperatively and the CTAs of a tile
 * wait for one another with the bounded wait of the "wait_limit_us" option (expiry is reported through `status`; the
 * scratch must then be cleared before its next use).
 *   map_os / row_of / tile_masks   a plain [T_al][K] map (row_of = tile_masks = NULL) or a grouped one
 *   scratch   caller-owned, 16-byte aligned; its first 1024 bytes are tile counters that must be ZERO on entry and are
 *             zero again when the call completes, the rest is overwritten.  Calls that share a scratch must be ordered
 *             on one stream.
 * spira_b200_conv_os_split_plan reports the largest `splits` a layer takes (1: none -- more than 128 tiles, tiles x 2
 * beyond the SM count, c_out / splits not a multiple of 8, or fewer than 4 chunks per CTA) and the scratch bytes needed
 * at that count: 1024 + T_al * splits * c_out * 4. */
int spira_b200_conv_os_split_plan(int64_t num_targets, int K, int c_in, int c_out, int *max_splits, size_t *scratch_bytes);
int spira_b200_conv_os_split(const void *feats, const void *packed, const spira_b200_epilogue *epilogue,
                             const int32_t *map_os, const int32_t *row_of, const uint32_t *tile_masks, int64_t num_sources,
                             int64_t num_targets, int K, int c_in, int c_out, int splits, void *scratch,
                             size_t scratch_bytes, void *out, int32_t *status, void *stream);

/* One convolution from a descriptor: the tensor-core paths of spira_b200_conv_os / _os_grouped / _os_split (dataflow 0) and
 * spira_b200_conv_ws_fused (dataflow 1) behind one call, plus two forms the positional entry points do not have:
 *   two sources   the input rows are the channel concatenation of two tensors that share the map, never materialised:
 *                 channels [0, c_in_a) of source row s come from feats[s][0..c_in_a), channels [c_in_a, c_in) from
 *                 feats_b[s][0..c_in - c_in_a).  The weights stay [K][c_in][c_out].  c_in_a must be a multiple of 8.
 *                 (The reference concatenates first: spira/operators.py:11-13 -- one more read and write of both tensors.)
 *   identity map  dataflow 0 with K == 1 and map_os == NULL: target t reads source t (a 1x1x1 layer: the reference runs it
 *                 as a dense matrix product, spira/nn/conv.py:312-316).  With sources of whole 32-channel groups the
 *                 layer runs on a kernel of its own whose input tiles are TMA boxes ("identity_tma" option).
 * `packed` is the SPIRA_B200_PACK_OS image for dataflow 0 and the SPIRA_B200_PACK_WS image for dataflow 1.  A layer
 * outside the tensor-core kernels (spira_b200_tensor_core_eligible == 0) passes packed = NULL and its plain `weights`
 * instead: dataflow 0 only, one source, no identity map, and a grouped map only for the narrow-input shapes
 * spira_b200_conv_os_grouped takes without an image.  Everything else -- epilogue, status word, scratch contracts,
 * stream binding of dataflow 1 -- is as documented for the positional calls. */
typedef struct spira_b200_conv_desc {
  int32_t dataflow;            /* 0 output-stationary, 1 weight-stationary (single fused launch) */
  int32_t K, c_in, c_out;
  int32_t c_in_a;              /* channels taken from `feats`; 0 or c_in: one source */
  int32_t rows, mirror, swap;  /* dataflow 1: as for spira_b200_conv_ws */
  int32_t splits;              /* dataflow 0: CTAs per tile (0 or 1: one), as for spira_b200_conv_os_split */
  int32_t reserved;
  int64_t num_sources, num_targets;
  int64_t num_tiles128;        /* dataflow 1: qnaddrs[rows] / 128, or -1 */
  const void *feats, *feats_b;
  const void *packed;
  const void *weights;         /* fp16 [K][c_in][c_out]; read only when packed == NULL */
  const spira_b200_epilogue *epilogue;   /* may be NULL */
  const int32_t *map_os;       /* dataflow 0: [T_al][K], plain or grouped; NULL = identity (K == 1) */
  const int32_t *row_of;       /* dataflow 0, grouped map: with tile_masks, else both NULL */
  const uint32_t *tile_masks;
  const int32_t *in_idx, *out_idx, *naddrs, *qnaddrs;   /* dataflow 1 */
  float *zeroed_accum;         /* dataflow 1: the always-zero scratch of spira_b200_conv_ws_fused */
  void *split_scratch;         /* dataflow 0, splits > 1 */
  size_t split_scratch_bytes;
  void *out;                   /* fp16 [num_targets][c_out] */
} spira_b200_conv_desc;
int spira_b200_conv(const spira_b200_conv_desc *desc, int32_t *status, void *stream);

/* A whole network forward as ONE call: the operators of a recorded forward pass, executed in order on `stream`.  No
 * reference counterpart (its forward is eager PyTorch, one Python call chain per layer: spira/nn/conv.py:310-419); the
 * host cost of a scene drops from one interpreter round trip per layer to one per scene.
 *   ops     the static part: operator kinds, shapes, weight images, epilogue constants, and which SLOT (feature tensor
 *           of the forward pass) each operator reads and writes
 *   maps    the kernel maps of THIS scene, indexed by spira_b200_tape_op.map
 *   slots   per slot its row count for this scene, its channel count, and its address: slots with a non-NULL `ptr`
 *           (the network input, the outputs the caller wants to keep) are used as given, the others are placed in
 *           `arena` -- slots that share a `buffer` number share storage (the caller assigns the numbers from the
 *           lifetimes of the recorded pass); `ptr` is filled in for every slot on return
 *   arena   caller-owned device memory, 256-byte aligned; if `arena_bytes` is too small the call launches nothing,
 *           stores the size it needs in *arena_needed and returns SPIRA_B200_ERR_UNSUPPORTED
 * Operator kinds:
 *   SPIRA_B200_TAPE_CONV       spira_b200_conv on maps[op.map]: dataflow 0 uses its output-stationary form (the grouped
 *                              one if op.grouped != 0 and the map has it; transposed != 0: the inverted forms `*_t`
 *                              with sources and targets exchanged), dataflow 1 its pair lists (transposed != 0: swap)
 *   SPIRA_B200_TAPE_IDENTITY   a 1x1x1 layer through the identity map (rows of in_a)
 *   SPIRA_B200_TAPE_POINTWISE  spira_b200_pointwise (1x1x1 layer with at most 32 output channels)
 * The residual slot of an operator, if any, replaces epilogue.residual. */
#define SPIRA_B200_TAPE_CONV 0
#define SPIRA_B200_TAPE_IDENTITY 1
#define SPIRA_B200_TAPE_POINTWISE 2
typedef struct spira_b200_tape_map {
  int64_t num_sources, num_targets;
  const int32_t *map_os;       /* [T_al][K] in target order, or NULL when the scene built only the lists */
  const int32_t *grouped_map;  /* its grouped twin with row_of and tile_masks, or all three NULL */
  const int32_t *row_of;
  const uint32_t *tile_masks;
  const int32_t *map_os_t;     /* inverted map [S_al][K] for transposed layers run output-stationary, else NULL */
  const int32_t *grouped_map_t;
  const int32_t *row_of_t;
  const uint32_t *tile_masks_t;
  const int32_t *in_idx, *out_idx, *naddrs, *qnaddrs;
  int32_t rows, mirror;
  int64_t num_tiles128;
} spira_b200_tape_map;
typedef struct spira_b200_tape_op {
  int32_t kind;
  int32_t dataflow, transposed;
  int32_t map;                 /* index into maps (TAPE_CONV) */
  int32_t in_a, in_b;          /* input slots; in_b = -1: one source */
  int32_t residual;            /* slot or -1 */
  int32_t out;                 /* output slot */
  int32_t K, c_in, c_in_a, c_out;
  int32_t grouped;             /* dataflow 0: run over the grouped twin of the map where it exists */
  int32_t reserved;
  const void *packed;          /* TAPE_CONV / TAPE_IDENTITY: weight image of the operator's dataflow, or NULL */
  const void *weights;         /* TAPE_POINTWISE: fp16 [c_in][c_out]; TAPE_CONV with packed == NULL: fp16 [K][c_in][c_out] */
  spira_b200_epilogue epilogue;   /* bias / scale / shift / relu of the operator (residual is taken from the slot) */
} spira_b200_tape_op;
typedef struct spira_b200_tape_slot {
  int64_t rows;
  int32_t channels;
  int32_t buffer;              /* arena buffer number, -1 with a caller-given ptr */
  void *ptr;
} spira_b200_tape_slot;
int spira_b200_run_tape(const spira_b200_tape_op *ops, int n_ops, const spira_b200_tape_map *maps, int n_maps,
                        spira_b200_tape_slot *slots, int n_slots, void *arena, size_t arena_bytes, size_t *arena_needed,
                        float *zeroed_accum, size_t zeroed_accum_floats, int32_t *status, void *stream);

/* Weight-stationary gather-GEMM-scatter over compacted pair lists: for row k and pair p in
 * [naddrs[k], naddrs[k+1]):  accum[out_idx[p]][:] += feats[in_idx[p]][:] @ W[k].  With
 * `mirror` != 0 (submanifold map, rows == (K+1)/2) every row k is also applied with in/out swapped
 * and weight K-1-k, except the centre row (K-1)/2 of an odd K, which is its own mirror image
 * (csrc/spira/cuda/kernels/weight_stat.cuh:786-798; even K: the weight-stationary part of a hybrid map).  With
 * `swap` != 0 the roles of in_idx and out_idx are exchanged (transposed layer on the map of its
 * non-transposed twin, spira/nn/conv.py:341-348).  accum is fp32 [num_targets][c_out] scratch,
 * zeroed by the call; out is fp16 [num_targets][c_out].  `qnaddrs` holds the 128-rounded prefix
 * sums and `num_tiles128` = qnaddrs[rows] / 128 if the caller knows it, or -1: the kernels then read it from
 * `qnaddrs` on the device, so list sizes never have to travel to the host.
 * Replaces cuda_sparse_convolution_forward_ws_merged
 * (csrc/spira/torch/cuda_sparse_convolution_forward.cu:183-246). */
int spira_b200_conv_ws(const void *feats, const void *weights, const void *packed,
                       const spira_b200_epilogue *epilogue, const int32_t *in_idx, const int32_t *out_idx,
                       const int32_t *naddrs, const int32_t *qnaddrs, int rows, int64_t num_tiles128, int mirror,
                       int swap, int64_t num_sources, int64_t num_targets, int K, int c_in, int c_out, float *accum,
                       void *out, int32_t *status, void *stream);

/* spira_b200_conv_ws with the zero-fill and the final conversion inside the convolution kernel (one launch instead of
 * three; tensor-core eligible layers only, `packed` required).  No reference counterpart.  The grid has at most one
 * CTA per SM (see the "ws_cooperative_launch" option for how it is launched): after their last tile the CTAs meet at a
 * grid barrier (bounded wait, reported through `status`), then
 * every CTA converts its slice of the scratch to fp16 with the epilogue applied and writes zeros back.  Contract:
 *   zeroed_accum[0 .. num_targets * c_out) holds zeros on entry and holds zeros again when the call has completed;
 *   calls on one device must be ordered on one stream (they share the arrival counter of the grid barrier): the first
 *   call binds the device to its stream, a call on another stream returns SPIRA_B200_ERR_ARGUMENT until
 *   spira_b200_ws_barrier_resync() releases the binding. */
int spira_b200_conv_ws_fused(const void *feats, const void *packed, const spira_b200_epilogue *epilogue,
                             const int32_t *in_idx, const int32_t *out_idx, const int32_t *naddrs, const int32_t *qnaddrs,
                             int rows, int64_t num_tiles128, int mirror, int swap, int64_t num_sources, int64_t num_targets,
                             int K, int c_in, int c_out, float *zeroed_accum, void *out, int32_t *status, void *stream);

/* Capacity, in floats, of the scratch array built into the library for spira_b200_conv_ws_static (16 MiB per GPU). */
#define SPIRA_B200_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)

/* Same computation and arguments as spira_b200_conv_ws, minus `accum`: the fp32 accumulation scratch is a fixed
 * device array inside the library, so the call needs no memory beyond its inputs and outputs and performs no
 * allocation of any kind.  It has no counterpart in the reference.  It is meant for hosts that must not allocate on
 * the request path: an inference server that carves up device memory once at start-up and treats any later
 * allocation as a fault, or a plain C / C++ embedder that has no caching allocator to borrow scratch from.
 *   - limit: num_targets * c_out <= SPIRA_B200_STATIC_SCRATCH_FLOATS, otherwise the call fails with
 *     SPIRA_B200_ERR_ARGUMENT and a message naming the limit (use spira_b200_conv_ws then);
 *   - the first call on a device looks up the array's device address; make that call before capturing a stream;
 *   - all calls on a GPU share the one array (it is cleared at the start of every call and keeps the last call's
 *     partial sums afterwards), so two calls that overlap on the GPU -- different streams, or different host threads
 *     -- race with each other: serialise them. */
int spira_b200_conv_ws_static(const void *feats, const void *weights, const void *packed,
                              const spira_b200_epilogue *epilogue, const int32_t *in_idx, const int32_t *out_idx,
                              const int32_t *naddrs, const int32_t *qnaddrs, int rows, int64_t num_tiles128, int mirror,
                              int swap, int64_t num_sources, int64_t num_targets, int K, int c_in, int c_out, void *out,
                              int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SPIRA_B200_H_ */

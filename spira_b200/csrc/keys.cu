// Packed voxel keys: pack / unpack, feature permutation, strided down-sampling of UNSORTED keys.
//
// The sort of a scene's keys and the down-sampling of sorted keys (the path every scene takes) are hand-written
// cooperative kernels in ingest.cu; the general down-sampling here (unsorted input, arbitrary power-of-two strides)
// uses CUB's radix sort and run-length "unique" (library-class ops).
#include <cub/cub.cuh>

#include "common.cuh"

namespace sb {

template <typename KeyT>
__global__ void __launch_bounds__(256) pack_kernel(const int32_t *__restrict__ coords, int64_t n,
                                                    KeyT *__restrict__ keys, int32_t *__restrict__ iota) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  // 12 bytes per voxel: three 4-byte loads, coalesced across the warp through L1.
  KeyT x = static_cast<KeyT>(coords[3 * i + 0]);
  KeyT y = static_cast<KeyT>(coords[3 * i + 1]);
  KeyT z = static_cast<KeyT>(coords[3 * i + 2]);
  keys[i] = (x << KeyShift<KeyT>::X) | (y << KeyShift<KeyT>::Y) | z;
  if (iota != nullptr) iota[i] = static_cast<int32_t>(i);
}

template <typename KeyT>
__global__ void __launch_bounds__(256) unpack_kernel(const KeyT *__restrict__ keys, int64_t n,
                                                      int32_t *__restrict__ coords) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  using L = KeyLayout<KeyT>;
  KeyT k = keys[i];
  coords[3 * i + 0] = static_cast<int32_t>((k >> KeyShift<KeyT>::X) & ((KeyT(1) << L::XB) - 1));
  coords[3 * i + 1] = static_cast<int32_t>((k >> KeyShift<KeyT>::Y) & ((KeyT(1) << L::YB) - 1));
  coords[3 * i + 2] = static_cast<int32_t>(k & ((KeyT(1) << L::ZB) - 1));
}

// rows_out[i] = rows_in[perm[i]], 16-byte vectors when the row size allows, else 2-byte units.
template <typename VecT>
__global__ void __launch_bounds__(256) permute_rows_kernel(const VecT *__restrict__ in, const int32_t *__restrict__ perm,
                                                            int64_t n, int vecs_per_row, VecT *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  int64_t row = g / vecs_per_row;
  int v = static_cast<int>(g - row * vecs_per_row);
  if (row >= n) return;
  out[row * vecs_per_row + v] = in[int64_t(perm[row]) * vecs_per_row + v];
}

template <typename KeyT, int L>
struct MaskPack {
  KeyT mask[L];
  KeyT *out[L];
};

// One pass over the level-0 keys writes the masked keys of every level.
template <typename KeyT>
__global__ void __launch_bounds__(256) mask_levels_kernel(const KeyT *__restrict__ keys, int64_t n, int n_levels,
                                                           MaskPack<KeyT, SPIRA_B200_MAX_LEVELS> p) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  KeyT k = keys[i];
#pragma unroll
  for (int l = 0; l < SPIRA_B200_MAX_LEVELS; ++l)
    if (l < n_levels) p.out[l][i] = k & p.mask[l];
}

template <typename KeyT>
size_t sort_keys_temp(int64_t n) {
  size_t a = 0, b = 0;
  cub::DoubleBuffer<KeyT> dk(nullptr, nullptr);
  cub::DeviceRadixSort::SortKeys(nullptr, a, dk, static_cast<int>(n), 0, int(sizeof(KeyT) * 8));
  cub::DeviceSelect::Unique(nullptr, b, (const KeyT *)nullptr, (KeyT *)nullptr, (int32_t *)nullptr,
                            static_cast<int>(n));
  return a > b ? a : b;
}

inline size_t round256(size_t b) { return (b + 255) / 256 * 256; }

template <typename KeyT>
KeyT stride_mask(const int32_t *s) {
  using L = KeyLayout<KeyT>;
  KeyT xm = ((KeyT(1) << L::XB) - 1) & ~static_cast<KeyT>(s[0] - 1);
  KeyT ym = ((KeyT(1) << L::YB) - 1) & ~static_cast<KeyT>(s[1] - 1);
  KeyT zm = ((KeyT(1) << L::ZB) - 1) & ~static_cast<KeyT>(s[2] - 1);
  return (xm << KeyShift<KeyT>::X) | (ym << KeyShift<KeyT>::Y) | zm;
}

template <typename KeyT>
int downsample_impl(const KeyT *keys, int64_t n, int n_levels, const int32_t *strides, void *const *out_keys,
                    int32_t *counts, void *ws, size_t ws_bytes, cudaStream_t stream) {
  // workspace: per level [masked n][alt n], then one shared cub temp
  size_t temp = sort_keys_temp<KeyT>(n);
  size_t per_level = 2 * round256(n * sizeof(KeyT));
  size_t need = per_level * n_levels + temp;
  if (ws_bytes < need) return fail(SPIRA_B200_ERR_WORKSPACE, "downsample: workspace %zu < %zu bytes", ws_bytes, need);
  if (n == 0) {
    SB_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * n_levels, stream));
    return SPIRA_B200_OK;
  }
  char *base = static_cast<char *>(ws);
  MaskPack<KeyT, SPIRA_B200_MAX_LEVELS> mp;
  for (int l = 0; l < SPIRA_B200_MAX_LEVELS; ++l) {
    mp.mask[l] = 0;
    mp.out[l] = nullptr;
  }
  for (int l = 0; l < n_levels; ++l) {
    mp.mask[l] = stride_mask<KeyT>(strides + 3 * l);
    mp.out[l] = reinterpret_cast<KeyT *>(base + per_level * l);
  }
  void *temp_ptr = base + per_level * n_levels;
  mask_levels_kernel<KeyT><<<static_cast<int>(div_up(n, 256)), 256, 0, stream>>>(keys, n, n_levels, mp);
  SB_CHECK_LAUNCH();
  for (int l = 0; l < n_levels; ++l) {
    KeyT *a = mp.out[l];
    KeyT *b = reinterpret_cast<KeyT *>(base + per_level * l + round256(n * sizeof(KeyT)));
    cub::DoubleBuffer<KeyT> dk(a, b);
    size_t t = temp;
    SB_CHECK_CUDA(cub::DeviceRadixSort::SortKeys(temp_ptr, t, dk, static_cast<int>(n), 0, int(sizeof(KeyT) * 8), stream));
    t = temp;
    SB_CHECK_CUDA(cub::DeviceSelect::Unique(temp_ptr, t, dk.Current(), static_cast<KeyT *>(out_keys[l]), counts + l,
                                            static_cast<int>(n), stream));
  }
  return SPIRA_B200_OK;
}

// strides[l] must be, per axis, equal to or twice strides[l-1] (strides[-1] = 1)
inline bool strides_double(int n_levels, const int32_t *strides) {
  int prev[3] = {1, 1, 1};
  for (int l = 0; l < n_levels; ++l)
    for (int a = 0; a < 3; ++a) {
      const int s = strides[3 * l + a];
      if (s != prev[a] && s != 2 * prev[a]) return false;
      prev[a] = s;
    }
  return true;
}

// scene ingest in cooperative launches (ingest.cu)
size_t ingest_sort_workspace(int64_t n, int key_bytes);
int ingest_sort(const int32_t *coords, int64_t n, int key_bytes, void *sorted_keys, int32_t *perm, void *ws, size_t ws_bytes,
                int32_t *status, cudaStream_t stream);
size_t ingest_coarsen_workspace(int64_t n, int key_bytes);
int ingest_coarsen(const void *keys, int64_t n, int key_bytes, int n_levels, const int32_t *strides, void *const *out_keys,
                   int32_t *counts, void *ws, size_t ws_bytes, int32_t *status, cudaStream_t stream);

}  // namespace sb

using namespace sb;

#define SB_KEY_DISPATCH(key_bytes, ...)                                                     \
  if ((key_bytes) == 4) {                                                                   \
    using KeyT = uint32_t;                                                                  \
    __VA_ARGS__                                                                             \
  } else if ((key_bytes) == 8) {                                                            \
    using KeyT = uint64_t;                                                                  \
    __VA_ARGS__                                                                             \
  } else {                                                                                  \
    return fail(SPIRA_B200_ERR_ARGUMENT, "key_bytes must be 4 or 8, got %d", (key_bytes));  \
  }

extern "C" int spira_b200_pack(const int32_t *coords, int64_t n, int key_bytes, void *keys, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "pack: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n == 0 || (coords && keys), "pack: null pointer");
  if (n == 0) return SPIRA_B200_OK;
  SB_KEY_DISPATCH(key_bytes, {
    pack_kernel<KeyT><<<static_cast<int>(div_up(n, 256)), 256, 0, as_stream(stream)>>>(
        coords, n, static_cast<KeyT *>(keys), nullptr);
  })
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_unpack(const void *keys, int64_t n, int key_bytes, int32_t *coords, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "unpack: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n == 0 || (coords && keys), "unpack: null pointer");
  if (n == 0) return SPIRA_B200_OK;
  SB_KEY_DISPATCH(key_bytes, {
    unpack_kernel<KeyT><<<static_cast<int>(div_up(n, 256)), 256, 0, as_stream(stream)>>>(
        static_cast<const KeyT *>(keys), n, coords);
  })
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_flatten_sort_workspace(int64_t n, int key_bytes, size_t *bytes) {
  SB_CHECK_ARG(bytes != nullptr, "flatten_sort_workspace: null output");
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "flatten_sort: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(key_bytes == 4 || key_bytes == 8, "key_bytes must be 4 or 8, got %d", key_bytes);
  *bytes = ingest_sort_workspace(n, key_bytes);
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_flatten_sort(const int32_t *coords, int64_t n, int key_bytes, void *sorted_keys,
                                       int32_t *perm, void *workspace, size_t workspace_bytes, int32_t *status, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "flatten_sort: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n == 0 || (coords && sorted_keys && perm && workspace), "flatten_sort: null pointer");
  SB_CHECK_ARG(key_bytes == 4 || key_bytes == 8, "key_bytes must be 4 or 8, got %d", key_bytes);
  return ingest_sort(coords, n, key_bytes, sorted_keys, perm, workspace, workspace_bytes, status, as_stream(stream));
}

extern "C" int spira_b200_permute_rows(const void *rows_in, const int32_t *perm, int64_t n, int64_t row_bytes,
                                       void *rows_out, void *stream) {
  SB_CHECK_ARG(n >= 0 && row_bytes > 0 && row_bytes % 2 == 0, "permute_rows: bad sizes n=%lld row_bytes=%lld",
               (long long)n, (long long)row_bytes);
  if (n == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(rows_in && perm && rows_out, "permute_rows: null pointer");
  bool vec16 = row_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(rows_in) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(rows_out) % 16 == 0);
  if (vec16) {
    int vpr = static_cast<int>(row_bytes / 16);
    SB_CHECK_CUDA(launch_dependent(permute_rows_kernel<uint4>, dim3(static_cast<unsigned>(div_up(n * vpr, 256))), dim3(256), 0,
                                   as_stream(stream), static_cast<const uint4 *>(rows_in), perm, n, vpr, static_cast<uint4 *>(rows_out)));
  } else {
    int vpr = static_cast<int>(row_bytes / 2);
    SB_CHECK_CUDA(launch_dependent(permute_rows_kernel<uint16_t>, dim3(static_cast<unsigned>(div_up(n * vpr, 256))), dim3(256), 0,
                                   as_stream(stream), static_cast<const uint16_t *>(rows_in), perm, n, vpr,
                                   static_cast<uint16_t *>(rows_out)));
  }
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_downsample_workspace(int64_t n, int key_bytes, int n_levels, size_t *bytes) {
  SB_CHECK_ARG(bytes != nullptr, "downsample_workspace: null output");
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "downsample: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n_levels >= 1 && n_levels <= SPIRA_B200_MAX_LEVELS, "downsample: n_levels=%d not in [1,%d]", n_levels,
               SPIRA_B200_MAX_LEVELS);
  SB_KEY_DISPATCH(key_bytes, { *bytes = 2 * round256(n * sizeof(KeyT)) * n_levels + sort_keys_temp<KeyT>(n) + 256; })
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_downsample(const void *keys, int64_t n, int key_bytes, int n_levels,
                                     const int32_t *host_strides, void *const *host_out_keys, int32_t *counts,
                                     void *workspace, size_t workspace_bytes, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "downsample: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n_levels >= 1 && n_levels <= SPIRA_B200_MAX_LEVELS, "downsample: n_levels=%d not in [1,%d]", n_levels,
               SPIRA_B200_MAX_LEVELS);
  SB_CHECK_ARG(host_strides && host_out_keys && counts, "downsample: null pointer");
  for (int l = 0; l < n_levels; ++l) {
    for (int a = 0; a < 3; ++a) {
      int s = host_strides[3 * l + a];
      SB_CHECK_ARG(s >= 1 && (s & (s - 1)) == 0, "downsample: stride %d of level %d is not a power of two", s, l);
    }
    SB_CHECK_ARG(n == 0 || host_out_keys[l] != nullptr, "downsample: null output for level %d", l);
  }
  SB_CHECK_ARG(n == 0 || (keys && workspace), "downsample: null pointer");
  SB_KEY_DISPATCH(key_bytes, {
    return downsample_impl<KeyT>(static_cast<const KeyT *>(keys), n, n_levels, host_strides, host_out_keys, counts,
                                 workspace, workspace_bytes, as_stream(stream));
  })
}

extern "C" int spira_b200_downsample_sorted_workspace(int64_t n, int key_bytes, size_t *bytes) {
  SB_CHECK_ARG(bytes != nullptr, "downsample_sorted_workspace: null output");
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "downsample_sorted: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(key_bytes == 4 || key_bytes == 8, "key_bytes must be 4 or 8, got %d", key_bytes);
  *bytes = ingest_coarsen_workspace(n, key_bytes);
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_downsample_sorted(const void *sorted_keys, int64_t n, int key_bytes, int n_levels,
                                            const int32_t *host_strides, void *const *host_out_keys, int32_t *counts,
                                            void *workspace, size_t workspace_bytes, int32_t *status, void *stream) {
  SB_CHECK_ARG(n >= 0 && n < (int64_t(1) << 31), "downsample_sorted: n=%lld out of range", (long long)n);
  SB_CHECK_ARG(n_levels >= 1 && n_levels <= SPIRA_B200_MAX_LEVELS, "downsample_sorted: n_levels=%d not in [1,%d]", n_levels,
               SPIRA_B200_MAX_LEVELS);
  SB_CHECK_ARG(host_strides && host_out_keys && counts, "downsample_sorted: null pointer");
  for (int l = 0; l < n_levels; ++l) {
    for (int a = 0; a < 3; ++a) {
      int s = host_strides[3 * l + a];
      SB_CHECK_ARG(s >= 1 && (s & (s - 1)) == 0, "downsample_sorted: stride %d of level %d is not a power of two", s, l);
    }
    SB_CHECK_ARG(n == 0 || host_out_keys[l] != nullptr, "downsample_sorted: null output for level %d", l);
  }
  if (!strides_double(n_levels, host_strides))
    return fail(SPIRA_B200_ERR_UNSUPPORTED, "downsample_sorted: every stride must equal or double the stride of the level before");
  SB_CHECK_ARG(n == 0 || (sorted_keys && workspace), "downsample_sorted: null pointer");
  SB_CHECK_ARG(key_bytes == 4 || key_bytes == 8, "key_bytes must be 4 or 8, got %d", key_bytes);
  return ingest_coarsen(sorted_keys, n, key_bytes, n_levels, host_strides, host_out_keys, counts, workspace, workspace_bytes,
                        status, as_stream(stream));
}

// 1x1x1 layers on the tensor cores without a map: out[n][c_out] = epilogue([feats_a | feats_b][n][c_in] . W[c_in][c_out]).
//
// The reference sends every 1x1x1 layer to torch.mm and runs BatchNorm, the residual add and ReLU as separate passes
// (spira/nn/conv.py:312-316).  A 1x1x1 layer gathers nothing: row t of the output reads row t of the input, so the input
// tile of 128 rows is a dense box of the feature tensor and TMA moves it (no producer threads, no index arithmetic, no
// L1 traffic).  The layer reads n*c_in*2 bytes and writes n*c_out*2: it is bound by HBM.
//
// One persistent CTA per SM, 12 warps:
//   warp 0      one thread issues, per 64 channels of the reduction, two TMA boxes of 32 channels x 128 rows (64-byte
//               swizzle; a box never straddles the two source tensors: their channel counts are multiples of 32) and the
//               matching 64-channel chunk of the packed weight image (one bulk copy; or all chunks once, when the image
//               is small and the CTA has several tiles);
//   warp 1      one thread issues the tcgen05 MMAs (M = 128 rows, N = c_out, fp32 accumulator in tensor memory, two
//               accumulator buffers);
//   warps 4-11  epilogue, two warps per tensor-memory lane quarter, half of the columns each: tcgen05.ld, bias /
//               BatchNorm / residual / ReLU on fp32, one rounding, 32-byte stores.
// Every wait is bounded; an expired wait raises the status word and the CTA drains.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace sb {

using namespace sb::ptx;

constexpr int kDRows = 128;                 // rows per tile (MMA M)
constexpr int kDBox = 32;                   // channels per TMA box (64 bytes: one row of the 64-byte swizzle)
constexpr int kDBoxBytes = kDRows * 64;     // 8 KB
constexpr int kDStageA = 2 * kDBoxBytes;    // a stage holds 64 channels of the reduction
constexpr int kDMaxStages = 8;
constexpr int kDEpilogueWarps = 8;
constexpr int kDFirstEpilogueWarp = 4;      // (a warp reads the tensor-memory lane quarter warp % 4)
constexpr int kDThreads = (kDFirstEpilogueWarp + kDEpilogueWarps) * 32;
constexpr int kDSmemBudget = 220 * 1024;
constexpr int kDResidentLimit = 64 * 1024;  // weight images up to this size stay in shared memory

struct DenseParams {
  const unsigned char *packed;   // [ceil(c_in / 64)][c_out][128 bytes], 128-byte swizzle (the K = 1 image of spira_b200_pack_weights)
  __half *out;
  const __half *bias;
  const float *scale, *shift;
  const __half *residual;
  int relu;
  int32_t *status;
  int n, n_tiles, c_in, c_a, c_out, n_chunks;
  int stages, resident, b_bytes, acc_stride, tmem_cols;
  int off_b, off_ep, off_bar;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
               : "memory");
}

// K-major operand tile stored with the 64-byte swizzle: rows of 64 bytes (32 fp16 along K), 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;                            // layout: SWIZZLE_64B
  return d;
}

__global__ void __launch_bounds__(kDThreads, 1) dense_tc_kernel(const __grid_constant__ DenseParams P,
                                                                 const __grid_constant__ CUtensorMap tmap_a,
                                                                 const __grid_constant__ CUtensorMap tmap_b) {
  extern __shared__ unsigned char dense_smem_raw[];
  const uint32_t raw = smem_u32(dense_smem_raw);
  unsigned char *smem = dense_smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + P.off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kDMaxStages + s); };
  auto bar_acc_full = [&](int b) { return bar0 + 8u * (2 * kDMaxStages + b); };
  auto bar_acc_empty = [&](int b) { return bar0 + 8u * (2 * kDMaxStages + 2 + b); };
  const uint32_t bar_weights = bar0 + 8u * (2 * kDMaxStages + 4);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + P.off_bar + 8 * (2 * kDMaxStages + 5));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + P.off_bar + 8 * (2 * kDMaxStages + 5) + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stages = P.stages;
  pdl_trigger();
  // ---- set-up that touches no global memory
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 32 * kDEpilogueWarps);
    }
    mbar_init(bar_weights, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), P.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();      // barriers and the tensor-memory address are visible; nothing has touched global memory yet
  tc_fence_after();
  pdl_wait();           // before the first global read of any thread (features, weights, epilogue constants)
  // The epilogue applies (acc + bias[c]) * scale[c] + shift[c] with one thread per ROW: the constants of every channel are
  // staged as fp32 by the epilogue warps themselves (barrier 1), off the path of the first copies and MMAs.
  float4 *s_ep = reinterpret_cast<float4 *>(smem + P.off_ep);      // {bias, scale, shift, -} per channel
  const bool has_affine = P.bias != nullptr || P.scale != nullptr;
  const uint32_t tmem_base = *tmem_slot;
  const int n_tiles = P.n_tiles, G = gridDim.x;

  if (warp == 0) {
    // =========================== producer ===========================
    if (lane == 0) {
      if (P.resident && static_cast<int>(blockIdx.x) < n_tiles) {
        mbar_arrive_expect_tx(bar_weights, static_cast<uint32_t>(P.n_chunks) * P.b_bytes);
        for (int j = 0; j < P.n_chunks; ++j)
          bulk_g2s(sbase + P.off_b + j * P.b_bytes, P.packed + static_cast<int64_t>(j) * P.b_bytes, P.b_bytes, bar_weights);
      }
      int stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += G) {
        const int y = tile * kDRows;
        for (int j = 0; j < P.n_chunks; ++j) {
          if (!mbar_wait(bar_empty(stage), phase ^ 1, abort_flag, P.wait_ns)) { ok = false; break; }
          const int ch0 = j * 64;
          const int boxes = P.c_in - ch0 >= 64 ? 2 : 1;
          mbar_arrive_expect_tx(bar_full(stage), boxes * kDBoxBytes + (P.resident ? 0 : P.b_bytes));
          for (int h = 0; h < boxes; ++h) {
            const int ch = ch0 + h * kDBox;
            const uint32_t dst = sbase + stage * kDStageA + h * kDBoxBytes;
            if (ch < P.c_a) tma_load_2d(dst, &tmap_a, ch, y, bar_full(stage));
            else tma_load_2d(dst, &tmap_b, ch - P.c_a, y, bar_full(stage));
          }
          if (!P.resident)
            bulk_g2s(sbase + P.off_b + stage * P.b_bytes, P.packed + static_cast<int64_t>(j) * P.b_bytes, P.b_bytes, bar_full(stage));
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = idesc_f16_m128(P.c_out);
      int stage = 0, phase = 0, tile_i = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      if (P.resident && static_cast<int>(blockIdx.x) < n_tiles) ok = mbar_wait(bar_weights, 0, abort_flag, P.wait_ns);
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += G, ++tile_i) {
        const int b = tile_i & 1;
        if (!mbar_wait(bar_acc_empty(b), ((acc_phase >> b) & 1u) ^ 1u, abort_flag, P.wait_ns)) break;
        acc_phase ^= 1u << b;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * P.acc_stride;
        for (int j = 0; j < P.n_chunks; ++j) {
          if (!mbar_wait(bar_full(stage), phase, abort_flag, P.wait_ns)) { ok = false; break; }
          tc_fence_after();
          const int boxes = P.c_in - j * 64 >= 64 ? 2 : 1;
          // the weight chunk keeps the 128-byte swizzle of the packed image: the k-th 16-channel step starts 32 k bytes into its rows
          const uint64_t b_desc = smem_desc_k_sw128(sbase + P.off_b + (P.resident ? j : stage) * P.b_bytes);
          for (int h = 0; h < boxes; ++h) {
            const uint64_t a_desc = smem_desc_k_sw64(sbase + stage * kDStageA + h * kDBoxBytes);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              mma_f16_ss(d_tmem, a_desc + 2 * ks, b_desc + 4 * h + 2 * ks, idesc, (j == 0 && h == 0 && ks == 0) ? 0u : 1u);
          }
          mma_commit(bar_empty(stage));
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(bar_acc_full(b));
      }
    }
    __syncwarp();
  } else if (warp >= kDFirstEpilogueWarp) {
    // =========================== epilogue ===========================
    const int q = warp & 3;
    const int half = (warp - kDFirstEpilogueWarp) >> 2;
    const int row = q * 32 + lane;
    const bool out_v8 = (reinterpret_cast<uintptr_t>(P.out) & 31) == 0;
    const bool res = P.residual != nullptr;
    if (has_affine) {
      for (int c = tid - kDFirstEpilogueWarp * 32; c < P.c_out; c += kDEpilogueWarps * 32)
        s_ep[c] = make_float4(P.bias ? __half2float(P.bias[c]) : 0.f, P.scale ? P.scale[c] : 1.f, P.scale ? P.shift[c] : 0.f, 0.f);
      named_bar_sync(1, kDEpilogueWarps * 32);
    }
    // the two warps of a lane quarter take one half of the columns each (in steps of 16: 96 channels are 48 + 48)
    const int c_split = ((P.c_out >> 1) + 15) & ~15;
    const int c_begin = half ? c_split : 0, c_end = half ? P.c_out : c_split;
    uint32_t acc_phase = 0;
    int tile_i = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += G, ++tile_i) {
      const int b = tile_i & 1;
      const int64_t t = static_cast<int64_t>(tile) * kDRows + row;
      const int64_t out_row = t < P.n ? t : -1;
      uint4 res_next[4];      // residual of the next 32 columns: on its way before the accumulator is awaited
      auto fetch_residual = [&](int c0) {
        if (out_row >= 0 && res && c0 < c_end) {
          const __half *src = P.residual + out_row * P.c_out + c0;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (c0 + 8 * i < c_end) res_next[i] = *reinterpret_cast<const uint4 *>(src + 8 * i);
        }
      };
      fetch_residual(c_begin);
      if (!mbar_wait(bar_acc_full(b), (acc_phase >> b) & 1u, abort_flag, P.wait_ns)) break;
      acc_phase ^= 1u << b;
      tc_fence_after();
      const uint32_t taddr = tmem_base + b * P.acc_stride + (static_cast<uint32_t>(q * 32) << 16);
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t r[32];
        const bool full = c0 + 32 <= c_end;
        if (full) {
          tmem_ld_32x32(taddr + c0, r);
        } else {
          uint32_t h[16];
          tmem_ld_32x16(taddr + c0, h);
#pragma unroll
          for (int i = 0; i < 16; ++i) { r[i] = h[i]; r[16 + i] = 0; }
        }
        tmem_ld_wait();
        const int width = full ? 32 : 16;
        if (out_row >= 0) {
          __half *dst = P.out + out_row * P.c_out + c0;
#pragma unroll
          for (int i = 0; i < 32; i += 16) {
            if (i < width) {
              uint4 pack[2];
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                uint32_t *pw = reinterpret_cast<uint32_t *>(&pack[hh]);
                const uint4 rv = res_next[(i >> 3) + hh];
                const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int cc = c0 + i + 8 * hh + 2 * e;
                  float v0 = __uint_as_float(r[i + 8 * hh + 2 * e]), v1 = __uint_as_float(r[i + 8 * hh + 2 * e + 1]);
                  if (has_affine) {
                    const float4 k0 = s_ep[cc], k1 = s_ep[cc + 1];
                    v0 = (v0 + k0.x) * k0.y + k0.z;
                    v1 = (v1 + k1.x) * k1.y + k1.z;
                  }
                  if (res) { v0 += __low2float(rh[e]); v1 += __high2float(rh[e]); }
                  if (P.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
                  __half2 hv = __floats2half2_rn(v0, v1);
                  pw[e] = *reinterpret_cast<uint32_t *>(&hv);
                }
              }
              if (out_v8) {
                st_global_v8(dst + i, pack[0], pack[1]);
              } else {
                *reinterpret_cast<uint4 *>(dst + i) = pack[0];
                *reinterpret_cast<uint4 *>(dst + i + 8) = pack[1];
              }
            }
          }
          fetch_residual(c0 + 32);
        }
      }
      tc_fence_before();
      mbar_arrive(bar_acc_empty(b));
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // a bounded wait expired: report, give copies in flight time to land, then release the tensor memory
    if (tid == 0 && P.status) atomicExch(P.status, 1);
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, P.tmem_cols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D map over rows[n][channels] (fp16): boxes of 32 channels x 128 rows, 64-byte swizzle, zero fill past the last row.
static int make_rows_tensor_map(CUtensorMap *map, const void *rows, int64_t n, int channels) {
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(channels), static_cast<cuuint64_t>(n)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(channels) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kDBox), static_cast<cuuint32_t>(kDRows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(rows), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SPIRA_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return SPIRA_B200_OK;
}

static int round16(int n) { return (n + 15) & ~15; }

// Shared-memory plan: [stages x 16 KB of rows][weight chunks: one per stage, or the whole image][epilogue constants][barriers].
static size_t plan_dense(DenseParams &P, bool resident) {
  P.b_bytes = P.c_out * 128;
  const int fixed = round16(P.c_out * 16) + 8 * (2 * kDMaxStages + 6) + 16 + (resident ? P.n_chunks * P.b_bytes : 0);
  const int per_stage = kDStageA + (resident ? 0 : P.b_bytes);
  int stages = (kDSmemBudget - fixed) / per_stage;
  if (stages > kDMaxStages) stages = kDMaxStages;
  if (stages < 2) return 0;
  P.stages = stages;
  P.resident = resident ? 1 : 0;
  P.off_b = stages * kDStageA;
  P.off_ep = P.off_b + (resident ? P.n_chunks : stages) * P.b_bytes;
  P.off_bar = P.off_ep + round16(P.c_out * 16);
  return static_cast<size_t>(P.off_bar) + 8 * (2 * kDMaxStages + 6) + 16 + 1024;
}

bool dense_applies(int64_t n, int c_in, int c_a, int c_out, const void *feats, const void *feats_b, const void *packed) {
  if (n <= 0 || n >= (int64_t(1) << 31) - 128) return false;
  if (c_in < 32 || c_in % kDBox != 0 || c_a % kDBox != 0 || c_a < 0 || c_a > c_in || c_out < 16 || c_out > 256 || c_out % 16 != 0) return false;
  if (reinterpret_cast<uintptr_t>(feats) % 16 != 0 || reinterpret_cast<uintptr_t>(packed) % 16 != 0) return false;
  if (c_a < c_in && (feats_b == nullptr || reinterpret_cast<uintptr_t>(feats_b) % 16 != 0)) return false;
  return encode_tiled_fn() != nullptr;
}

int dense_run(const void *feats, const void *feats_b, int c_a, const void *packed, const spira_b200_epilogue *epilogue, int64_t n,
              int c_in, int c_out, void *out, int32_t *status, unsigned long long wait_ns, cudaStream_t st) {
  DenseParams P{};
  P.packed = static_cast<const unsigned char *>(packed);
  P.out = static_cast<__half *>(out);
  if (epilogue) {
    P.bias = static_cast<const __half *>(epilogue->bias);
    P.scale = epilogue->scale;
    P.shift = epilogue->shift;
    P.residual = static_cast<const __half *>(epilogue->residual);
    P.relu = epilogue->relu;
  }
  P.status = status;
  P.n = static_cast<int>(n);
  P.n_tiles = static_cast<int>(div_up(n, kDRows));
  P.c_in = c_in; P.c_a = c_a; P.c_out = c_out;
  P.n_chunks = static_cast<int>(div_up(c_in, 64));
  P.acc_stride = 32;
  while (P.acc_stride < c_out) P.acc_stride *= 2;
  P.tmem_cols = 2 * P.acc_stride;
  P.wait_ns = wait_ns;
  const int grid = P.n_tiles < sm_count() ? P.n_tiles : sm_count();
  size_t smem = 0;
  if (P.n_tiles > grid && P.n_chunks * c_out * 128 <= kDResidentLimit) smem = plan_dense(P, true);
  if (smem == 0) smem = plan_dense(P, false);
  if (smem == 0) return fail(SPIRA_B200_ERR_UNSUPPORTED, "dense layer: c_out=%d does not fit the shared-memory plan", c_out);
  alignas(64) CUtensorMap map_a, map_b;
  int rc = make_rows_tensor_map(&map_a, feats, n, c_a);
  if (rc != SPIRA_B200_OK) return rc;
  if (c_a < c_in) {
    rc = make_rows_tensor_map(&map_b, feats_b, n, c_in - c_a);
    if (rc != SPIRA_B200_OK) return rc;
  } else {
    std::memcpy(&map_b, &map_a, sizeof(map_a));
  }
  SB_CHECK_CUDA(cudaFuncSetAttribute(dense_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  SB_CHECK_CUDA(launch_dependent(dense_tc_kernel, dim3(static_cast<unsigned>(grid)), dim3(kDThreads), smem, st, P, map_a, map_b));
  return SPIRA_B200_OK;
}

}  // namespace sb

// Sparse-convolution feature compute: fp16 in/out, fp32 accumulate.
//
// Two dataflows share one persistent, warp-specialised tcgen05 kernel (conv_tc_kernel):
//
//   output-stationary (OS): a tile is 128 consecutive targets.  The reduction runs over all
//     (offset, channel) pairs in 64-wide chunks; chunks whose offsets have no neighbour in the tile
//     are skipped.  The accumulator lives in tensor memory for the whole tile and is stored once,
//     so there are no atomics and the result is deterministic.
//   weight-stationary (WS): a tile is 128 compacted (in, out) pairs of ONE offset, so every MMA
//     row is a real pair.  The 128 x c_out product is added into an fp32 scratch with vector
//     reductions; the same launch (after a grid barrier) or a second small kernel applies the epilogue and rounds to fp16.
//
// Roles inside a CTA (800 threads, one CTA per SM):
//   warps 0-15 producers: gather feature rows with 16-byte cp.async (zero-fill for missing rows)
//              into a 128-byte-swizzled K-major A tile and let the copies arrive on the stage's
//              mbarrier asynchronously (no thread waits for its own data); one thread bulk-copies
//              the matching pre-packed weight chunk (already an MMA-ready image) and posts its bytes;
//   warp  24   one elected thread issues tcgen05.mma (M=128, N=c_out, K=16) into one of two
//              TMEM accumulator buffers and commits stage / accumulator barriers;
//   warps 16-23 epilogue, two per TMEM lane quarter: tcgen05.ld the finished accumulator (one row per thread,
//              alternate 32-column blocks), apply the fused epilogue, store fp16 rows (OS) or issue fp32 vector
//              reductions (WS) while the next tile is already being multiplied.
// All mbarrier waits are bounded; on expiry the kernel raises a status word and drains.
//
// Channel counts the tensor-core path cannot tile (c_in % 8 != 0, c_out % 16 != 0, c_out > 256)
// run on simple SIMT kernels (conv_os_simt_kernel / conv_ws_simt_kernel) -- those layers
// (3-5 input channels) are bandwidth-bound and tiny.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "ptx.cuh"

namespace sb {

using namespace sb::ptx;

constexpr int kRows = 128;              // MMA M / rows per tile
constexpr int kChunk = 64;              // fp16 elements of the reduction per pipeline stage (128 bytes)
constexpr int kABytes = kRows * 128;    // one A stage
constexpr int kProducers = 512;          // cp.async producers: teams of 128 (or 256 / 512) threads, 8 lanes per tile row
constexpr int kProducerWarps = kProducers / 32;
// Epilogue: warps kProducerWarps .. +7.  A warp can only read the TMEM lane quarter warp % 4, so two warps share each
// quarter and take alternate 32-column blocks (256-target kernel: alternate blocks of 32 targets): an epilogue warp is a
// serial chain of a few hundred instructions per block, and the last tile's epilogue of every launch is exposed.
constexpr int kEpilogueWarps = 8;
constexpr int kMmaWarp = kProducerWarps + kEpilogueWarps;
static_assert(kProducerWarps % 4 == 0, "epilogue warps must start at a multiple of 4");
constexpr int kConvThreads = (kMmaWarp + 1) * 32;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 224 * 1024;
constexpr int kScatterRing = 16;        // WS: scatter-row lists kept for tiles in flight (producers run at most kMaxStages tiles ahead of
                                        // the MMA, the MMA two tiles ahead of the epilogue)

struct Epilogue {
  const __half *bias;
  const float *scale;
  const float *shift;
  const __half *residual;
  int relu;
};

// Tile number of a persistent CTA's i-th turn.  Rounds alternate direction: grouped maps are sorted from the heaviest
// tile (most offsets present) to the lightest, so CTA 0 would otherwise receive the heaviest tile of every round.
__device__ __forceinline__ int snake_tile(int i) {
  const int G = gridDim.x, b = blockIdx.x;
  return i * G + ((i & 1) ? G - 1 - b : b);
}

struct ConvParams {
  // Input rows may come from two tensors that share the map (a channel concatenation that is never materialised):
  // channels [0, c_a) of a row from feats (row pitch c_a), channels [c_a, c_in) from feats_b (row pitch c_in - c_a).
  // One source: c_a == c_in.  A 16-byte piece (8 channels) never straddles the two: c_a is a multiple of 8.
  const __half *feats;
  const __half *feats_b;
  int c_a;
  const unsigned char *packed;
  __half *out;      // OS
  float *accum;     // WS
  Epilogue ep;
  int32_t *status;
  // OS
  const int32_t *map;           // [T_al][K]
  const int32_t *row_of;        // grouped map: output row of map row i (-1: padding), else null
  const uint32_t *tile_masks;   // grouped map: per 128 rows, bit k = some row has a neighbour at offset k, else null
  // WS
  const int32_t *in_idx, *out_idx, *naddrs, *qnaddrs;
  int rows, mirror, n_tiles_plain, centre_tiles;
  int fused;                 // WS: the CTAs meet at a grid barrier and convert the scratch themselves (cooperative launch)
  unsigned barrier_target;   // value of the device-wide arrival counter once every CTA of this launch has arrived
  // common
  int T, n_tiles, K, c_in, c_out, R, n_chunks;  // n_chunks: OS = ceil(R/64); WS = ceil(c_in/64) per offset
  int stages, teams, slab_bufs, b_bytes, acc_stride, tmem_cols;
  int off_b, off_slab, off_flags, off_cm, off_meta, off_bar;
  int off_ep;                   // per-channel epilogue constants as fp32: {bias, scale, shift, -}[256]
  int off_tr;                   // WS: per epilogue warp a 32 x 36-word tile for the transposition of the accumulator
  int ws_epilogue_warps;        // WS: 8 (two warps per lane quarter) where the tiles fit beside four stages, else 4
  // OS, 1x1x1 layer through the identity map: all weight chunks are fetched once and stay in shared memory
  // (chunk j at off_b + j * b_bytes) instead of travelling with every pipeline stage
  int resident;
  // OS, split reduction: `split` CTAs share one tile, CTA blockIdx.x % split takes every split-th non-empty chunk, the
  // partial sums meet in split_scratch [tile][split][c_out][128] fp32 and every CTA reduces c_out / split columns
  int split;
  float *split_scratch;
  unsigned *split_counters;     // [2][n_tiles]: arrivals and leavers per tile, zero between launches
  unsigned long long wait_ns;   // limit of every internal wait (mbarriers, grid barrier)
};

__device__ __forceinline__ float epilogue_apply(float v, int c, const Epilogue &ep) {
  if (ep.bias) v += __half2float(ep.bias[c]);
  if (ep.scale) v = v * ep.scale[c] + ep.shift[c];
  return v;
}

// Arrival counter of the grid barrier of fused weight-stationary launches.  It only ever grows: launch number n of a
// device (in stream order) waits for the value the host computed as the sum of the grid sizes up to and including n.
__device__ unsigned g_grid_arrivals = 0;

// kTma: the producers are ONE warp whose lanes each issue a TMA gather4 (4 feature rows x 128 bytes, zero fill for
// row index -1) per pipeline stage; otherwise 128 threads gather with 16-byte cp.async.
template <bool kWS, bool kTma>
__global__ void __launch_bounds__(kConvThreads, 1) conv_tc_kernel(const __grid_constant__ ConvParams P,
                                                                   const __grid_constant__ CUtensorMap tmap_feats) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);

  int32_t *slab = reinterpret_cast<int32_t *>(smem + P.off_slab);
  uint32_t *cmask = reinterpret_cast<uint32_t *>(smem + P.off_cm);
  int32_t *meta = reinterpret_cast<int32_t *>(smem + P.off_meta);
  const uint32_t bar0 = sbase + P.off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  auto bar_acc_full = [&](int b) { return bar0 + 8u * (2 * kMaxStages + b); };
  auto bar_acc_empty = [&](int b) { return bar0 + 8u * (2 * kMaxStages + 2 + b); };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + P.off_bar + 8 * (2 * kMaxStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + P.off_bar + 8 * (2 * kMaxStages + 4) + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int stages = P.stages;
  pdl_trigger();
  // ---- set-up that touches no global memory: it may overlap the drain of the kernel before this one
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full(s), kTma ? 1 : kRows + 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 32 * kEpilogueWarps);
    }
    mbar_init(bar0 + 8u * (2 * kMaxStages + 5), 1);   // resident weights (one bulk copy)
    mbar_init(bar0 + 8u * (2 * kMaxStages + 6), 1);   // map slab buffers (bulk copies)
    mbar_init(bar0 + 8u * (2 * kMaxStages + 7), 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), P.tmem_cols);
    tmem_relinquish();
  }
  // ---- everything the kernel reads from global memory (maps, lists, features, but also weights and epilogue constants,
  // which an earlier kernel on the stream may just have written) comes after this point
  pdl_wait();
  // tile counts: given by the host, or (weight-stationary lists whose sizes never left the device) read here
  int n_tiles = P.n_tiles, n_tiles_plain = P.n_tiles_plain;
  // weight-stationary: list offsets of all rows, staged once (finding the row of a tile is a walk over them, and a walk
  // over global memory costs one L2 round trip per step); visible to all roles after the set-up barrier below
  int32_t *s_naddrs = reinterpret_cast<int32_t *>(smem + P.off_flags);
  int32_t *s_qnaddrs = s_naddrs + ((P.rows + 1 + 3) & ~3);
  if constexpr (kWS) {
    for (int i = tid; i <= P.rows; i += kConvThreads) {
      s_naddrs[i] = P.naddrs[i];
      s_qnaddrs[i] = P.qnaddrs[i];
    }
    if (P.n_tiles < 0) {
      n_tiles_plain = P.qnaddrs[P.rows] >> 7;
      n_tiles = P.mirror ? 2 * n_tiles_plain - P.centre_tiles : n_tiles_plain;
    }
  }

  // The epilogue applies (acc + bias[c]) * scale[c] + shift[c] with one thread per ROW, i.e. every thread needs the
  // constants of every channel: they are staged once as fp32 (identity values where the caller gave none) and read
  // back as shared-memory broadcasts instead of three global loads per element.
  float4 *s_ep = reinterpret_cast<float4 *>(smem + P.off_ep);      // {bias, scale, shift, -} per channel: one 16-byte read
  if constexpr (!kWS) {      // (weight-stationary: the conversion pass applies the epilogue, the region does not exist)
    for (int c = tid; c < P.c_out; c += kConvThreads)
      s_ep[c] = make_float4(P.ep.bias ? __half2float(P.ep.bias[c]) : 0.f, P.ep.scale ? P.ep.scale[c] : 1.f,
                            P.ep.scale ? P.ep.shift[c] : 0.f, 0.f);
  }
  const bool has_affine = P.ep.bias != nullptr || P.ep.scale != nullptr;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // i-th tile of this CTA: the output-stationary cp.async path alternates the direction of the rounds
  const int split = (!kWS && !kTma) ? P.split : 1;
  const int split_rank = split > 1 ? static_cast<int>(blockIdx.x) % split : 0;
  auto tile_at = [&](int i) -> int {
    if constexpr (!kWS && !kTma) {
      if (split > 1) return i == 0 ? static_cast<int>(blockIdx.x) / split : 0x7fffffff;      // one tile per CTA
      return snake_tile(i);
    }
    return static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
  };

  if (kTma && warp < kProducerWarps) {
    // =========================== producer (TMA gather4): warp 0 only ===========================
    if (warp == 0) {
      const uint64_t tmap = reinterpret_cast<uint64_t>(&tmap_feats);
      const int cpo = P.n_chunks;  // 64-wide chunks per offset
      int stage = 0, phase = 0;
      bool ok = true;
      int tile_i = 0;
      const int slab_int4 = (kRows / 4) * P.K;
      if constexpr (!kWS) {
        if (static_cast<int>(blockIdx.x) < n_tiles) {
          const int4 *s4 = reinterpret_cast<const int4 *>(P.map + static_cast<int64_t>(blockIdx.x) * kRows * P.K);
          for (int i = lane; i < slab_int4; i += 32) cp_async_16(sbase + P.off_slab + i * 16, s4 + i, 16u);
        }
        cp_async_commit();
      }
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++tile_i) {
        int idx[4] = {-1, -1, -1, -1};
        int w_row = 0, n_offsets = 1;
        uint32_t kmask[16];
        const int32_t *my_slab = slab;
        if constexpr (kWS) {
          int tt = tile;
          const bool mirrored = tt >= n_tiles_plain;
          if (mirrored) tt -= n_tiles_plain;
          const int q0 = tt * kRows;
          int k = 0;
          while (k + 1 < P.rows && s_qnaddrs[k + 1] <= q0) ++k;
          const int p0 = s_naddrs[k] + (q0 - s_qnaddrs[k]);
          const int n = min(kRows, s_naddrs[k + 1] - p0);
          w_row = mirrored ? (P.K - 1 - k) : k;
          const int32_t *g = mirrored ? P.out_idx : P.in_idx;
          const int32_t *sc = mirrored ? P.in_idx : P.out_idx;
          int32_t *scatter = slab + kRows + (tile_i & (kScatterRing - 1)) * kRows;
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int m = 4 * lane + r;
            idx[r] = m < n ? g[p0 + m] : -1;
            scatter[m] = m < n ? sc[p0 + m] : -1;
          }
        } else {
          const int buf = (P.slab_bufs == 2) ? (tile_i & 1) : 0;
          my_slab = slab + buf * kRows * P.K;
          if (P.slab_bufs == 1 && tile_i > 0) {
            __syncwarp();
            const int4 *s4 = reinterpret_cast<const int4 *>(P.map + static_cast<int64_t>(tile) * kRows * P.K);
            for (int i = lane; i < slab_int4; i += 32) cp_async_16(sbase + P.off_slab + i * 16, s4 + i, 16u);
            cp_async_commit();
          }
          cp_async_wait<0>();
          __syncwarp();
          if (P.slab_bufs == 2) {
            const int next = tile + gridDim.x;
            if (next < n_tiles) {
              const int4 *n4 = reinterpret_cast<const int4 *>(P.map + static_cast<int64_t>(next) * kRows * P.K);
              const uint32_t dst = sbase + P.off_slab + (buf ^ 1) * kRows * P.K * 4;
              for (int i = lane; i < slab_int4; i += 32) cp_async_16(dst + i * 16, n4 + i, 16u);
            }
            cp_async_commit();
          }
          // offsets with at least one neighbour in this tile
#pragma unroll
          for (int w = 0; w < 16; ++w) kmask[w] = 0;
          n_offsets = 0;
          for (int k = 0; k < P.K; ++k) {
            int v = -1;
#pragma unroll
            for (int r = 0; r < 4; ++r) v = max(v, my_slab[(4 * lane + r) * P.K + k]);
            if (__ballot_sync(0xffffffffu, v >= 0)) {
              kmask[k >> 5] |= 1u << (k & 31);
              ++n_offsets;
            }
          }
          if (n_offsets == 0) { kmask[0] = 1u; n_offsets = 1; }   // a tile always sends at least one offset
        }
        const int total = n_offsets * cpo;
        int sent = 0;
        for (int kw = 0; ok && kw < (kWS ? 1 : ((P.K + 31) >> 5)); ++kw) {
          uint32_t bits = kWS ? 1u : kmask[kw];
          while (ok && bits) {
            const int k = (kw << 5) + __ffs(bits) - 1;
            bits &= bits - 1;
            if constexpr (!kWS) {
              w_row = k;
#pragma unroll
              for (int r = 0; r < 4; ++r) idx[r] = my_slab[(4 * lane + r) * P.K + k];
            }
            for (int jj = 0; jj < cpo; ++jj) {
              ++sent;
              if (!mbar_wait(bar_empty(stage), phase ^ 1, abort_flag, P.wait_ns)) { ok = false; break; }
              if (lane == 0) {
                const int valid = min(kChunk, P.c_in - jj * kChunk);
                meta[stage] = ((valid + 15) >> 4) | ((sent == 1) << 8) | ((sent == total) << 9);
                mbar_arrive_expect_tx(bar_full(stage), kABytes + P.b_bytes);
                bulk_g2s(sbase + P.off_b + stage * P.b_bytes,
                         P.packed + static_cast<int64_t>(w_row * cpo + jj) * P.b_bytes, P.b_bytes, bar_full(stage));
              }
              __syncwarp();
              tma_gather4(sbase + stage * kABytes + lane * 512, tmap, jj * kChunk, idx[0], idx[1], idx[2], idx[3],
                          bar_full(stage));
              if (++stage == stages) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
      cp_async_wait<0>();
    }
  } else if (warp < kProducerWarps) {
    // =========================== producers (cp.async) ===========================
    // The producer warps form teams of 4 warps (128 threads).  A team fills a whole pipeline stage: thread r copies
    // ONE 16-byte piece (r & 7) of 8 rows (r >> 3, +16, ...), zero-filling rows without a neighbour, so that the eight
    // lanes sharing a row read 128 contiguous bytes (a warp-level copy touches 4 rows; with one row per lane it would
    // touch 32 cache lines and the L1, which handles one line per cycle, becomes the limit).  The copies arrive on the
    // stage's mbarrier asynchronously; thread 0 of the team also posts the weight chunk.  Teams work on different
    // stages concurrently.  Stage s is ALWAYS filled by team s % teams: a
    // parity wait can only tell two consecutive phases of an mbarrier apart, so the waiter must have taken part in
    // every earlier phase of that barrier itself (stages is a multiple of teams).
    const int team = warp >> 2, r = tid & 127;
    const int teams = P.teams;
    const bool active = team < teams;
    const int piece = r & 7, rowbase = r >> 3;
    const uint32_t dst_off = rowbase * 128 + ((piece ^ (rowbase & 7)) << 4);   // (row & 7) == (rowbase & 7) for all 8 rows
    bool ok = true;
    int tile_i = 0;
    auto post_weights = [&](int stage, int chunk_id, int valid, bool first, bool last) {
      meta[stage] = ((valid + 15) >> 4) | (first << 8) | (last << 9) | (chunk_id << 16);
      if (!kWS && P.resident) {
        mbar_arrive(bar_full(stage));      // the chunk is in shared memory already
        return;
      }
      mbar_arrive_expect_tx(bar_full(stage), P.b_bytes);
      bulk_g2s(sbase + P.off_b + stage * P.b_bytes, P.packed + static_cast<int64_t>(chunk_id) * P.b_bytes, P.b_bytes,
               bar_full(stage));
    };
    if constexpr (kWS) {
      // ---- weight-stationary: a tile is 128 pairs of one offset; no CTA-level barriers
      // Pipeline item q = (CTA-local tile number) * cpo + (chunk of the tile) goes to stage q % stages; this team
      // owns the items with q % teams == team.  Tile number, chunk, stage and phase are advanced incrementally.
      const int cpo = P.n_chunks;
      int jj = team;
      while (jj >= cpo) { jj -= cpo; ++tile_i; }
      int my_stage = team;
      uint32_t my_phase = 0;
      int loaded_tile = -1, k_hint = 0, w_row = 0;
      int idx[8];
      bool hint_mirrored = false;
      while (active && ok) {
        const int tile = blockIdx.x + tile_i * gridDim.x;
        if (tile >= n_tiles) break;
        if (tile_i != loaded_tile) {
          loaded_tile = tile_i;
          int tt = tile;
          const bool mirrored = tt >= n_tiles_plain;
          if (mirrored) tt -= n_tiles_plain;
          const int q0 = tt * kRows;
          int k = (mirrored == hint_mirrored) ? k_hint : 0;     // tiles arrive in increasing order
          while (k + 1 < P.rows && s_qnaddrs[k + 1] <= q0) ++k;
          k_hint = k;
          hint_mirrored = mirrored;
          const int p0 = s_naddrs[k] + (q0 - s_qnaddrs[k]);
          const int n = min(kRows, s_naddrs[k + 1] - p0);
          w_row = mirrored ? (P.K - 1 - k) : k;
          const int32_t *g = mirrored ? P.out_idx : P.in_idx;
#pragma unroll
          for (int i = 0; i < 8; ++i) idx[i] = (rowbase + 16 * i) < n ? g[p0 + rowbase + 16 * i] : -1;
          // the scatter list (written by the team of the tile's first chunk) is read by the epilogue at most
          // kScatterRing - 1 tiles later
          if (jj == 0)
            slab[kRows + (tile_i & (kScatterRing - 1)) * kRows + r] = r < n ? (mirrored ? P.in_idx : P.out_idx)[p0 + r] : -1;
        }
        const int stage = my_stage;
        if (!mbar_wait(bar_empty(stage), my_phase ^ 1, abort_flag, P.wait_ns)) { ok = false; break; }
        if (r == 0) post_weights(stage, w_row * cpo + jj, min(kChunk, P.c_in - jj * kChunk), jj == 0, jj == cpo - 1);
        const uint32_t dst = sbase + stage * kABytes + dst_off;
        const int c = jj * kChunk + piece * 8;
        const bool second = c >= P.c_a;
        const __half *fbase = second ? P.feats_b + (c - P.c_a) : P.feats + c;
        const int64_t pitch = second ? P.c_in - P.c_a : P.c_a;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool take = idx[i] >= 0 && c < P.c_in;
          cp_async_16(dst + i * 2048, take ? fbase + idx[i] * pitch : P.feats, take ? 16u : 0u);
        }
        cp_async_mbar_arrive_noinc(bar_full(stage));
        my_stage += teams;
        if (my_stage >= stages) { my_stage -= stages; my_phase ^= 1; }
        jj += teams;
        while (jj >= cpo) { jj -= cpo; ++tile_i; }
      }
    } else {
      // ---- output-stationary: all producer warps prepare a tile together, the teams then take its non-empty
      // chunks in turn
      const float inv_c_in = 1.0f / static_cast<float>(P.c_in);
      const int n_words = (P.n_chunks + 31) >> 5;
      const uint32_t slab_bytes = kRows * P.K * 4;
      const uint32_t bar_slab0 = bar0 + 8u * (2 * kMaxStages + 6);
      uint32_t q_base = 0;
      int q_mod_teams = 0;            // q_base % teams
      int my_stage = team;            // stage of this team's next item (items of a team advance by `teams` stages)
      int my_slot = 0;                // my_stage / teams
      uint32_t my_phase = 0;
      // This thread always writes the same 8 (row, piece) places of its team's stages; bit slot * 8 + i remembers that
      // place i of stage slot * teams + team holds zeros, so the zero-fill for a missing neighbour (most of them are
      // missing) is skipped when the place is zero already.  stages / teams <= 4 slots.
      uint32_t zero_rows = 0;
      // P.map == nullptr: the identity map of a 1x1x1 layer (K == 1, two slab buffers): row t gathers row t, and the
      // producers write the 128 entries of a tile themselves instead of fetching them
      const bool identity = P.map == nullptr;
      if (tid == 0 && P.resident) {
        const uint32_t bar_wres = bar0 + 8u * (2 * kMaxStages + 5);
        mbar_arrive_expect_tx(bar_wres, static_cast<uint32_t>(P.n_chunks) * P.b_bytes);
        bulk_g2s(sbase + P.off_b, P.packed, static_cast<uint32_t>(P.n_chunks) * P.b_bytes, bar_wres);
      }
      if (tid == 0 && P.slab_bufs == 2 && tile_at(0) < n_tiles && !identity) {
        mbar_arrive_expect_tx(bar_slab0, slab_bytes);
        bulk_g2s(sbase + P.off_slab, P.map + static_cast<int64_t>(tile_at(0)) * kRows * P.K, slab_bytes, bar_slab0);
      }
      for (int w = tid; w < 2 * n_words; w += kProducers) cmask[w] = 0;
      // grouped maps come with the offsets present in each tile; the mask of the next tile is fetched a tile ahead
      uint32_t tile_mask = (P.tile_masks && tile_at(0) < n_tiles) ? P.tile_masks[tile_at(0)] : 0u;
      const bool have_masks = P.tile_masks != nullptr || identity;      // (identity: every tile has its one offset)
      if (identity) tile_mask = 1u;
      // Every thread runs the same sequence of named barriers; a failed wait only takes effect through the
      // OR-reduction of those barriers, so that all producer warps leave the loop in the same iteration.
      for (int tile = tile_at(0); tile < n_tiles; tile = tile_at(++tile_i)) {
        const int next = tile_at(tile_i + 1);
        const uint32_t this_mask = tile_mask;
        if (P.tile_masks && next < n_tiles) tile_mask = P.tile_masks[next];
        if (identity) tile_mask = 1u;
        const int buf = (P.slab_bufs == 2) ? (tile_i & 1) : 0;
        const int32_t *my_slab = slab + buf * kRows * P.K;
        uint32_t *my_cmask = cmask + (tile_i & 1) * n_words;
        if (P.slab_bufs == 2) {
          if (identity) {
            // (this buffer was last read two tiles ago, and every warp has passed the barrier of the tile in between)
            if (tid < kRows) {
              const int64_t t = static_cast<int64_t>(tile) * kRows + tid;
              slab[buf * kRows + tid] = t < P.T ? static_cast<int32_t>(t) : -1;
            }
          } else if (!mbar_wait(bar_slab0 + 8u * buf, (tile_i >> 1) & 1, abort_flag, P.wait_ns)) {
            ok = false;
          }
          // all warps have issued their share of the previous tile: the other slab and chunk mask are free
          if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
          if (tid == 0 && next < n_tiles && !identity) {
            mbar_arrive_expect_tx(bar_slab0 + 8u * (buf ^ 1), slab_bytes);
            bulk_g2s(sbase + P.off_slab + (buf ^ 1) * slab_bytes, P.map + static_cast<int64_t>(next) * kRows * P.K, slab_bytes,
                     bar_slab0 + 8u * (buf ^ 1));
          }
        } else {
          if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
          if (tid == 0) {
            mbar_arrive_expect_tx(bar_slab0, slab_bytes);
            bulk_g2s(sbase + P.off_slab, P.map + static_cast<int64_t>(tile) * kRows * P.K, slab_bytes, bar_slab0);
          }
          if (!mbar_wait(bar_slab0, tile_i & 1, abort_flag, P.wait_ns)) ok = false;
        }
        // which 64-wide reduction chunks touch at least one neighbour of this tile: one bit per chunk, the
        // chunks are spread over the warps
        for (int j = warp; j < P.n_chunks; j += kProducerWarps) {
          const int k_lo = __float2int_rd((static_cast<float>(j * kChunk) + 0.5f) * inv_c_in);
          const int k_hi = min(__float2int_rd((static_cast<float>(j * kChunk + kChunk - 8) + 0.5f) * inv_c_in), P.K - 1);
          bool any;
          if (have_masks) {
            any = (this_mask & ((0xffffffffu >> (31 - (k_hi - k_lo))) << k_lo)) != 0;    // K <= 32 for grouped maps
          } else {
            int v = -1;
            for (int k = k_lo; k <= k_hi; ++k)
#pragma unroll
              for (int qd = 0; qd < 4; ++qd) v = max(v, my_slab[(lane + 32 * qd) * P.K + k]);
            any = __ballot_sync(0xffffffffu, v >= 0) != 0;
          }
          if (any && lane == 0) atomicOr(&my_cmask[j >> 5], 1u << (j & 31));
        }
        if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
        // the mask of the NEXT tile starts from zero (its previous user, tile_i - 1, is finished for all warps)
        for (int w = tid; w < n_words; w += kProducers) cmask[((tile_i + 1) & 1) * n_words + w] = 0;
        int n_chunks_tile = 0;
        for (int w = 0; w < n_words; ++w) n_chunks_tile += __popc(my_cmask[w]);
        // A CTA always sends at least one chunk: a tile without neighbours, or (split reduction) a CTA whose share of the
        // tile's chunks is empty, sends chunk 0 with all rows zero.
        const bool force_first = (n_chunks_tile <= split_rank);
        int my_last = 0;                                 // the last chunk number e this CTA sends
        if (force_first) {
          n_chunks_tile = 1;
        } else {
          my_last = split_rank + (n_chunks_tile - 1 - split_rank) / split * split;
        }
        // Chunk number e (0-based, in increasing j) of the tile is pipeline item q = q_base + e and goes to stage
        // q % stages; this team owns the items with q % teams == team (teams divides stages).  All of it is tracked
        // incrementally: an integer division per chunk would dominate this latency-bound instruction stream.
        // (Split reduction: this CTA's items are the chunks e = rank, rank + split, ...; item number (e - rank) / split.)
        int word = 0, pos = 0;                           // walks the set bits of the mask: `pos` of them are behind
        uint32_t bits = force_first ? 1u : my_cmask[0];
        int e = team - q_mod_teams;
        if (e < 0) e += teams;
        const int e_step = teams * split;
        if (split > 1) e = force_first ? team : split_rank + team * split;
        for (; active && ok && e < n_chunks_tile; e += e_step) {
          while (true) {                                 // e < number of set bits, so the walk stays inside the mask
            while (bits == 0) bits = my_cmask[++word];
            if (pos == e) break;
            bits &= bits - 1;
            ++pos;
          }
          const int j = (word << 5) + __ffs(bits) - 1;
          const int stage = my_stage, slot_shift = my_slot * 8;
          if (!mbar_wait(bar_empty(stage), my_phase ^ 1, abort_flag, P.wait_ns)) { ok = false; break; }
          my_stage += teams;
          ++my_slot;
          if (my_stage >= stages) { my_stage -= stages; my_slot = 0; my_phase ^= 1; }
          if (r == 0) post_weights(stage, j, min(kChunk, P.R - j * kChunk), e == (force_first ? 0 : split_rank), e == my_last);
          // this thread's piece belongs to one offset k and starts at channel c of it
          const int rr = j * kChunk + piece * 8;
          const int k = __float2int_rd((static_cast<float>(rr) + 0.5f) * inv_c_in);
          const int c = rr - k * P.c_in;
          const bool piece_valid = rr < P.R;
          const uint32_t dst = sbase + stage * kABytes + dst_off;
          const int32_t *col = my_slab + rowbase * P.K + k;
          const uint32_t was_zero = zero_rows >> slot_shift;
          uint32_t now_zero = 0;
          // all map entries first: the copies below are compiler barriers, and a shared-memory load issued between
          // them would queue behind them in the load/store unit
          int idx[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) idx[i] = (piece_valid && !(force_first && split > 1)) ? col[i * 16 * P.K] : -1;
          const bool second = c >= P.c_a;
          const __half *fbase = second ? P.feats_b + (c - P.c_a) : P.feats + c;
          const int64_t pitch = second ? P.c_in - P.c_a : P.c_a;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const __half *src = idx[i] >= 0 ? fbase + idx[i] * pitch : P.feats;
            // a missing neighbour needs zeros: nothing to do if the previous fill of this stage left zeros there
            if (idx[i] >= 0 || !((was_zero >> i) & 1u)) cp_async_16(dst + i * 2048, src, idx[i] >= 0 ? 16u : 0u);
            now_zero |= (idx[i] >= 0 ? 0u : 1u) << i;
          }
          zero_rows = (zero_rows & ~(0xffu << slot_shift)) | (now_zero << slot_shift);
          cp_async_mbar_arrive_noinc(bar_full(stage));
        }
        q_base += n_chunks_tile;
        q_mod_teams += n_chunks_tile % teams;
        if (q_mod_teams >= teams) q_mod_teams -= teams;
      }
    }
    // nothing of this thread may still be in flight when the CTA tears down
    cp_async_wait_all();
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      const uint32_t idesc = idesc_f16_m128(P.c_out);
      int stage = 0, phase = 0;
      uint32_t acc_phase = 0;   // bit b: phase of accumulator buffer b
      bool ok = true;
      int tile_i = 0;
      const bool resident = !kWS && !kTma && P.resident;
      if (resident && tile_at(0) < n_tiles) ok = mbar_wait(bar0 + 8u * (2 * kMaxStages + 5), 0, abort_flag, P.wait_ns);
      for (int tile = tile_at(0); ok && tile < n_tiles; tile = tile_at(++tile_i)) {
        const int b = tile_i & 1;
        if (!mbar_wait(bar_acc_empty(b), ((acc_phase >> b) & 1u) ^ 1u, abort_flag, P.wait_ns)) break;
        acc_phase ^= 1u << b;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * P.acc_stride;
        while (true) {
          if (!mbar_wait(bar_full(stage), phase, abort_flag, P.wait_ns)) { ok = false; break; }
          fence_proxy_async();     // the rows were written by cp.async (generic proxy), the MMA reads them through the async proxy
          tc_fence_after();
          const int m = meta[stage];
          const int nk = m & 0xff;
          const bool first = (m >> 8) & 1, last = (m >> 9) & 1;
          // descriptors of the first 16-wide K step; each further step is 32 bytes (2 units of 16 bytes) on
          const uint64_t a_desc = smem_desc_k_sw128(sbase + stage * kABytes);
          const uint64_t b_desc = smem_desc_k_sw128(sbase + P.off_b + (resident ? (m >> 16) : stage) * P.b_bytes);
          for (int ks = 0; ks < nk; ++ks)
            mma_f16_ss(d_tmem, a_desc + 2 * ks, b_desc + 2 * ks, idesc, (first && ks == 0) ? 0u : 1u);
          mma_commit(bar_empty(stage));
          if (++stage == stages) { stage = 0; phase ^= 1; }
          if (last) {
            mma_commit(bar_acc_full(b));
            break;
          }
        }
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue ===========================
    const int q = warp & 3;
    const int half = (warp - kProducerWarps) >> 2;      // which of the two warps of this lane quarter
    const int row = q * 32 + lane;
    uint32_t *tr_ws = reinterpret_cast<uint32_t *>(smem + P.off_tr);
    const bool out_v8 = (reinterpret_cast<uintptr_t>(P.out) & 31) == 0;      // rows are multiples of 32 bytes (c_out % 16 == 0)
    uint32_t acc_phase = 0;   // bit b: phase of accumulator buffer b
    int tile_i = 0;
    for (int tile = tile_at(0); tile < n_tiles; tile = tile_at(++tile_i)) {
      const int b = tile_i & 1;
      int64_t out_row = -1;
      uint4 res_next[4];          // residual of the next 32 columns: requested before the wait for the accumulator / the TMEM load
      auto fetch_residual = [&](int c0) {
        if (out_row >= 0 && P.ep.residual && c0 < P.c_out) {
          const __half *src = P.ep.residual + out_row * P.c_out + c0;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (c0 + 8 * i < P.c_out) res_next[i] = *reinterpret_cast<const uint4 *>(src + 8 * i);
        }
      };
      if constexpr (!kWS) {
        // the output row and the first residual values are on their way while the tile's MMAs are still running
        const int64_t t = static_cast<int64_t>(tile) * kRows + row;
        out_row = t < P.T ? (P.row_of ? P.row_of[t] : t) : -1;
        if (split <= 1) fetch_residual(32 * half);
      }
      if (!mbar_wait(bar_acc_full(b), (acc_phase >> b) & 1u, abort_flag, P.wait_ns)) break;
      acc_phase ^= 1u << b;
      tc_fence_after();
      const uint32_t taddr = tmem_base + b * P.acc_stride + (static_cast<uint32_t>(q * 32) << 16);
      if constexpr (kWS) out_row = slab[kRows + (tile_i & (kScatterRing - 1)) * kRows + row];
      if constexpr (!kWS && !kTma) {
        if (split > 1 && half == 1) {      // (the split reduction is the work of one warp per lane quarter)
          tc_fence_before();
          mbar_arrive(bar_acc_empty(b));
          continue;
        }
        if (split > 1) {
          // ---- split reduction: park this CTA's partial sums (column-major, so that a warp writes 32 consecutive rows
          // of a column), meet the other CTAs of the tile, then reduce this CTA's share of the columns in a fixed order
          float *part = P.split_scratch + (static_cast<int64_t>(tile) * split + split_rank) * P.c_out * kRows + row;
          for (int c0 = 0; c0 < P.c_out; c0 += 16) {
            uint32_t h[16];
            tmem_ld_32x16(taddr + c0, h);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) __stcg(part + (c0 + i) * kRows, __uint_as_float(h[i]));
          }
          tc_fence_before();
          mbar_arrive(bar_acc_empty(b));
          __threadfence();
          named_bar_sync(2, kRows);
          if (q == 0 && lane == 0) {
            atomicAdd(P.split_counters + tile, 1u);
            const unsigned long long t0 = global_timer_ns();
            int polls = 0;
            while (*reinterpret_cast<volatile unsigned *>(P.split_counters + tile) < static_cast<unsigned>(split)) {
              if ((++polls & 31) == 0 && global_timer_ns() - t0 > P.wait_ns) { *abort_flag = 1; break; }
            }
            __threadfence();
          }
          named_bar_sync(2, kRows);
          if (*abort_flag != 0) break;
          const int cw = P.c_out / split, cbase = split_rank * cw;        // cw is a multiple of 8
          const float *all = P.split_scratch + static_cast<int64_t>(tile) * split * P.c_out * kRows + row;
          for (int c8 = 0; c8 < cw; c8 += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            for (int sp = 0; sp < split; ++sp) {
              const float *src = all + (static_cast<int64_t>(sp) * P.c_out + cbase + c8) * kRows;
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += __ldcg(src + i * kRows);
            }
            if (out_row >= 0) {
              const int c = cbase + c8;
              uint4 rv = make_uint4(0, 0, 0, 0);
              if (P.ep.residual) rv = *reinterpret_cast<const uint4 *>(P.ep.residual + out_row * P.c_out + c);
              const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
              uint4 pack;
              uint32_t *pw = reinterpret_cast<uint32_t *>(&pack);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float v0 = epilogue_apply(v[2 * e], c + 2 * e, P.ep);
                float v1 = epilogue_apply(v[2 * e + 1], c + 2 * e + 1, P.ep);
                if (P.ep.residual) { v0 += __low2float(rh[e]); v1 += __high2float(rh[e]); }
                if (P.ep.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
                const __half2 hv = __floats2half2_rn(v0, v1);
                pw[e] = *reinterpret_cast<const uint32_t *>(&hv);
              }
              *reinterpret_cast<uint4 *>(P.out + out_row * P.c_out + c) = pack;
            }
          }
          // the last CTA to leave the tile clears its counters for the next launch
          named_bar_sync(2, kRows);
          if (q == 0 && lane == 0) {
            unsigned *leavers = P.split_counters + n_tiles + tile;
            if (atomicAdd(leavers, 1u) == static_cast<unsigned>(split) - 1u) {
              P.split_counters[tile] = 0u;
              *leavers = 0u;
            }
          }
          continue;
        }
      }
      const bool both_halves = !kWS || P.ws_epilogue_warps == kEpilogueWarps;
      for (int c0 = both_halves ? 32 * half : (half == 0 ? 0 : P.c_out); c0 < P.c_out; c0 += both_halves ? 64 : 32) {
        uint32_t r[32];
        const bool full = c0 + 32 <= P.c_out;
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
        if constexpr (kWS) {
          // A thread holds 32 channels of ONE pair, so a vector reduction issued from these registers touches 32 rows
          // per warp instruction (32 wavefronts).  The block goes through a 32 x 36-word tile instead and comes back
          // with eight lanes per row: one instruction then covers 4 rows x 128 contiguous bytes (4 wavefronts) with the
          // same sixteen-byte reductions.  (Scalar reductions of 32 consecutive channels per instruction were measured
          // 1.5x slower: the L2 performs one operation per reduction, whatever its width.)
          uint32_t *tile = tr_ws + (warp - kProducerWarps) * (32 * 36);
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<uint4 *>(tile + lane * 36 + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
          __syncwarp();
          const int32_t *rows_of_warp = slab + kRows + (tile_i & (kScatterRing - 1)) * kRows + q * 32;
          const int sub = lane >> 3, col = (lane & 7) * 4;
          if (col < width) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int rr = 4 * k + sub;
              const int orow = rows_of_warp[rr];
              const uint4 v = *reinterpret_cast<const uint4 *>(tile + rr * 36 + col);
              if (orow >= 0)
                red_add_v4_f32(P.accum + static_cast<int64_t>(orow) * P.c_out + c0 + col, __uint_as_float(v.x), __uint_as_float(v.y),
                               __uint_as_float(v.z), __uint_as_float(v.w));
            }
          }
          __syncwarp();
        } else {
          if (out_row >= 0) {
            __half *dst = P.out + out_row * P.c_out + c0;
            const bool res = P.ep.residual != nullptr;
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
                    if (P.ep.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
                    __half2 hv = __floats2half2_rn(v0, v1);
                    pw[e] = *reinterpret_cast<uint32_t *>(&hv);
                  }
                }
                // 16 channels = one 32-byte sector: a single 256-bit store where the output allows it (two 16-byte
                // stores of a thread reach L2 as two partial-sector writes and cost two transactions)
                if (out_v8) {
                  st_global_v8(dst + i, pack[0], pack[1]);
                } else {
                  *reinterpret_cast<uint4 *>(dst + i) = pack[0];
                  *reinterpret_cast<uint4 *>(dst + i + 8) = pack[1];
                }
              }
            }
            fetch_residual(c0 + 64);      // (the accumulator registers are free again: no pressure from the values in flight)
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_acc_empty(b));
    }
    if constexpr (kWS) {
      if (P.fused) __threadfence();      // this thread's reductions are performed before the CTA arrives at the grid barrier
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    // a bounded wait expired: report, give copies in flight time to land, then release TMEM
    if (tid == 0 && P.status) atomicExch(P.status, 1);
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if constexpr (kWS) {
    if (P.fused) {
      // ---- grid barrier (all CTAs are resident: cooperative launch), then every CTA converts its slice of the scratch:
      // fp32 sums -> epilogue -> fp16 output, and the slice is zeroed again for the next layer that uses the scratch.
      // Every CTA arrives exactly once, also after a failed wait, so the counter stays in step with the host.
      __shared__ int s_go;
      if (tid == 0) {
        __threadfence();
        atomicAdd(&g_grid_arrivals, 1u);
        bool arrived = false;
        if (*abort_flag == 0) {
          const unsigned long long t0 = global_timer_ns();
          while (true) {
            const unsigned seen = *reinterpret_cast<volatile unsigned *>(&g_grid_arrivals);
            if (static_cast<int>(seen - P.barrier_target) >= 0) { arrived = true; break; }
            if (global_timer_ns() - t0 > P.wait_ns) break;
          }
          if (!arrived && P.status) atomicExch(P.status, 1);
        }
        __threadfence();
        s_go = arrived ? 1 : 0;
      }
      __syncthreads();
      if (s_go) {
        const int64_t n4 = static_cast<int64_t>(P.T) * P.c_out / 4;      // c_out % 16 == 0: a float4 stays in one row
        const int64_t per = (n4 + gridDim.x - 1) / gridDim.x;
        const int64_t lo = per * blockIdx.x, hi = min(n4, lo + per);
        float4 *acc4 = reinterpret_cast<float4 *>(P.accum);
        for (int64_t i = lo + tid; i < hi; i += kConvThreads) {
          const float4 a = __ldcg(acc4 + i);
          const int c = static_cast<int>((i * 4) % P.c_out);
          float v[4] = {epilogue_apply(a.x, c, P.ep), epilogue_apply(a.y, c + 1, P.ep), epilogue_apply(a.z, c + 2, P.ep),
                        epilogue_apply(a.w, c + 3, P.ep)};
          if (P.ep.residual) {
            const uint2 rv = *reinterpret_cast<const uint2 *>(P.ep.residual + i * 4);
            const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
            v[0] += __low2float(rh[0]); v[1] += __high2float(rh[0]); v[2] += __low2float(rh[1]); v[3] += __high2float(rh[1]);
          }
          if (P.ep.relu) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = fmaxf(v[e], 0.f);
          }
          const __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t *>(&h0);
          o.y = *reinterpret_cast<const uint32_t *>(&h1);
          *reinterpret_cast<uint2 *>(P.out + i * 4) = o;
          __stcg(acc4 + i, make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
    }
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, P.tmem_cols);
  }
}

// =====================================================================================================================
// Output-stationary kernel for c_out <= 128: the operand roles are exchanged.  The tensor pipe spends ~128 cycles on an
// M=128, K=16 MMA whatever N <= 256 is, so a narrow layer (N = c_out = 32..128) wastes most of it.  Here the WEIGHTS are
// the M operand (c_out rows padded to 128; the padding rows read whatever follows in shared memory and produce
// accumulator rows nobody reads) and 256 TARGETS are the N operand: one MMA covers two 128-target tiles.
// Accumulator: TMEM lane = output channel, column = target.  Epilogue thread c owns channel c, so bias / scale / shift
// are per-thread constants, and for a fixed target the 32 lanes of a warp store 32 consecutive channels (64 bytes).
// =====================================================================================================================
constexpr int kN2Rows = 256;                 // targets per tile (MMA N)
constexpr int kN2FeatBytes = kN2Rows * 128;  // one feature stage

struct ConvN2Params {
  const __half *feats;          // channels [0, c_a) of an input row, row pitch c_a
  const __half *feats_b;        // channels [c_a, c_in), row pitch c_in - c_a (one source: c_a == c_in)
  int c_a;
  const unsigned char *packed;
  __half *out;
  Epilogue ep;
  int32_t *status;
  const int32_t *map;           // [T_al][K]
  const int32_t *row_of;        // grouped map: output row of map row i (-1: padding), else null
  const uint32_t *tile_masks;   // grouped map: per 128 rows, bit k = some row has a neighbour at offset k, else null
  int T, T_al, n_tiles, K, c_in, c_out, R, n_chunks;
  int stages, w_bytes, w_stride;
  int off_feat, off_slab, off_tr, off_cm, off_meta, off_bar;
  unsigned long long wait_ns;   // limit of every internal wait
};

// Producer teams of 128 threads fill one stage together (4 teams; 8 lanes per row, so a thread owns one 16-byte piece
// of 16 rows).  Stage s is filled by team s % 4.  (Teams of 256 or 512 threads were measured equal or slower.)
constexpr int kN2TeamThreads = 128;
__global__ void __launch_bounds__(kConvThreads, 1) conv_os_n256_kernel(const __grid_constant__ ConvN2Params P) {
  constexpr int kRowsPerThread = kN2Rows * 8 / kN2TeamThreads;   // 16
  constexpr int kRowStep = kN2TeamThreads / 8;                   // rows between two places of a thread
  constexpr uint32_t kSlotMask = (1u << kRowsPerThread) - 1u;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  unsigned char *smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const uint32_t sbase = smem_u32(smem);
  int32_t *slab = reinterpret_cast<int32_t *>(smem + P.off_slab);
  uint32_t *cmask = reinterpret_cast<uint32_t *>(smem + P.off_cm);
  int32_t *meta = reinterpret_cast<int32_t *>(smem + P.off_meta);
  const uint32_t bar0 = sbase + P.off_bar;
  auto bar_full = [&](int s) { return bar0 + 8u * s; };
  auto bar_empty = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
  auto bar_acc_full = [&](int b) { return bar0 + 8u * (2 * kMaxStages + b); };
  auto bar_acc_empty = [&](int b) { return bar0 + 8u * (2 * kMaxStages + 2 + b); };
  const uint32_t bar_slab = bar0 + 8u * (2 * kMaxStages + 6);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + P.off_bar + 8 * (2 * kMaxStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + P.off_bar + 8 * (2 * kMaxStages + 4) + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_trigger();
  const int stages = P.stages;
  constexpr int kTeams = kProducers / kN2TeamThreads;   // 4

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full(s), kN2TeamThreads + 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 32 * kEpilogueWarps);
    }
    mbar_init(bar_slab, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();      // from here on the kernel reads what earlier kernels on the stream wrote

  if (warp < kProducerWarps) {
    // =========================== producers: teams of 128 threads, stage s is filled by team s % kTeams ======
    // Thread r of a team owns ONE 16-byte piece (r & 7) of kRowsPerThread rows (r >> 3, + kRowStep, ...): the eight lanes
    // that share a row read 128 contiguous bytes, so a warp-level copy touches 4 rows instead of 32 different cache lines
    // (the L1 processes one line per cycle: a thread-per-row mapping is bound by that, not by bandwidth).
    const int team = tid / kN2TeamThreads, r = tid % kN2TeamThreads;
    const int piece = r & 7, rowbase = r >> 3;
    const uint32_t dst_off = rowbase * 128 + ((piece ^ (rowbase & 7)) << 4);   // (row & 7) == (rowbase & 7) for all rows
    const float inv_c_in = 1.0f / static_cast<float>(P.c_in);
    const int n_words = (P.n_chunks + 31) >> 5;
    bool ok = true;
    int tile_i = 0, q_mod_teams = 0, my_stage = team, my_slot = 0;
    uint32_t my_phase = 0;
    // Most neighbours of an output-stationary tile are missing (~70 % on LiDAR scenes) and their rows must read as
    // zeros.  This thread always writes the same (row, piece) places of the same stages (stage = slot * kTeams + team),
    // so it remembers which of them hold zeros (bit slot * kRowsPerThread + i) and skips the zero-fill of a place that is
    // zero already.
    uint32_t zero_rows = 0;
    for (int w = tid; w < 2 * n_words; w += kProducers) cmask[w] = 0;
    // grouped maps come with the offsets present in each 128-row tile; the masks of the next tile are fetched a tile ahead
    const int n_tiles128 = P.T_al >> 7;
    auto load_tile_mask = [&](int tile) -> uint32_t {
      if (!P.tile_masks || tile >= P.n_tiles) return 0u;
      uint32_t m = P.tile_masks[2 * tile];
      if (2 * tile + 1 < n_tiles128) m |= P.tile_masks[2 * tile + 1];
      return m;
    };
    uint32_t tile_mask = load_tile_mask(snake_tile(0));
    for (int tile = snake_tile(0); tile < P.n_tiles; tile = snake_tile(++tile_i)) {
      const uint32_t this_mask = tile_mask;
      tile_mask = load_tile_mask(snake_tile(tile_i + 1));
      uint32_t *my_cmask = cmask + (tile_i & 1) * n_words;
      // every warp has issued its share of the previous tile: the slab may be overwritten
      if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
      const int t0 = tile * kN2Rows;
      const int rows_here = min(kN2Rows, P.T_al - t0);          // the map has T_al rows (a multiple of 128)
      if (tid == 0) {
        const uint32_t bytes = static_cast<uint32_t>(rows_here) * P.K * 4;
        mbar_arrive_expect_tx(bar_slab, bytes);
        bulk_g2s(sbase + P.off_slab, P.map + static_cast<int64_t>(t0) * P.K, bytes, bar_slab);
      }
      for (int i = rows_here * P.K + tid; i < kN2Rows * P.K; i += kProducers) slab[i] = -1;
      if (!mbar_wait(bar_slab, tile_i & 1, abort_flag, P.wait_ns)) ok = false;
      if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
      // non-empty 64-wide reduction chunks of this tile (one bit per chunk), spread over the warps
      for (int j = warp; j < P.n_chunks; j += kProducerWarps) {
        const int k_lo = __float2int_rd((static_cast<float>(j * kChunk) + 0.5f) * inv_c_in);
        const int k_hi = min(__float2int_rd((static_cast<float>(j * kChunk + kChunk - 8) + 0.5f) * inv_c_in), P.K - 1);
        bool any;
        if (P.tile_masks) {
          any = (this_mask & ((0xffffffffu >> (31 - (k_hi - k_lo))) << k_lo)) != 0;      // K <= 32 for grouped maps
        } else {
          int v = -1;
          for (int k = k_lo; k <= k_hi; ++k)
#pragma unroll
            for (int qd = 0; qd < 8; ++qd) v = max(v, slab[(lane + 32 * qd) * P.K + k]);
          any = __ballot_sync(0xffffffffu, v >= 0) != 0;
        }
        if (any && lane == 0) atomicOr(&my_cmask[j >> 5], 1u << (j & 31));
      }
      if (named_bar_red_or(1, kProducers, !ok || *abort_flag != 0)) break;
      for (int w = tid; w < n_words; w += kProducers) cmask[((tile_i + 1) & 1) * n_words + w] = 0;
      int n_chunks_tile = 0;
      for (int w = 0; w < n_words; ++w) n_chunks_tile += __popc(my_cmask[w]);
      const bool force_first = (n_chunks_tile == 0);
      if (force_first) n_chunks_tile = 1;
      int word = 0, pos = 0;                             // walks the set bits of the mask: `pos` of them are behind
      uint32_t bits = force_first ? 1u : my_cmask[0];
      int e = team - q_mod_teams;
      if (e < 0) e += kTeams;
      for (; ok && e < n_chunks_tile; e += kTeams) {
        while (true) {                                   // e < number of set bits, so the walk stays inside the mask
          while (bits == 0) bits = my_cmask[++word];
          if (pos == e) break;
          bits &= bits - 1;
          ++pos;
        }
        const int j = (word << 5) + __ffs(bits) - 1;
        const int stage = my_stage, slot_shift = my_slot * kRowsPerThread;
        if (!mbar_wait(bar_empty(stage), my_phase ^ 1, abort_flag, P.wait_ns)) { ok = false; break; }
        my_stage += kTeams;
        ++my_slot;
        if (my_stage >= stages) { my_stage -= stages; my_slot = 0; my_phase ^= 1; }
        if (r == 0) {
          const int valid = min(kChunk, P.R - j * kChunk);
          meta[stage] = ((valid + 15) >> 4) | ((e == 0) << 8) | ((e == n_chunks_tile - 1) << 9);
          mbar_arrive_expect_tx(bar_full(stage), P.w_bytes);
          bulk_g2s(sbase + stage * P.w_stride, P.packed + static_cast<int64_t>(j) * P.w_bytes, P.w_bytes, bar_full(stage));
        }
        // this thread's piece belongs to one offset k and starts at channel c of it
        const int rr = j * kChunk + piece * 8;
        const int k = __float2int_rd((static_cast<float>(rr) + 0.5f) * inv_c_in);
        const int c = rr - k * P.c_in;
        const bool piece_valid = rr < P.R;
        const uint32_t dst = sbase + P.off_feat + stage * kN2FeatBytes + dst_off;
        const int32_t *col = slab + rowbase * P.K + k;
        const uint32_t was_zero = zero_rows >> slot_shift;
        uint32_t now_zero = 0;
        // all map entries first: the copies below are compiler barriers, and a shared-memory load issued between them
        // would queue behind them in the load/store unit
        int idx[kRowsPerThread];
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) idx[i] = piece_valid ? col[i * kRowStep * P.K] : -1;
        const bool second = c >= P.c_a;
        const __half *fbase = second ? P.feats_b + (c - P.c_a) : P.feats + c;
        const int64_t pitch = second ? P.c_in - P.c_a : P.c_a;
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
          const __half *src = idx[i] >= 0 ? fbase + idx[i] * pitch : P.feats;
          // a missing neighbour needs zeros: nothing to do if the previous fill of this stage left zeros there
          if (idx[i] >= 0 || !((was_zero >> i) & 1u)) cp_async_16(dst + i * (kRowStep * 128), src, idx[i] >= 0 ? 16u : 0u);
          now_zero |= (idx[i] >= 0 ? 0u : 1u) << i;
        }
        zero_rows = (zero_rows & ~(kSlotMask << slot_shift)) | (now_zero << slot_shift);
        cp_async_mbar_arrive_noinc(bar_full(stage));
      }
      q_mod_teams += n_chunks_tile % kTeams;
      if (q_mod_teams >= kTeams) q_mod_teams -= kTeams;
    }
    cp_async_wait_all();
  } else if (warp == kMmaWarp) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      // fp16 x fp16 -> fp32, both K-major, M = 128 (channels), N = 256 (targets)
      const uint32_t idesc = (1u << 4) | ((static_cast<uint32_t>(kN2Rows) >> 3) << 17) | ((128u >> 4) << 24);
      int stage = 0, phase = 0;
      uint32_t acc_phase = 0;   // bit b: phase of accumulator buffer b
      bool ok = true;
      int tile_i = 0;
      for (int tile = snake_tile(0); ok && tile < P.n_tiles; tile = snake_tile(++tile_i)) {
        const int b = tile_i & 1;
        if (!mbar_wait(bar_acc_empty(b), ((acc_phase >> b) & 1u) ^ 1u, abort_flag, P.wait_ns)) break;
        acc_phase ^= 1u << b;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * kN2Rows;
        while (true) {
          if (!mbar_wait(bar_full(stage), phase, abort_flag, P.wait_ns)) { ok = false; break; }
          fence_proxy_async();     // the rows were written by cp.async (generic proxy), the MMA reads them through the async proxy
          tc_fence_after();
          const int m = meta[stage];
          const int nk = m & 0xff;
          const bool first = (m >> 8) & 1, last = (m >> 9) & 1;
          const uint64_t w_desc = smem_desc_k_sw128(sbase + stage * P.w_stride);
          const uint64_t f_desc = smem_desc_k_sw128(sbase + P.off_feat + stage * kN2FeatBytes);
          for (int ks = 0; ks < nk; ++ks)
            mma_f16_ss(d_tmem, w_desc + 2 * ks, f_desc + 2 * ks, idesc, (first && ks == 0) ? 0u : 1u);
          mma_commit(bar_empty(stage));
          if (++stage == stages) { stage = 0; phase ^= 1; }
          if (last) {
            mma_commit(bar_acc_full(b));
            break;
          }
        }
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue ===========================
    // Accumulator lane = output channel, column = target.  Thread c applies the per-channel affine (its own constants)
    // to the fp32 accumulator of channel c for 32 targets at a time and parks the fp32 values, 16 targets per pass, in a
    // small per-warp tile.  The warp reads the tile transposed: thread (target tl = lane & 15, channel half lane >> 4)
    // then holds 16 consecutive channels of ONE target in fp32, adds the residual (two 16-byte loads), applies the
    // ReLU, rounds ONCE to fp16 and writes two 16-byte stores.
    const int q = warp & 3;
    const int c = q * 32 + lane;
    const bool has_channel = c < P.c_out;
    const int n_valid = min(32, P.c_out - q * 32);          // channels of this warp that exist (a multiple of 16)
    const float bias = (has_channel && P.ep.bias) ? __half2float(P.ep.bias[c]) : 0.f;
    const float scale = (has_channel && P.ep.scale) ? P.ep.scale[c] : 1.f;
    const float shift = (has_channel && P.ep.shift) ? P.ep.shift[c] : 0.f;
    const bool relu = P.ep.relu != 0;
    const int tl = lane & 15, ch0 = (lane >> 4) * 16;       // second half of a pass: this thread's target and first channel
    const int half = (warp - kProducerWarps) >> 2;          // the two warps of a lane quarter take alternate blocks of 32 targets
    uint32_t *tr = reinterpret_cast<uint32_t *>(smem + P.off_tr) + (warp - kProducerWarps) * (32 * 17);
    uint32_t acc_phase = 0;   // bit b: phase of accumulator buffer b
    int tile_i = 0;
    const bool has_res = P.ep.residual != nullptr;
    const bool out_v8 = (reinterpret_cast<uintptr_t>(P.out) & 31) == 0;      // 16 channels of a row are one aligned 32-byte sector
    for (int tile = snake_tile(0); tile < P.n_tiles; tile = snake_tile(++tile_i)) {
      const int b = tile_i & 1;
      const int64_t t0 = static_cast<int64_t>(tile) * kN2Rows;
      // Output rows and residual values do not depend on the accumulator: under the load of the row gathers a dependent
      // global load takes ~2 k cycles, so they are fetched ahead -- the output rows two blocks of 32 targets ahead, the
      // residual one block ahead, the first ones while the tile's MMAs are still running.
      auto orow_of = [&](int jb) -> int {      // output row of target jb * 32 + lane (-1: none)
        const int64_t t = t0 + jb * 32 + lane;
        return (jb < kN2Rows / 32 && t < P.T) ? (P.row_of ? P.row_of[t] : static_cast<int>(t)) : -1;
      };
      uint4 res[2][2];
      auto fetch_residual = [&](int orow_lane, int h) {      // (all lanes take part in the shuffle)
        const int orow = __shfl_sync(0xffffffffu, orow_lane, 16 * h + tl);
        if (has_res && orow >= 0 && ch0 < n_valid) {
          const __half *src = P.ep.residual + static_cast<int64_t>(orow) * P.c_out + q * 32 + ch0;
          res[h][0] = *reinterpret_cast<const uint4 *>(src);
          res[h][1] = *reinterpret_cast<const uint4 *>(src + 8);
        }
      };
      int orow_cur = orow_of(half), orow_next = orow_of(half + 2);
      fetch_residual(orow_cur, 0);
      fetch_residual(orow_cur, 1);
      if (!mbar_wait(bar_acc_full(b), (acc_phase >> b) & 1u, abort_flag, P.wait_ns)) break;
      acc_phase ^= 1u << b;
      tc_fence_after();
      if (n_valid > 0) {
        const uint32_t taddr = tmem_base + b * kN2Rows + (static_cast<uint32_t>(q * 32) << 16);
        for (int jb = half; jb < kN2Rows / 32; jb += 2) {
          if (t0 + jb * 32 >= P.T) break;                       // warp-uniform: no target left in this block
          const int orow_after = orow_of(jb + 4);
          uint32_t v[32];
          tmem_ld_32x32(taddr + jb * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              tr[lane * 17 + i] = __float_as_uint((__uint_as_float(v[16 * h + i]) + bias) * scale + shift);
            __syncwarp();
            const int orow = __shfl_sync(0xffffffffu, orow_cur, 16 * h + tl);
            float x[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) x[m] = __uint_as_float(tr[(ch0 + m) * 17 + tl]);
            __syncwarp();
            const bool mine = orow >= 0 && ch0 < n_valid;
            if (mine && has_res) {
              const __half2 *rh0 = reinterpret_cast<const __half2 *>(&res[h][0]), *rh1 = reinterpret_cast<const __half2 *>(&res[h][1]);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                x[2 * e] += __low2float(rh0[e]); x[2 * e + 1] += __high2float(rh0[e]);
                x[8 + 2 * e] += __low2float(rh1[e]); x[8 + 2 * e + 1] += __high2float(rh1[e]);
              }
            }
            fetch_residual(orow_next, h);                       // the same half of the next block
            if (mine) {
              const int64_t base = static_cast<int64_t>(orow) * P.c_out + q * 32 + ch0;
              uint32_t y[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                float a0 = x[2 * e], a1 = x[2 * e + 1];
                if (relu) { a0 = fmaxf(a0, 0.f); a1 = fmaxf(a1, 0.f); }
                const __half2 hv = __floats2half2_rn(a0, a1);       // the single rounding
                y[e] = *reinterpret_cast<const uint32_t *>(&hv);
              }
              if (out_v8) {
                st_global_v8(P.out + base, make_uint4(y[0], y[1], y[2], y[3]), make_uint4(y[4], y[5], y[6], y[7]));
              } else {
                *reinterpret_cast<uint4 *>(P.out + base) = make_uint4(y[0], y[1], y[2], y[3]);
                *reinterpret_cast<uint4 *>(P.out + base + 8) = make_uint4(y[4], y[5], y[6], y[7]);
              }
            }
          }
          orow_cur = orow_next;
          orow_next = orow_after;
        }
      }
      tc_fence_before();
      mbar_arrive(bar_acc_empty(b));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) {
    if (tid == 0 && P.status) atomicExch(P.status, 1);
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- weight image ---------------------------------------------------------------------------

// one thread per 16-byte piece of the image: chunk j, row n (output channel), piece p
__global__ void __launch_bounds__(256) pack_weights_kernel(const __half *__restrict__ w, int K, int c_in, int c_out,
                                                            int ws_mode, int chunks_per_offset, int64_t n_pieces,
                                                            unsigned char *__restrict__ packed) {
  int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (g >= n_pieces) return;
  const int p = static_cast<int>(g & 7);
  const int n = static_cast<int>((g >> 3) % c_out);
  const int64_t j = (g >> 3) / c_out;
  __align__(16) __half v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int k, c;
    bool valid;
    if (ws_mode) {
      k = static_cast<int>(j / chunks_per_offset);
      c = static_cast<int>(j % chunks_per_offset) * kChunk + p * 8 + e;
      valid = c < c_in;
    } else {
      int64_t r = j * kChunk + p * 8 + e;
      k = static_cast<int>(r / c_in);
      c = static_cast<int>(r % c_in);
      valid = k < K;
    }
    v[e] = valid ? w[(static_cast<int64_t>(k) * c_in + c) * c_out + n] : __float2half(0.f);
  }
  unsigned char *dst = packed + j * (static_cast<int64_t>(c_out) * 128) + n * 128 + ((p ^ (n & 7)) << 4);
  *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(v);
}

// ---- SIMT kernels (any channel count) -----------------------------------------------------------

// one warp per target row; lanes over output channels
__global__ void __launch_bounds__(128) conv_os_simt_kernel(const __half *__restrict__ feats,
                                                            const __half *__restrict__ w, Epilogue ep,
                                                            const int32_t *__restrict__ map, int64_t T, int K, int c_in,
                                                            int c_out, __half *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * int64_t(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  for (int co = lane; co < c_out; co += 32) {
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const int m = map[t * K + k];
      if (m < 0) continue;
      const __half *f = feats + static_cast<int64_t>(m) * c_in;
      const __half *wk = w + static_cast<int64_t>(k) * c_in * c_out + co;
      for (int ci = 0; ci < c_in; ++ci) acc = fmaf(__half2float(f[ci]), __half2float(wk[static_cast<int64_t>(ci) * c_out]), acc);
    }
    float v = epilogue_apply(acc, co, ep);
    if (ep.residual) v += __half2float(ep.residual[t * c_out + co]);
    if (ep.relu) v = fmaxf(v, 0.f);
    out[t * c_out + co] = __float2half_rn(v);
  }
}


// Output-stationary kernel for the network stems (3-8 input channels, 16/32/64 output channels): far too little
// arithmetic for the tensor cores and rows too short for 16-byte gathers.  One thread keeps all COUT accumulators of
// one target (row tid of the block's 128-row tile) in registers; the weights sit in shared memory as fp32 and are read
// as broadcast float4; the tile's map slab is staged with coalesced 16-byte loads.  On a grouped map (rows sorted by
// neighbour pattern) the lanes of a warp skip the same offsets: 36 -> 26 us on the 4 -> 32 stem of a 127 k-voxel
// scene.  (Two targets per thread, or the row loads of nine offsets issued together, were measured slower: they cost
// registers and shared memory, and the resident warps they displace were worth more.)
template <int COUT>
__global__ void __launch_bounds__(128) conv_os_stem_kernel(const __half *__restrict__ feats, const __half *__restrict__ w,
                                                            Epilogue ep, const int32_t *__restrict__ map,
                                                            const int32_t *__restrict__ row_of, int64_t T, int K,
                                                            int c_in, __half *__restrict__ out) {
  extern __shared__ __align__(16) unsigned char stem_smem[];
  float *ws = reinterpret_cast<float *>(stem_smem);                              // [K][c_in][COUT]
  int32_t *slab = reinterpret_cast<int32_t *>(stem_smem + static_cast<size_t>(K) * c_in * COUT * 4);   // [128][K]
  const int tid = threadIdx.x;
  pdl_trigger();
  pdl_wait();      // (before the first global read: also the weights may have been written by the kernel before this one)
  if (reinterpret_cast<uintptr_t>(w) % 16 == 0) {                               // (COUT is a multiple of 16: whole 8-value groups)
    for (int i = tid; i < K * c_in * COUT / 8; i += 128) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(w) + i);
      const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f2 = __half22float2(h[e]);
        ws[8 * i + 2 * e] = f2.x;
        ws[8 * i + 2 * e + 1] = f2.y;
      }
    }
  } else {
    for (int i = tid; i < K * c_in * COUT; i += 128) ws[i] = __half2float(w[i]);
  }
  // the map has T_al rows (T rounded up to 128): every block finds its 128 rows
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * 128;
  const int4 *s4 = reinterpret_cast<const int4 *>(map + t0 * K);
  for (int i = tid; i < 32 * K; i += 128) reinterpret_cast<int4 *>(slab)[i] = s4[i];
  __syncthreads();
  float acc[COUT];
#pragma unroll
  for (int co = 0; co < COUT; ++co) acc[co] = 0.f;
  for (int k = 0; k < K; ++k) {
    const int idx = slab[tid * K + k];
    if (idx < 0) continue;
    const __half *f = feats + static_cast<int64_t>(idx) * c_in;
    uint4 raw = make_uint4(0, 0, 0, 0);
    // the row in one load where its size allows it (4 channels: 8 bytes, 8 channels: 16 bytes)
    if (c_in == 4) {
      const uint2 v = __ldg(reinterpret_cast<const uint2 *>(f));
      raw.x = v.x; raw.y = v.y;
    } else if (c_in == 8) {
      raw = __ldg(reinterpret_cast<const uint4 *>(f));
    } else {
      __half *xs = reinterpret_cast<__half *>(&raw);
#pragma unroll
      for (int ci = 0; ci < 8; ++ci)
        if (ci < c_in) xs[ci] = f[ci];
    }
    const float4 *wk = reinterpret_cast<const float4 *>(ws + static_cast<size_t>(k) * c_in * COUT);
#pragma unroll
    for (int ci = 0; ci < 8; ++ci) {
      if (ci >= c_in) break;
      const float x = __half2float(reinterpret_cast<const __half *>(&raw)[ci]);
#pragma unroll
      for (int c4 = 0; c4 < COUT / 4; ++c4) {
        const float4 wv = wk[ci * (COUT / 4) + c4];
        acc[4 * c4 + 0] = fmaf(x, wv.x, acc[4 * c4 + 0]);
        acc[4 * c4 + 1] = fmaf(x, wv.y, acc[4 * c4 + 1]);
        acc[4 * c4 + 2] = fmaf(x, wv.z, acc[4 * c4 + 2]);
        acc[4 * c4 + 3] = fmaf(x, wv.w, acc[4 * c4 + 3]);
      }
    }
  }
  const int64_t t = t0 + tid;
  // a grouped map names the output row of each of its rows; its padding rows carry -1
  const int64_t out_row = row_of != nullptr ? static_cast<int64_t>(row_of[t]) : (t < T ? t : -1);
  if (out_row < 0) return;
  __half *dst = out + out_row * COUT;
  const __half *res = ep.residual ? ep.residual + out_row * COUT : nullptr;
#pragma unroll
  for (int c8 = 0; c8 < COUT / 8; ++c8) {
    uint4 pack, rv = make_uint4(0, 0, 0, 0);
    if (res) rv = *reinterpret_cast<const uint4 *>(res + 8 * c8);
    const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
    uint32_t *pw = reinterpret_cast<uint32_t *>(&pack);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int co = 8 * c8 + 2 * e;
      float v0 = epilogue_apply(acc[co], co, ep), v1 = epilogue_apply(acc[co + 1], co + 1, ep);
      if (res) { v0 += __low2float(rh[e]); v1 += __high2float(rh[e]); }
      if (ep.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
      const __half2 hv = __floats2half2_rn(v0, v1);
      pw[e] = *reinterpret_cast<const uint32_t *>(&hv);
    }
    *reinterpret_cast<uint4 *>(dst + 8 * c8) = pack;
  }
}

// one warp per pair; grid.y = list rows (doubled when mirrored)
__global__ void __launch_bounds__(128) conv_ws_simt_kernel(const __half *__restrict__ feats,
                                                            const __half *__restrict__ w,
                                                            const int32_t *__restrict__ in_idx,
                                                            const int32_t *__restrict__ out_idx,
                                                            const int32_t *__restrict__ naddrs, int rows, int K,
                                                            int c_in, int c_out, float *__restrict__ accum) {
  const int lane = threadIdx.x & 31;
  int k = blockIdx.y;
  const bool mirrored = k >= rows;
  if (mirrored) k -= rows;
  const int begin = naddrs[k], end = naddrs[k + 1];
  const int wk_row = mirrored ? (K - 1 - k) : k;
  for (int p = begin + blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < end; p += gridDim.x * (blockDim.x >> 5)) {
    const int i = mirrored ? out_idx[p] : in_idx[p];
    const int o = mirrored ? in_idx[p] : out_idx[p];
    const __half *f = feats + static_cast<int64_t>(i) * c_in;
    for (int co = lane; co < c_out; co += 32) {
      const __half *wk = w + static_cast<int64_t>(wk_row) * c_in * c_out + co;
      float acc = 0.f;
      for (int ci = 0; ci < c_in; ++ci) acc = fmaf(__half2float(f[ci]), __half2float(wk[static_cast<int64_t>(ci) * c_out]), acc);
      atomicAdd(accum + static_cast<int64_t>(o) * c_out + co, acc);
    }
  }
}

__global__ void __launch_bounds__(256) finalize_kernel(const float *__restrict__ accum, Epilogue ep, int64_t n,
                                                        int c_out, __half *__restrict__ out) {
  int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int c = static_cast<int>(i % c_out);
  float v = epilogue_apply(accum[i], c, ep);
  if (ep.residual) v += __half2float(ep.residual[i]);
  if (ep.relu) v = fmaxf(v, 0.f);
  out[i] = __float2half_rn(v);
}

// ---- host side ------------------------------------------------------------------------------------

static bool tc_eligible(int K, int c_in, int c_out) {
  return K >= 1 && c_in >= 8 && c_in % 8 == 0 && c_out >= 16 && c_out % 16 == 0 && c_out <= 256;
}

static Epilogue make_epilogue(const spira_b200_epilogue *e) {
  Epilogue ep{nullptr, nullptr, nullptr, nullptr, 0};
  if (e) {
    ep.bias = static_cast<const __half *>(e->bias);
    ep.scale = e->scale;
    ep.shift = e->shift;
    ep.residual = static_cast<const __half *>(e->residual);
    ep.relu = e->relu;
  }
  return ep;
}

static int round16(int x) { return (x + 15) / 16 * 16; }

// ---- run-time options -----------------------------------------------------------------------------
static int g_gather_tma = 0;      // 1: producers use TMA gather4, 0: cp.async
static int g_identity_tma = 1;    // 1: 1x1x1 layers whose channel counts allow it run on the dense TMA kernel
static int g_wait_limit_us = kDefaultWaitLimitUs;   // limit of every wait inside the tensor-core kernels
static int g_ws_barrier_skew_once = 0;              // added to the grid-barrier target of the NEXT fused launch only

static unsigned long long wait_limit_ns() { return static_cast<unsigned long long>(g_wait_limit_us) * 1000ull; }

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

// 2-D map over feats[num_rows][c_in] (fp16), box = 64 channels x 1 row, 128-byte swizzle, zero fill out of bounds.
static int make_feats_tensor_map(CUtensorMap *map, const void *feats, int64_t num_rows, int c_in) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(SPIRA_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(c_in), static_cast<cuuint64_t>(num_rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(c_in) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kChunk), 1};   // gather4 takes ONE row per index (a 4-row box is rejected by the hardware)
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(feats), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SPIRA_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return SPIRA_B200_OK;
}

// Fused weight-stationary launches of one device share the arrival counter of their grid barrier (and, by contract,
// the caller's zero scratch), so they must be ordered on ONE stream.  The first fused launch binds the device to its
// stream; a launch on another stream is refused instead of being left to run into the wait limit.
// spira_b200_ws_barrier_resync() releases the binding.
static int g_ws_cooperative_launch = 0;      // 1: the fused weight-stationary call uses cudaLaunchCooperativeKernel
static unsigned g_arrivals_host[64] = {0};   // per device: sum of the grid sizes of all fused launches so far
static cudaStream_t g_fused_stream[64] = {nullptr};
static bool g_fused_bound[64] = {false};

template <bool kWS>
static int launch_conv_tc(ConvParams &P, bool tma, size_t smem, int64_t num_sources, cudaStream_t st) {
  alignas(64) CUtensorMap tmap;
  std::memset(&tmap, 0, sizeof(tmap));
  int grid = (P.n_tiles >= 0 && P.n_tiles < sm_count()) ? P.n_tiles : sm_count();
  if (kWS && P.fused) {
    // the CTAs wait for one another: cooperative launch (all of them resident), at least one CTA to convert the scratch
    if (grid <= 0) grid = 1;
    int dev = 0;
    SB_CHECK_CUDA(cudaGetDevice(&dev));
    SB_CHECK_ARG(dev >= 0 && dev < 64, "conv_ws_fused: device %d out of range", dev);
    SB_CHECK_ARG(!g_fused_bound[dev] || g_fused_stream[dev] == st,
                 "conv_ws_fused: device %d runs its fused weight-stationary calls on another stream; they share one grid-barrier "
                 "counter and must stay on one stream (spira_b200_ws_barrier_resync() rebinds, spira_b200_conv_ws has no such limit)",
                 dev);
    SB_CHECK_CUDA(cudaFuncSetAttribute(conv_tc_kernel<kWS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    g_fused_bound[dev] = true;
    g_fused_stream[dev] = st;
    g_arrivals_host[dev] += static_cast<unsigned>(grid);
    P.barrier_target = g_arrivals_host[dev] + static_cast<unsigned>(g_ws_barrier_skew_once);
    g_ws_barrier_skew_once = 0;
    // The grid barrier needs every CTA resident.  A cooperative launch guarantees that but is never overlapped with its
    // predecessor; an ordinary (dependent) launch of at most one CTA per SM gets there as well -- its CTAs only ever wait
    // for CTAs of the same grid, and those become resident as soon as earlier kernels, which wait for nobody, drain --
    // and saves 1.3-2.1 us per layer (measured).  The bounded wait of the barrier covers what an ordinary launch cannot
    // promise (another barrier kernel of another stream holding SMs): "ws_cooperative_launch" = 1 restores the guarantee.
    int per_sm = 0;
    if (!g_ws_cooperative_launch) {
      static size_t fits[8] = {0};      // shared-memory sizes already known to leave room for one CTA per SM
      static int n_fits = 0;
      for (int i = 0; i < n_fits; ++i)
        if (fits[i] == smem) per_sm = 1;
      if (per_sm == 0) {
        SB_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, conv_tc_kernel<kWS, false>, kConvThreads, smem));
        if (per_sm >= 1 && n_fits < 8) fits[n_fits++] = smem;
      }
    }
    cudaError_t e;
    if (!g_ws_cooperative_launch && per_sm >= 1 && grid <= sm_count()) {
      e = launch_dependent(conv_tc_kernel<kWS, false>, dim3(grid), dim3(kConvThreads), smem, st, P, tmap);
    } else {
      void *args[] = {&P, &tmap};
      e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&conv_tc_kernel<kWS, false>), dim3(grid), dim3(kConvThreads), args,
                                      smem, st);
    }
    if (e != cudaSuccess) {
      g_arrivals_host[dev] -= static_cast<unsigned>(grid);      // nothing was launched: nobody will arrive
      return fail(SPIRA_B200_ERR_CUDA, "conv_ws_fused: launch failed: %s", cudaGetErrorString(e));
    }
    return SPIRA_B200_OK;
  }
  if (grid <= 0) return SPIRA_B200_OK;
  if (!kWS && P.split > 1) {
    // the CTAs of a tile wait for one another: cooperative launch, all of them resident
    grid = P.n_tiles * P.split;
    SB_CHECK_CUDA(cudaFuncSetAttribute(conv_tc_kernel<kWS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    void *args[] = {&P, &tmap};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&conv_tc_kernel<kWS, false>), dim3(grid),
                                                dim3(kConvThreads), args, smem, st);
    if (e != cudaSuccess) return fail(SPIRA_B200_ERR_CUDA, "conv_os_split: cooperative launch failed: %s", cudaGetErrorString(e));
    return SPIRA_B200_OK;
  }
  if (tma) {
    int rc = make_feats_tensor_map(&tmap, P.feats, num_sources, P.c_in);
    if (rc != SPIRA_B200_OK) return rc;
    SB_CHECK_CUDA(cudaFuncSetAttribute(conv_tc_kernel<kWS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SB_CHECK_CUDA(launch_dependent(conv_tc_kernel<kWS, true>, dim3(grid), dim3(kConvThreads), smem, st, P, tmap));
  } else {
    SB_CHECK_CUDA(cudaFuncSetAttribute(conv_tc_kernel<kWS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SB_CHECK_CUDA(launch_dependent(conv_tc_kernel<kWS, false>, dim3(grid), dim3(kConvThreads), smem, st, P, tmap));
  }
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

// Fills the shared-memory plan of ConvParams; returns the dynamic shared memory size or 0 if it does not fit.
constexpr int kEpilogueBytes = 256 * 16;
static size_t plan_smem(ConvParams &P, bool ws, bool resident = false) {
  P.b_bytes = P.c_out * 128;
  int acc = 32;
  while (acc < P.c_out) acc <<= 1;
  P.acc_stride = acc;
  P.tmem_cols = 2 * acc;
  int slab_one = ws ? (1 + kScatterRing) * kRows * 4 : kRows * P.K * 4;
  P.slab_bufs = (!ws && 2 * slab_one <= 32 * 1024) ? 2 : 1;
  int slab_bytes = ws ? slab_one : P.slab_bufs * slab_one;
  int n_words = ws ? 1 : (P.n_chunks + 31) / 32;
  // weight-stationary: the list offsets of all rows (naddrs, qnaddrs: rows + 1 entries each) are staged in shared memory
  const int rowtab_bytes = ws ? 2 * round16((P.rows + 1) * 4) : round16(P.K * 4);
  int tr_bytes = ws ? kEpilogueWarps * 32 * 36 * 4 : 0;
  const int ep_bytes = ws ? 0 : kEpilogueBytes;
  P.ws_epilogue_warps = kEpilogueWarps;
  if (ws) {
    // eight transposition tiles must not cost the pipeline its fourth stage
    const int fixed8 = slab_bytes + rowtab_bytes + round16(2 * n_words * 4) + round16(kMaxStages * 4) + tr_bytes + 8 * (2 * kMaxStages + 8) + 16;
    if ((kSmemBudget - fixed8) / (kABytes + P.b_bytes) < 4) {
      tr_bytes /= 2;
      P.ws_epilogue_warps = 4;
    }
  }
  int fixed = slab_bytes + rowtab_bytes + round16(2 * n_words * 4) + round16(kMaxStages * 4) + ep_bytes + tr_bytes + 8 * (2 * kMaxStages + 8) + 16;
  int per_stage = kABytes + P.b_bytes;
  if (resident) {           // all weight chunks stay, the stages hold feature rows only
    per_stage = kABytes;
    fixed += P.n_chunks * P.b_bytes;
    if (fixed >= kSmemBudget) return 0;
  }
  int stages = (kSmemBudget - fixed) / per_stage;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < (resident ? 4 : 2)) return 0;
  // producer teams: stage s is filled by team s % teams, so the stage count is a multiple of the team count
  if (stages == 7) stages = 6;
  if (stages == 5) stages = 4;
  P.teams = (stages % 4 == 0) ? 4 : (stages % 3 == 0) ? 3 : 2;
  P.stages = stages;
  P.off_b = stages * kABytes;
  P.off_slab = P.off_b + (resident ? P.n_chunks : stages) * P.b_bytes;
  P.off_flags = P.off_slab + slab_bytes;
  P.off_cm = P.off_flags + rowtab_bytes;
  P.off_meta = P.off_cm + round16(2 * n_words * 4);
  P.off_ep = P.off_meta + round16(kMaxStages * 4);
  P.off_tr = P.off_ep + ep_bytes;
  P.off_bar = P.off_tr + tr_bytes;
  return static_cast<size_t>(P.off_bar) + 8 * (2 * kMaxStages + 8) + 16 + 1024;
}

// Shared-memory plan of conv_os_n256_kernel; returns the dynamic shared memory size or 0 if it does not fit.
static size_t plan_smem_n256(ConvN2Params &P, int teams) {
  P.w_bytes = P.c_out * 128;
  P.w_stride = (P.w_bytes + 1023) / 1024 * 1024;
  const int slab_bytes = kN2Rows * P.K * 4;
  const int n_words = (P.n_chunks + 31) / 32;
  const int tr_bytes = kEpilogueWarps * 32 * 17 * 4;   // per epilogue warp: 32 channels x 16 targets in fp32, padded rows
  const int fixed = slab_bytes + tr_bytes + round16(2 * n_words * 4) + round16(kMaxStages * 4) + 8 * (2 * kMaxStages + 8) + 16;
  const int per_stage = P.w_stride + kN2FeatBytes;
  int stages = (kSmemBudget - fixed) / per_stage;
  if (stages > kMaxStages) stages = kMaxStages;
  stages -= stages % teams;           // stage s is filled by team s % teams
  if (stages < 4) return 0;
  P.stages = stages;
  P.off_feat = stages * P.w_stride;   // the weight stages come first: an M=128 descriptor may read past a short one
  P.off_slab = P.off_feat + stages * kN2FeatBytes;
  P.off_tr = P.off_slab + slab_bytes;
  P.off_cm = P.off_tr + tr_bytes;
  P.off_meta = P.off_cm + round16(2 * n_words * 4);
  P.off_bar = P.off_meta + round16(kMaxStages * 4);
  return static_cast<size_t>(P.off_bar) + 8 * (2 * kMaxStages + 8) + 16 + 1024;
}

static int g_os_n256 = 1;          // 1: layers with 64 < c_out <= 128 use the exchanged-operand kernel
static int g_os_n256_min_targets = 0; // layers with fewer targets use the 128-target tiles (finer load balance)

}  // namespace sb

using namespace sb;

extern "C" int spira_b200_tensor_core_eligible(int K, int c_in, int c_out) { return tc_eligible(K, c_in, c_out) ? 1 : 0; }

extern "C" int spira_b200_packed_weight_bytes(int K, int c_in, int c_out, int pack_mode, size_t *bytes) {
  SB_CHECK_ARG(bytes != nullptr, "packed_weight_bytes: null output");
  SB_CHECK_ARG(tc_eligible(K, c_in, c_out), "packed_weight_bytes: (K=%d, c_in=%d, c_out=%d) is not tensor-core eligible", K,
               c_in, c_out);
  int64_t chunks = pack_mode == SPIRA_B200_PACK_WS ? static_cast<int64_t>(K) * div_up(c_in, kChunk)
                                                   : div_up(static_cast<int64_t>(K) * c_in, kChunk);
  *bytes = static_cast<size_t>(chunks) * c_out * 128;
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_pack_weights(const void *weights, int K, int c_in, int c_out, int pack_mode, void *packed,
                                       void *stream) {
  SB_CHECK_ARG(weights && packed, "pack_weights: null pointer");
  SB_CHECK_ARG(tc_eligible(K, c_in, c_out), "pack_weights: (K=%d, c_in=%d, c_out=%d) is not tensor-core eligible", K, c_in,
               c_out);
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(packed) % 16 == 0, "pack_weights: packed image must be 16-byte aligned");
  const bool ws = pack_mode == SPIRA_B200_PACK_WS;
  int cpo = static_cast<int>(div_up(c_in, kChunk));
  int64_t chunks = ws ? static_cast<int64_t>(K) * cpo : div_up(static_cast<int64_t>(K) * c_in, kChunk);
  int64_t pieces = chunks * c_out * 8;
  pack_weights_kernel<<<static_cast<unsigned>(div_up(pieces, 256)), 256, 0, as_stream(stream)>>>(
      static_cast<const __half *>(weights), K, c_in, c_out, ws ? 1 : 0, cpo, pieces, static_cast<unsigned char *>(packed));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

// Does the 256-target kernel take this output-stationary layer?  (Its shared-memory plan must hold four stages.)
static bool os_n256_applies(int K, int c_in, int c_out, int64_t num_targets) {
  if (!(g_os_n256 && !g_gather_tma && c_out > 64 && c_out <= 128 && K <= 32 && num_targets >= g_os_n256_min_targets)) return false;
  ConvN2Params Q{};
  Q.K = K; Q.c_in = c_in; Q.c_out = c_out;
  Q.R = K * c_in;
  Q.n_chunks = static_cast<int>(div_up(Q.R, kChunk));
  return plan_smem_n256(Q, kProducers / kN2TeamThreads) != 0;
}

static bool stem_applies(int K, int c_in, int c_out) {
  const size_t stem_smem = static_cast<size_t>(K) * c_in * c_out * 4 + static_cast<size_t>(128) * K * 4;
  return c_in <= 8 && (c_out == 16 || c_out == 32 || c_out == 64) && stem_smem <= 96 * 1024;
}

extern "C" int spira_b200_conv_kernel_choice(int weight_stationary, int K, int c_in, int c_out, int64_t num_targets) {
  if (K < 1 || c_in < 1 || c_out < 1 || num_targets < 0) return -1;
  const bool tc = tc_eligible(K, c_in, c_out);
  if (weight_stationary) return tc ? SPIRA_B200_KERNEL_TC_WS : SPIRA_B200_KERNEL_SIMT_WS;
  if (!tc) return stem_applies(K, c_in, c_out) ? SPIRA_B200_KERNEL_STEM_OS : SPIRA_B200_KERNEL_SIMT_OS;
  return os_n256_applies(K, c_in, c_out, num_targets) ? SPIRA_B200_KERNEL_N256_OS : SPIRA_B200_KERNEL_TC_OS;
}

// Split reduction of the output-stationary kernel: the head of the caller's scratch holds the per-tile counters (arrivals,
// leavers; zero whenever no launch is in flight), the fp32 partial sums follow.
constexpr size_t kSplitCounterBytes = 1024;
constexpr int kSplitMaxTiles = static_cast<int>(kSplitCounterBytes / 8);

static int split_limit(int64_t num_targets, int K, int c_in, int c_out) {
  if (!tc_eligible(K, c_in, c_out) || num_targets <= 0) return 1;
  const int64_t n_tiles = align128(num_targets) / kRows;
  if (n_tiles > kSplitMaxTiles) return 1;
  const int64_t chunks = div_up(static_cast<int64_t>(K) * c_in, kChunk);
  for (int s = 8; s >= 2; s >>= 1)
    if (n_tiles * s <= sm_count() && c_out % (8 * s) == 0 && chunks >= 4 * s) return s;
  return 1;
}

extern "C" int spira_b200_conv_os_split_plan(int64_t num_targets, int K, int c_in, int c_out, int *max_splits,
                                             size_t *scratch_bytes) {
  SB_CHECK_ARG(max_splits && scratch_bytes, "conv_os_split_plan: null output");
  SB_CHECK_ARG(K >= 1 && c_in >= 1 && c_out >= 1 && num_targets >= 0, "conv_os_split_plan: K=%d c_in=%d c_out=%d", K, c_in, c_out);
  const int s = split_limit(num_targets, K, c_in, c_out);
  *max_splits = s;
  *scratch_bytes = s > 1 ? kSplitCounterBytes + static_cast<size_t>(align128(num_targets)) * s * c_out * sizeof(float) : 0;
  return SPIRA_B200_OK;
}

static int conv_os_impl(const void *feats, const void *weights, const void *packed, const spira_b200_epilogue *epilogue,
                        const int32_t *map_os, const int32_t *row_of, const uint32_t *tile_masks, int64_t num_sources,
                        int64_t num_targets, int K, int c_in, int c_out, void *out, int32_t *status, void *stream,
                        int splits = 1, void *split_scratch = nullptr, size_t split_scratch_bytes = 0,
                        const void *feats_b = nullptr, int c_in_a = 0, bool identity = false) {
  SB_CHECK_ARG(num_sources >= 0 && num_targets >= 0 && num_targets < (int64_t(1) << 31) - 128 &&
                   num_sources < (int64_t(1) << 31),
               "conv_os: sizes out of range");
  SB_CHECK_ARG(K >= 1 && c_in >= 1 && c_out >= 1, "conv_os: K=%d c_in=%d c_out=%d", K, c_in, c_out);
  if (num_targets == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG((map_os || identity) && out && (feats || num_sources == 0), "conv_os: null pointer");
  Epilogue ep = make_epilogue(epilogue);
  SB_CHECK_ARG((ep.scale == nullptr) == (ep.shift == nullptr), "conv_os: scale and shift must be given together");
  const bool two = feats_b != nullptr && c_in_a > 0 && c_in_a < c_in;
  if (two)
    SB_CHECK_ARG(packed != nullptr && !g_gather_tma && c_in_a % 8 == 0 && reinterpret_cast<uintptr_t>(feats_b) % 16 == 0,
                 "conv_os: two sources need a packed weight image, the cp.async producers, c_in_a %% 8 == 0 (got %d) and a "
                 "16-byte aligned second tensor", c_in_a);
  if (identity)
    SB_CHECK_ARG(packed != nullptr && !g_gather_tma && K == 1 && map_os == nullptr && row_of == nullptr && splits <= 1 &&
                     num_sources >= num_targets,
                 "conv_os: the identity map is for 1x1x1 layers with a packed weight image (K=%d)", K);
  if (identity && g_identity_tma && dense_applies(num_targets, c_in, two ? c_in_a : c_in, c_out, feats, two ? feats_b : nullptr, packed))
    return dense_run(feats, two ? feats_b : nullptr, two ? c_in_a : c_in, packed, epilogue, num_targets, c_in, c_out, out, status,
                     wait_limit_ns(), as_stream(stream));
  if (packed == nullptr) {
    SB_CHECK_ARG(weights != nullptr, "conv_os: neither weights nor a packed image given");
    const size_t stem_smem = static_cast<size_t>(K) * c_in * c_out * 4 + static_cast<size_t>(128) * K * 4;
    const bool aligned16 = reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(map_os) % 16 == 0 &&
                           (ep.residual == nullptr || reinterpret_cast<uintptr_t>(ep.residual) % 16 == 0);
    if (c_in <= 8 && (c_out == 16 || c_out == 32 || c_out == 64) && stem_smem <= 96 * 1024 && aligned16) {
      const unsigned grid = static_cast<unsigned>(div_up(num_targets, 128));
      auto launch = [&](auto kernel) -> int {
        SB_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(stem_smem)));
        SB_CHECK_CUDA(launch_dependent(kernel, dim3(grid), dim3(128), stem_smem, as_stream(stream), static_cast<const __half *>(feats),
                                       static_cast<const __half *>(weights), ep, map_os, row_of, num_targets, K, c_in,
                                       static_cast<__half *>(out)));
        return SPIRA_B200_OK;
      };
      if (c_out == 16) return launch(conv_os_stem_kernel<16>);
      if (c_out == 32) return launch(conv_os_stem_kernel<32>);
      return launch(conv_os_stem_kernel<64>);
    }
    SB_CHECK_ARG(row_of == nullptr, "conv_os_grouped: without a packed weight image only c_in <= 8 with c_out 16, 32 or 64 is covered");
    conv_os_simt_kernel<<<static_cast<unsigned>(div_up(num_targets, 4)), 128, 0, as_stream(stream)>>>(
        static_cast<const __half *>(feats), static_cast<const __half *>(weights), ep, map_os, num_targets, K, c_in, c_out,
        static_cast<__half *>(out));
    SB_CHECK_LAUNCH();
    return SPIRA_B200_OK;
  }
  SB_CHECK_ARG(tc_eligible(K, c_in, c_out), "conv_os: (K=%d, c_in=%d, c_out=%d) is not tensor-core eligible", K, c_in, c_out);
  SB_CHECK_ARG(reinterpret_cast<uintptr_t>(feats) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(map_os) % 16 == 0 &&
                   (ep.residual == nullptr || reinterpret_cast<uintptr_t>(ep.residual) % 16 == 0),
               "conv_os: feats, packed, out, map and residual must be 16-byte aligned");
  const int c_a = two ? c_in_a : c_in;
  if (splits > 1) {
    SB_CHECK_ARG(packed != nullptr, "conv_os_split: needs a packed weight image");
    SB_CHECK_ARG((splits == 2 || splits == 4 || splits == 8) && splits <= split_limit(num_targets, K, c_in, c_out),
                 "conv_os_split: %d splits not possible for %lld targets, K=%d, c_in=%d, c_out=%d (see spira_b200_conv_os_split_plan)",
                 splits, static_cast<long long>(num_targets), K, c_in, c_out);
    SB_CHECK_ARG(split_scratch && reinterpret_cast<uintptr_t>(split_scratch) % 16 == 0 &&
                     split_scratch_bytes >= kSplitCounterBytes + static_cast<size_t>(align128(num_targets)) * splits * c_out * sizeof(float),
                 "conv_os_split: scratch missing, misaligned or too small");
  }
  // On grouped maps both kernels run at the speed of the row gathers; the 256-target tiles then only pay off for the
  // wider layers (measured: 32 channels 20 % slower, 64 equal, 96 5 % faster than 128-target tiles).
  if (splits <= 1 && !identity && os_n256_applies(K, c_in, c_out, num_targets)) {
    ConvN2Params Q{};
    Q.feats = static_cast<const __half *>(feats);
    Q.feats_b = static_cast<const __half *>(feats_b);
    Q.c_a = c_a;
    Q.packed = static_cast<const unsigned char *>(packed);
    Q.out = static_cast<__half *>(out);
    Q.ep = ep;
    Q.status = status;
    Q.map = map_os;
    Q.row_of = row_of;
    Q.tile_masks = tile_masks;
    Q.T = static_cast<int>(num_targets);
    Q.T_al = static_cast<int>(align128(num_targets));
    Q.n_tiles = static_cast<int>(div_up(num_targets, kN2Rows));
    Q.K = K; Q.c_in = c_in; Q.c_out = c_out;
    Q.R = K * c_in;
    Q.n_chunks = static_cast<int>(div_up(Q.R, kChunk));
    Q.wait_ns = wait_limit_ns();
    size_t smem2 = plan_smem_n256(Q, kProducers / kN2TeamThreads);
    if (smem2 != 0) {
      const int grid = Q.n_tiles < sm_count() ? Q.n_tiles : sm_count();
      SB_CHECK_CUDA(cudaFuncSetAttribute(conv_os_n256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem2)));
      SB_CHECK_CUDA(launch_dependent(conv_os_n256_kernel, dim3(grid), dim3(kConvThreads), smem2, as_stream(stream), Q));
      SB_CHECK_LAUNCH();
      return SPIRA_B200_OK;
    }
  }
  ConvParams P{};
  P.feats = static_cast<const __half *>(feats);
  P.feats_b = static_cast<const __half *>(feats_b);
  P.c_a = c_a;
  P.packed = static_cast<const unsigned char *>(packed);
  P.out = static_cast<__half *>(out);
  P.ep = ep;
  P.status = status;
  P.map = map_os;
  P.row_of = row_of;
  P.tile_masks = tile_masks;
  P.T = static_cast<int>(num_targets);
  P.n_tiles = static_cast<int>(align128(num_targets) / kRows);
  P.K = K; P.c_in = c_in; P.c_out = c_out;
  P.wait_ns = wait_limit_ns();
  const bool tma = g_gather_tma != 0 && num_sources > 0 && K <= 512 && splits <= 1;
  P.split = splits > 1 ? splits : 1;
  if (splits > 1) {
    P.split_counters = static_cast<unsigned *>(split_scratch);
    P.split_scratch = reinterpret_cast<float *>(static_cast<unsigned char *>(split_scratch) + kSplitCounterBytes);
  }
  P.R = K * c_in;
  // TMA gather: every offset owns ceil(c_in/64) chunks (PACK_WS image); cp.async: 64-wide chunks over the whole reduction
  P.n_chunks = tma ? static_cast<int>(div_up(c_in, kChunk)) : static_cast<int>(div_up(P.R, kChunk));
  size_t smem = 0;
  if (identity && P.n_tiles > sm_count()) {      // (with one tile per CTA the whole image would only delay the first MMA)
    smem = plan_smem(P, false, true);
    P.resident = smem != 0 ? 1 : 0;
  }
  if (smem == 0) smem = plan_smem(P, false);
  if (smem == 0) return fail(SPIRA_B200_ERR_UNSUPPORTED, "conv_os: K=%d c_out=%d does not fit the shared-memory plan", K, c_out);
  return launch_conv_tc<false>(P, tma, smem, num_sources, as_stream(stream));
}

extern "C" int spira_b200_conv_os(const void *feats, const void *weights, const void *packed,
                                  const spira_b200_epilogue *epilogue, const int32_t *map_os, int64_t num_sources,
                                  int64_t num_targets, int K, int c_in, int c_out, void *out, int32_t *status,
                                  void *stream) {
  return conv_os_impl(feats, weights, packed, epilogue, map_os, nullptr, nullptr, num_sources, num_targets, K, c_in, c_out,
                      out, status, stream);
}

extern "C" int spira_b200_conv_os_grouped(const void *feats, const void *weights, const void *packed,
                                          const spira_b200_epilogue *epilogue, const int32_t *grouped_map,
                                          const int32_t *row_of, const uint32_t *tile_masks, int64_t num_sources,
                                          int64_t num_targets, int K, int c_in, int c_out, void *out, int32_t *status,
                                          void *stream) {
  SB_CHECK_ARG(num_targets == 0 || (row_of && tile_masks && (packed || weights)), "conv_os_grouped: null pointer");
  SB_CHECK_ARG(K <= 32, "conv_os_grouped: K=%d, grouped maps have at most 32 offsets", K);
  return conv_os_impl(feats, weights, packed, epilogue, grouped_map, row_of, tile_masks, num_sources, num_targets, K, c_in,
                      c_out, out, status, stream);
}

extern "C" int spira_b200_conv_os_split(const void *feats, const void *packed, const spira_b200_epilogue *epilogue,
                                        const int32_t *map_os, const int32_t *row_of, const uint32_t *tile_masks,
                                        int64_t num_sources, int64_t num_targets, int K, int c_in, int c_out, int splits,
                                        void *scratch, size_t scratch_bytes, void *out, int32_t *status, void *stream) {
  SB_CHECK_ARG((row_of == nullptr) == (tile_masks == nullptr), "conv_os_split: row_of and tile_masks come together");
  SB_CHECK_ARG(row_of == nullptr || K <= 32, "conv_os_split: K=%d, grouped maps have at most 32 offsets", K);
  SB_CHECK_ARG(splits >= 1, "conv_os_split: splits=%d", splits);
  return conv_os_impl(feats, nullptr, packed, epilogue, map_os, row_of, tile_masks, num_sources, num_targets, K, c_in, c_out,
                      out, status, stream, splits, scratch, scratch_bytes);
}

static int conv_ws_impl(const void *feats, const void *weights, const void *packed, const spira_b200_epilogue *epilogue,
                        const int32_t *in_idx, const int32_t *out_idx, const int32_t *naddrs, const int32_t *qnaddrs, int rows,
                        int64_t num_tiles128, int mirror, int swap, int64_t num_sources, int64_t num_targets, int K, int c_in,
                        int c_out, float *accum, void *out, int32_t *status, void *stream, bool fused,
                        const void *feats_b = nullptr, int c_in_a = 0) {
  SB_CHECK_ARG(num_sources >= 0 && num_targets >= 0 && num_targets < (int64_t(1) << 31) && num_sources < (int64_t(1) << 31),
               "conv_ws: sizes out of range");
  SB_CHECK_ARG(K >= 1 && c_in >= 1 && c_out >= 1 && rows >= 1 && rows <= K, "conv_ws: K=%d c_in=%d c_out=%d rows=%d", K, c_in,
               c_out, rows);
  SB_CHECK_ARG(!mirror || (rows == (K + 1) / 2 && !swap), "conv_ws: mirror needs rows == (K+1)/2 and no swap");
  SB_CHECK_ARG(num_tiles128 >= -1 && num_tiles128 < (int64_t(1) << 30), "conv_ws: num_tiles128 out of range");
  if (num_targets == 0) return SPIRA_B200_OK;
  SB_CHECK_ARG(accum && out && naddrs, "conv_ws: null pointer");
  Epilogue ep = make_epilogue(epilogue);
  SB_CHECK_ARG((ep.scale == nullptr) == (ep.shift == nullptr), "conv_ws: scale and shift must be given together");
  cudaStream_t st = as_stream(stream);
  const int64_t n_out = num_targets * c_out;
  if (!fused) SB_CHECK_CUDA(cudaMemsetAsync(accum, 0, sizeof(float) * n_out, st));
  const int32_t *gi = swap ? out_idx : in_idx;
  const int32_t *go = swap ? in_idx : out_idx;
  const bool two = feats_b != nullptr && c_in_a > 0 && c_in_a < c_in;
  if (two)
    SB_CHECK_ARG(packed != nullptr && !g_gather_tma && c_in_a % 8 == 0 && reinterpret_cast<uintptr_t>(feats_b) % 16 == 0,
                 "conv_ws: two sources need a packed weight image, the cp.async producers, c_in_a %% 8 == 0 (got %d) and a "
                 "16-byte aligned second tensor", c_in_a);
  if (fused) {
    SB_CHECK_ARG(packed != nullptr && tc_eligible(K, c_in, c_out) && !g_gather_tma,
                 "conv_ws_fused: needs a tensor-core eligible layer with its packed weights and the cp.async producers");
    SB_CHECK_ARG(reinterpret_cast<uintptr_t>(out) % 16 == 0 && (!epilogue || reinterpret_cast<uintptr_t>(epilogue->residual) % 8 == 0),
                 "conv_ws_fused: out must be 16-byte and residual 8-byte aligned");
  }
  if (num_tiles128 != 0 || fused) {
    SB_CHECK_ARG((num_tiles128 == 0 || (gi && go)) && (feats || num_sources == 0), "conv_ws: null pointer");
    if (packed == nullptr) {
      SB_CHECK_ARG(weights != nullptr, "conv_ws: neither weights nor a packed image given");
      dim3 grid(static_cast<unsigned>(sm_count() * 2), static_cast<unsigned>(mirror ? K : rows));
      conv_ws_simt_kernel<<<grid, 128, 0, st>>>(static_cast<const __half *>(feats), static_cast<const __half *>(weights), gi,
                                                go, naddrs, rows, K, c_in, c_out, accum);
      SB_CHECK_LAUNCH();
    } else {
      SB_CHECK_ARG(tc_eligible(K, c_in, c_out), "conv_ws: (K=%d, c_in=%d, c_out=%d) is not tensor-core eligible", K, c_in, c_out);
      SB_CHECK_ARG(qnaddrs != nullptr, "conv_ws: null qnaddrs");
      SB_CHECK_ARG(reinterpret_cast<uintptr_t>(feats) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(accum) % 16 == 0,
                   "conv_ws: feats, packed and accum must be 16-byte aligned");
      ConvParams P{};
      P.feats = static_cast<const __half *>(feats);
      P.feats_b = static_cast<const __half *>(feats_b);
      P.c_a = two ? c_in_a : c_in;
      P.packed = static_cast<const unsigned char *>(packed);
      P.accum = accum;
      P.out = static_cast<__half *>(out);
      P.ep = ep;
      P.fused = fused ? 1 : 0;
      P.status = status;
      P.wait_ns = wait_limit_ns();
      P.in_idx = gi; P.out_idx = go; P.naddrs = naddrs; P.qnaddrs = qnaddrs;
      P.rows = rows; P.mirror = mirror;
      // the centre row of an odd kernel volume (last of the half list) is its own mirror image: its tiles are not repeated
      P.centre_tiles = (K % 2 == 1) ? static_cast<int>(div_up(num_targets, kRows)) : 0;
      if (num_tiles128 < 0) {
        P.n_tiles_plain = -1;      // the kernel reads qnaddrs[rows] itself
        P.n_tiles = -1;
      } else if (num_tiles128 == 0) {
        P.n_tiles_plain = 0;       // no pair at all (fused call: the scratch is still converted)
        P.n_tiles = 0;
      } else {
        P.n_tiles_plain = static_cast<int>(num_tiles128);
        P.n_tiles = static_cast<int>(mirror ? 2 * num_tiles128 - P.centre_tiles : num_tiles128);
      }
      P.T = static_cast<int>(num_targets);
      P.K = K; P.c_in = c_in; P.c_out = c_out;
      P.R = c_in;
      P.n_chunks = static_cast<int>(div_up(c_in, kChunk));
      size_t smem = plan_smem(P, true);
      if (smem == 0) return fail(SPIRA_B200_ERR_UNSUPPORTED, "conv_ws: c_out=%d does not fit the shared-memory plan", c_out);
      int rc = launch_conv_tc<true>(P, g_gather_tma != 0 && num_sources > 0, smem, num_sources, st);
      if (rc != SPIRA_B200_OK) return rc;
    }
  }
  if (fused) return SPIRA_B200_OK;
  finalize_kernel<<<static_cast<unsigned>(div_up(n_out, 256)), 256, 0, st>>>(accum, ep, n_out, c_out, static_cast<__half *>(out));
  SB_CHECK_LAUNCH();
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_conv_ws(const void *feats, const void *weights, const void *packed,
                                  const spira_b200_epilogue *epilogue, const int32_t *in_idx, const int32_t *out_idx,
                                  const int32_t *naddrs, const int32_t *qnaddrs, int rows, int64_t num_tiles128,
                                  int mirror, int swap, int64_t num_sources, int64_t num_targets, int K, int c_in,
                                  int c_out, float *accum, void *out, int32_t *status, void *stream) {
  return conv_ws_impl(feats, weights, packed, epilogue, in_idx, out_idx, naddrs, qnaddrs, rows, num_tiles128, mirror, swap,
                      num_sources, num_targets, K, c_in, c_out, accum, out, status, stream, false);
}

extern "C" int spira_b200_conv_ws_fused(const void *feats, const void *packed, const spira_b200_epilogue *epilogue,
                                        const int32_t *in_idx, const int32_t *out_idx, const int32_t *naddrs,
                                        const int32_t *qnaddrs, int rows, int64_t num_tiles128, int mirror, int swap,
                                        int64_t num_sources, int64_t num_targets, int K, int c_in, int c_out,
                                        float *zeroed_accum, void *out, int32_t *status, void *stream) {
  return conv_ws_impl(feats, nullptr, packed, epilogue, in_idx, out_idx, naddrs, qnaddrs, rows, num_tiles128, mirror, swap,
                      num_sources, num_targets, K, c_in, c_out, zeroed_accum, out, status, stream, true);
}

int sb::conv_run(const spira_b200_conv_desc &d, int32_t *status, void *stream) {
  SB_CHECK_ARG(d.dataflow == 0 || d.dataflow == 1, "conv: dataflow %d (0: output-stationary, 1: weight-stationary)", d.dataflow);
  SB_CHECK_ARG(d.packed != nullptr || (d.weights != nullptr && d.dataflow == 0),
               "conv: a packed weight image, or plain weights for an output-stationary layer outside the tensor-core kernels");
  SB_CHECK_ARG(d.c_in_a >= 0 && d.c_in_a <= d.c_in, "conv: c_in_a=%d outside [0, c_in=%d]", d.c_in_a, d.c_in);
  const bool two = d.c_in_a > 0 && d.c_in_a < d.c_in;
  SB_CHECK_ARG(!two || d.feats_b != nullptr, "conv: c_in_a=%d of c_in=%d channels but no second tensor", d.c_in_a, d.c_in);
  if (d.dataflow == 0) {
    const bool identity = d.map_os == nullptr && d.K == 1;
    SB_CHECK_ARG((d.row_of == nullptr) == (d.tile_masks == nullptr), "conv: row_of and tile_masks come together");
    SB_CHECK_ARG(d.row_of == nullptr || d.K <= 32, "conv: K=%d, grouped maps have at most 32 offsets", d.K);
    return conv_os_impl(d.feats, d.packed ? nullptr : d.weights, d.packed, d.epilogue, d.map_os, d.row_of, d.tile_masks, d.num_sources, d.num_targets,
                        d.K, d.c_in, d.c_out, d.out, status, stream, d.splits > 1 ? d.splits : 1, d.split_scratch,
                        d.split_scratch_bytes, two ? d.feats_b : nullptr, d.c_in_a, identity);
  }
  return conv_ws_impl(d.feats, nullptr, d.packed, d.epilogue, d.in_idx, d.out_idx, d.naddrs, d.qnaddrs, d.rows, d.num_tiles128,
                      d.mirror, d.swap, d.num_sources, d.num_targets, d.K, d.c_in, d.c_out, d.zeroed_accum, d.out, status,
                      stream, true, two ? d.feats_b : nullptr, d.c_in_a);
}

extern "C" int spira_b200_conv(const spira_b200_conv_desc *desc, int32_t *status, void *stream) {
  SB_CHECK_ARG(desc != nullptr, "conv: null descriptor");
  return sb::conv_run(*desc, status, stream);
}

extern "C" int spira_b200_set_option(const char *name, int value) {
  SB_CHECK_ARG(name != nullptr, "set_option: null name");
  if (std::strcmp(name, "gather_tma") == 0) { g_gather_tma = value ? 1 : 0; return SPIRA_B200_OK; }
  if (std::strcmp(name, "os_n256") == 0) { g_os_n256 = value ? 1 : 0; return SPIRA_B200_OK; }
  if (std::strcmp(name, "identity_tma") == 0) { g_identity_tma = value ? 1 : 0; return SPIRA_B200_OK; }
  if (std::strcmp(name, "pdl") == 0) { set_pdl_enabled(value != 0); return SPIRA_B200_OK; }
  if (std::strcmp(name, "ws_cooperative_launch") == 0) { g_ws_cooperative_launch = value ? 1 : 0; return SPIRA_B200_OK; }
  if (std::strcmp(name, "os_n256_min_targets") == 0) { g_os_n256_min_targets = value < 0 ? 0 : value; return SPIRA_B200_OK; }
  if (std::strcmp(name, "wait_limit_us") == 0) {
    SB_CHECK_ARG(value >= 100 && value <= 60 * 1000 * 1000, "set_option: wait_limit_us must lie in [100, 60000000]");
    g_wait_limit_us = value;
    return SPIRA_B200_OK;
  }
  if (std::strcmp(name, "ws_barrier_skew_once") == 0) { g_ws_barrier_skew_once = value; return SPIRA_B200_OK; }
  return fail(SPIRA_B200_ERR_ARGUMENT, "set_option: unknown option '%s'", name);
}

extern "C" int spira_b200_ws_barrier_resync(void) {
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64, "ws_barrier_resync: device %d out of range", dev);
  SB_CHECK_CUDA(cudaDeviceSynchronize());
  unsigned seen = 0;
  SB_CHECK_CUDA(cudaMemcpyFromSymbol(&seen, g_grid_arrivals, sizeof(seen)));
  g_arrivals_host[dev] = seen;
  g_fused_bound[dev] = false;
  g_fused_stream[dev] = nullptr;
  return SPIRA_B200_OK;
}

extern "C" int spira_b200_get_option(const char *name) {
  if (name == nullptr) return -1;
  if (std::strcmp(name, "gather_tma") == 0) return g_gather_tma;
  if (std::strcmp(name, "os_n256") == 0) return g_os_n256;
  if (std::strcmp(name, "identity_tma") == 0) return g_identity_tma;
  if (std::strcmp(name, "pdl") == 0) return pdl_enabled() ? 1 : 0;
  if (std::strcmp(name, "ws_cooperative_launch") == 0) return g_ws_cooperative_launch;
  if (std::strcmp(name, "wait_limit_us") == 0) return g_wait_limit_us;
  if (std::strcmp(name, "ws_barrier_skew_once") == 0) return g_ws_barrier_skew_once;
  if (std::strcmp(name, "os_n256_min_targets") == 0) return g_os_n256_min_targets;
  if (std::strcmp(name, "os_pack_mode") == 0) return g_gather_tma ? SPIRA_B200_PACK_WS : SPIRA_B200_PACK_OS;
  return -1;
}


// ---- weight-stationary convolution without any caller-provided scratch ------------------------------------------
// Scratch for the fp32 accumulation lives in this file-scope device array.  Every GPU that loads the library keeps
// its own copy (16 MiB) until the process exits.  In host code the array's name is only a handle: the device address
// is obtained once per device with cudaGetSymbolAddress while that device is current, and that pointer is what the
// kernels receive.
static __device__ __align__(256) float g_static_accum[SPIRA_B200_STATIC_SCRATCH_FLOATS];
static float *g_static_accum_ptr[64] = {nullptr};

extern "C" int spira_b200_conv_ws_static(const void *feats, const void *weights, const void *packed,
                                         const spira_b200_epilogue *epilogue, const int32_t *in_idx,
                                         const int32_t *out_idx, const int32_t *naddrs, const int32_t *qnaddrs, int rows,
                                         int64_t num_tiles128, int mirror, int swap, int64_t num_sources,
                                         int64_t num_targets, int K, int c_in, int c_out, void *out, int32_t *status,
                                         void *stream) {
  SB_CHECK_ARG(num_targets >= 0 && c_out >= 1, "conv_ws_static: bad sizes");
  SB_CHECK_ARG(num_targets * static_cast<int64_t>(c_out) <= static_cast<int64_t>(SPIRA_B200_STATIC_SCRATCH_FLOATS),
               "conv_ws_static: num_targets * c_out = %lld exceeds the built-in scratch of %lld floats; use spira_b200_conv_ws "
               "with caller-provided scratch",
               static_cast<long long>(num_targets * static_cast<int64_t>(c_out)),
               static_cast<long long>(SPIRA_B200_STATIC_SCRATCH_FLOATS));
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64, "conv_ws_static: device index %d out of range", dev);
  if (g_static_accum_ptr[dev] == nullptr) {
    // first call on this device: resolve the device address of the array (do this before any stream capture)
    float *p = nullptr;
    SB_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_static_accum));
    g_static_accum_ptr[dev] = p;
  }
  return spira_b200_conv_ws(feats, weights, packed, epilogue, in_idx, out_idx, naddrs, qnaddrs, rows, num_tiles128, mirror,
                            swap, num_sources, num_targets, K, c_in, c_out, g_static_accum_ptr[dev], out, status, stream);
}


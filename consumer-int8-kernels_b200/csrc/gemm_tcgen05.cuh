// Persistent, warp-specialised INT8 GEMM for sm_100a:  acc[m,n] = sum_k a[m,k] * w[n,k]  (INT32),
// out = bf16((float(acc) * sa[m]) * float(sw[n])).
//
//   warp 0      TMA producer: 128-byte-swizzled K-major tiles of A [M,K] and W [N,K] into a
//               shared-memory ring (one elected lane)
//   warp 1      tcgen05.mma kind::i8 issuer (one elected lane), accumulators in TMEM,
//               two 256-column accumulator buffers so a tile's epilogue overlaps the next
//               tile's main loop; also owns the TMEM allocation
//   warps 2..   epilogue: tcgen05.ld -> FP32 row scale -> FP32 channel scale -> BF16, staged
//               through a small swizzled shared-memory buffer and written with TMA tile stores
//               (full 128-byte lines; the same tile can be stored to several destinations, which
//               is how the N-sharded form writes its column block into every peer GPU's gathered
//               output while the main loop keeps running). Outputs whose row pitch is not a
//               multiple of 16 bytes take a direct-store path instead.
//
// kCtas == 1: one CTA per 128x256 output tile.
// kCtas == 2: a two-CTA cluster shares a 256x256 tile; each CTA stages its own 128 rows of A
//             and its own 128 rows of W (each CTA issues its own plain TMA loads) and the pair
//             leader issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory.
// Modes:
//   kModeFused      signed INT8 weights, BF16 output only (fused_channel_mm)
//   kModeWorkspace  as fused, and the INT32 accumulators are also written to a caller buffer
//                   (cutlass_channel_mm)
//   kModeBiased     UINT8 weights holding code+128 (channel_mm): the weight tile carries 248
//                   channels plus 8 rows of ones (one swizzle atom), so accumulator column 248 is
//                   sum_k a[m,k] and the signed product is acc - 128 * that sum, still exact
//                   INT32. In a CTA pair the second CTA holds the ones rows behind its 120
//                   channels; the first one loads 128 channels
//   kModeGrouped    K is G groups of 4096 with one activation scale per (group,row): each
//                   group's INT32 accumulator is converted, scaled and added in FP32 in
//                   ascending group order (separate multiply and add), then the channel
//                   scale is applied (grouped_channel_mm)
//   kModeSwiGLU     the gate/up projection with the SwiGLU fused into the epilogue: the weight rows
//                   are interleaved in blocks of 128 (tile t holds gate channels [128t, 128t+128) in
//                   its first 128 rows and the matching up channels in the other 128), so a tile's
//                   accumulator has a gate half and an up half; the epilogue rounds both to BF16
//                   exactly as kModeFused would have written them, and stores
//                   bf16(silu(gate) * up) [M, N/2] — bit-identical to fused_channel_mm followed
//                   by silu_mul, without the [M, N] round trip through HBM
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include "quantize.cuh"
#include "sm100_ptx.cuh"

namespace ci8 {

enum GemmMode { kModeFused = 0, kModeWorkspace = 1, kModeBiased = 2, kModeGrouped = 3, kModeSwiGLU = 4 };

constexpr int kMaxOutputs = 8;   // destinations of one output tile (this GPU + up to 7 peers)

struct GemmParams {
  const float* sa;            // [M] (grouped: [G,M])
  const __nv_bfloat16* sw;    // [N]
  __nv_bfloat16* out;         // [M,N] (direct-store path)
  int32_t* workspace;         // [M,N] or nullptr
  int m, n, k;                // k = K per group
  int groups;                 // 1 unless grouped
  int tiles_m, tiles_n;
  int group_m;                // row tiles per raster group (L2 reuse of the A rows)
  int num_outputs;            // TMA-store destinations in OutputMaps; 0 selects direct stores
  int tile_n;                 // output channels per tile: 256, or narrower (a multiple of 32) when that
                              // packs the tiles into fewer, fuller waves; 248 for the biased form
  int stage_tx;               // bytes one CTA's TMA loads deliver per stage (A box + W box)
  int stage_tx_slice;         // the same for a column slice (A box + the narrower W box)
  int full_tiles;             // work items [0, full_tiles) are whole tiles (the complete waves)
  int split;                  // each tile of the last, partial wave is cut into `split` column slices
  int total_items;            // full_tiles + (tiles - full_tiles) * split
  int out_n;                  // columns of the output matrix: n, or n / 2 for kModeSwiGLU
  int wide_tiles;             // mixed widths: the first wide_tiles channel tiles of every row stripe are
                              // tile_n + 32 columns wide, the others tile_n (0: all tiles are tile_n wide)
  // Grouped form with a caller workspace: every tile of the last, partial wave is cut ALONG THE GROUPS
  // into `groups` pieces that run on as many CTA pairs at once (piece_items = leftover tiles x groups
  // work items behind the whole tiles, drawn from a counter by the pairs that finish their whole tiles first). A piece writes its group's FP32 terms fmul(float(acc_g), sa_g)
  // to `terms`; when all pieces of a tile have arrived (piece_sync) each of them adds the terms of its
  // share of the tile in ascending group order (the same fadd chain as one CTA would run) and stores it.
  int piece_items;
  float* terms;               // [leftover tile][group][256 rows][256 columns]
  unsigned* piece_sync;       // [leftover tile][2]: pieces' warps arrived / departed, and word kPieceFetchWord:
                              // pieces drawn so far; all zero before and after a launch
};

// Word of the pieces' header (piece_sync) that counts the draws of a launch; the words before it are the
// arrival and departure counters of the leftover tiles (two each, at most 37 tiles on 74 workers).
constexpr int kPieceFetchWord = 192;

// Gathering form with the in-kernel rendezvous: after its first tile a worker does not walk the tiles with a
// fixed stride but draws the next one from a counter (state[2]). The CTAs of a GPU do not get equal shares of a
// saturated NVLink, and their tile stores are what paces them: with a fixed assignment the slowest CTA issued
// its last store 10 % after the median one. The worker's load warp draws and announces the tile to the other
// roles (of both CTAs of a pair) through a ring of kDrawSlots shared-memory words with a barrier each; the load
// warp is never more than the ring's stages plus the two accumulator buffers ahead of the slowest reader, which
// is less than kDrawSlots tiles.
constexpr int kDrawSlots = 16;

// Grouped form: item -> the tile index tile_coords takes, the groups [g_begin, g_end) the item covers
// and, for a piece, the index of its tile among the leftover tiles (-1 for a whole tile).
__device__ __forceinline__ void grouped_item(const GemmParams& p, int item, int& tile, int& g_begin, int& g_end,
                                             int& leftover) {
  tile = item;
  g_begin = 0;
  g_end = p.groups;
  leftover = -1;
  if (p.piece_items > 0 && item >= p.full_tiles) {
    const int q = item - p.full_tiles;
    leftover = q / p.groups;
    tile = p.full_tiles + leftover;
    g_begin = q - leftover * p.groups;
    g_end = g_begin + 1;
  }
}

// Tensor maps of the output destinations: BF16 [M,N] matrices, boxes of 64 columns x 32 rows.
// The gathering form can also close with a cross-GPU rendezvous inside the kernel. signal[d] points
// to kMaxOutputs arrival counters (64-bit, zero at first, never reset) in the memory of destination
// d's GPU, one per source rank; signal[0] is this GPU's own set. Every CTA of rank `source` adds one
// to counter `source` of every destination after its tile stores have completed, then waits until
// each of its own GPU's counters shows that all CTAs of that rank have arrived for this call: when the
// kernel ends, the whole gathered result is in this GPU's memory. state (four 64-bit words in this
// GPU's memory, zero at first) counts the calls, so that a call can be replayed from a CUDA graph:
// state[0] = completed calls, state[1] = CTAs of the running call that have left, state[2] = tiles drawn in
// the running call (see kDrawSlots), zero between calls; state[3] is spare.
struct OutputMaps {
  CUtensorMap map[kMaxOutputs];
  unsigned long long* signal[kMaxOutputs];
  unsigned long long* state;      // nullptr: no rendezvous, the caller orders a barrier after the call
  int source;                     // this rank
  // workspace form: the INT32 accumulator matrix [M,N] as boxes of 32 columns x 32 rows (has_ws_map != 0
  // when its pitch and base allow tile stores; otherwise the accumulators leave through direct stores)
  CUtensorMap ws_map;
  int has_ws_map;
};

template <int kCtas, int kMode>
struct GemmConfig {
  static constexpr int kBlockM = 128;                 // rows of A per CTA
  static constexpr int kTileN = 256;                  // accumulator columns per tile
  static constexpr int kBlockK = 128;                 // bytes of K per stage
  static constexpr int kOnesRows = kMode == kModeBiased ? 8 : 0;
  static constexpr int kChannelsPerTile = kTileN - kOnesRows;   // output channels per tile
  static constexpr int kBRowsSmem = kTileN / kCtas;   // weight rows held by one CTA
  // weight rows loaded by the CTA that also holds the ones rows (the only CTA, or the second of a pair)
  static constexpr int kBRowsLoad = kBRowsSmem - kOnesRows;
  static constexpr int kABytes = kBlockM * kBlockK;
  static constexpr int kBBytes = kBRowsSmem * kBlockK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // (the workspace form gives one ring stage to the staging boxes of its INT32 tile stores)
  static constexpr int kStages = (kCtas == 1 ? 4 : 6) - (kMode == kModeWorkspace ? 1 : 0);
  static constexpr int kEpiWarps = kMode == kModeGrouped ? 8 : 4;
  // Warp 0 loads, warp 1 issues the MMAs, the epilogue warps follow. The grouped form keeps 128 FP32 running
  // sums per epilogue thread: its epilogue warps start at warp 4 (warps 2 and 3 idle), so that the first
  // warpgroup can hand most of its registers to the two epilogue warpgroups (setmaxnreg); with ten warps
  // one scheduler would hold three of them, 168 registers each, and the sums would spill.
  static constexpr int kFirstEpiWarp = kMode == kModeGrouped ? 4 : 2;
  static constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
  // 384 threads start with 168 registers each; 128 x 40 + 256 x 232 is the same pool
  static constexpr int kRegsFrontWarps = 40, kRegsEpiWarps = 232;
  static constexpr int kColsPerEpiWarp = kTileN / (kEpiWarps / 4);
  static constexpr int kStoreBoxBytes = 32 * 128;     // one staged store box: 32 rows x 64 BF16
  static constexpr int kStoreBufs = kEpiWarps == 4 ? 2 : 1;   // staging boxes per epilogue warp
  static constexpr int kWsBufs = kMode == kModeWorkspace ? 2 : 0;   // INT32 staging boxes (32 x 32) per epilogue warp
  static constexpr int kStagingBytes = kEpiWarps * (kStoreBufs + kWsBufs) * kStoreBoxBytes;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Tile order: row tiles are walked in groups of group_m; inside a group the row tile index runs
// fastest, then the channel tile. One wave of CTAs then touches a bounded set of A rows (which
// stay in L2 while the weights stream past) instead of every row of a tall A.
//
// Work items: the tiles of the complete waves are whole; the tiles of the last, partial wave are cut
// into `split` column slices of tile_n/split accumulator columns that spread over the CTAs the wave
// would leave idle. A slice still streams the full K extent of A, but its MMAs are narrower and take
// about N/2 cycles each, so a half slice lasts ~0.6 of a whole tile.
//
// Mixed widths (wide_tiles > 0, never together with slices): the channels of a row stripe are cut into
// tiles_n tiles of which wide_tiles are 32 columns wider than the rest. The host picks tiles_n so that
// tiles_m * tiles_n fills whole waves of the persistent grid when no single width does (M = 2048,
// N = 7168 on 74 CTA pairs: 35 tiles of 192 and 2 of 224 per stripe are 296 tiles, exactly four per
// pair, where 224-wide tiles alone need 3.46 waves). The wide tiles sit at the front of the stripe in
// even raster groups and at its back in odd ones, so that they do not all land on the same workers.
// item -> tile (mt, nt), n_start = first output column of the item, n_width = its accumulator columns,
// alt = the item loads its weights through the second (slice / wide-tile) tensor map.
__host__ __device__ __forceinline__ void tile_coords(const GemmParams& p, int item, int& mt, int& nt, int& n_start,
                                                     int& n_width, bool& alt) {
  int tile = item, n_off = 0;
  n_width = p.tile_n;
  alt = false;
  if (item >= p.full_tiles) {
    const int extra = item - p.full_tiles;
    tile = p.full_tiles + extra / p.split;
    n_width = p.tile_n / p.split;
    n_off = (extra % p.split) * n_width;
    alt = true;
  }
  const int per_group = p.group_m * p.tiles_n;
  const int group = tile / per_group;
  const int within = tile - group * per_group;
  const int first_m = group * p.group_m;
  const int rows_left = p.tiles_m - first_m;
  const int rows_in_group = p.group_m < rows_left ? p.group_m : rows_left;
  mt = first_m + within % rows_in_group;
  nt = within / rows_in_group;
  if (p.wide_tiles > 0) {
    const int narrow = p.tiles_n - p.wide_tiles;
    // wide tiles before this one in the stripe
    const int wide_before = (group & 1) ? (nt > narrow ? nt - narrow : 0) : (nt < p.wide_tiles ? nt : p.wide_tiles);
    alt = (group & 1) ? nt >= narrow : nt < p.wide_tiles;
    n_width = p.tile_n + (alt ? 32 : 0);
    n_start = nt * p.tile_n + 32 * wide_before;
  } else {
    n_start = nt * p.tile_n + n_off;
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Grouped form, the pieces' workspace. One group's FP32 terms of one 256 x 256 tile are a plane of 16384
// float4, cut into blocks of 32 rows x 32 columns (row blocks outer): inside a block the eight float4 of a
// row's 32 columns are spread with the row (the lane) as the fastest index, so that a warp whose lanes hold
// one row each writes, and later reads, 512 contiguous bytes per instruction.
__device__ __forceinline__ int piece_term_index(int row_block, int col_block, int quad, int lane) {
  return ((row_block * 8 + col_block) * 8 + quad) * 32 + lane;
}

// Grouped form, end of a piece: the warp reports its terms, waits until every warp of every piece of the
// tile has done so, then adds the terms of this piece's share of the tile in ascending group order
// and stores it.
template <int kCtas, int kMode>
__device__ __forceinline__ void finish_piece(float* terms, unsigned* piece_sync, const __nv_bfloat16* channel_scales,
                                          __nv_bfloat16* out, int m, int n, int groups, int leftover, int g_begin, int mt,
                                          int n0, int n_width, int rank, int epi, int lane, bool out_vec,
                                          volatile int* abort_flag) {
  using Cfg = GemmConfig<kCtas, kMode>;
  struct { float* terms; unsigned* piece_sync; const __nv_bfloat16* sw; __nv_bfloat16* out; int m, n, groups; } p =
      {terms, piece_sync, channel_scales, out, m, n, groups};
  unsigned* sync = p.piece_sync + 2 * leftover;
  const unsigned expected = static_cast<unsigned>(p.groups) * Cfg::kEpiWarps * kCtas;   // warps over all pieces
  __threadfence();
  __syncwarp();
  unsigned all_in = 1u;
  if (lane == 0) {
    atomicAdd(sync, 1u);
    const unsigned long long start = global_timer_ns();
    for (uint32_t spin = 1; ld_acquire_gpu_u32(sync) < expected; ++spin) {
      __nanosleep(64);
      if ((spin & 255u) == 0u && (*abort_flag || global_timer_ns() - start > kWaitDeadlineNs)) {
        atomicOr(&g_ci8_status, kStatusWaitTimeout);   // a piece never arrived: this tile stays unwritten
        all_in = 0u;
        break;
      }
    }
  }
  all_in = __shfl_sync(0xffffffffu, all_in, 0);
  if (all_in) {
    // Share of piece g_begin: units [begin, end) of the plane's 256 units (a unit: the 32 rows of a block x
    // 8 columns, i.e. two adjacent float4 per lane), walked by the epilogue warps of both CTAs. Ascending-
    // group fadd chain, then the channel scale.
    constexpr int kTileRows = Cfg::kBlockM * kCtas, kPlane = kTileRows * Cfg::kTileN / 4, kUnits = kPlane / 64;
    const int begin = static_cast<int>(static_cast<long long>(kUnits) * g_begin / p.groups);
    const int end = static_cast<int>(static_cast<long long>(kUnits) * (g_begin + 1) / p.groups);
    const float4* tile_terms = reinterpret_cast<const float4*>(p.terms) + static_cast<size_t>(leftover) * p.groups * kPlane;
    const int tile_row0 = mt * kTileRows;
    const bool sw_vec = reinterpret_cast<uintptr_t>(p.sw) % 16 == 0;
    // Two units per round, all of their loads in flight together: with eight groups a warp's whole share
    // (two units) costs one round trip to L2.
    constexpr int kStep = kCtas * Cfg::kEpiWarps;
    for (int unit0 = begin + rank * Cfg::kEpiWarps + epi; unit0 < end; unit0 += 2 * kStep) {
      int col[2], out_row[2];
      bool live[2];
      const float4* src[2];
      uint4 sw_words[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int unit = unit0 + u * kStep;
        const int block = unit >> 2, pair = unit & 3;
        const int row_block = block >> 3, col_block = block & 7;
        const int col8 = col_block * 32 + pair * 8;
        out_row[u] = tile_row0 + row_block * 32 + lane;
        col[u] = n0 + col8;
        live[u] = unit < end && col[u] < p.n && col8 < n_width;      // the same for every lane
        src[u] = tile_terms + piece_term_index(row_block, col_block, 2 * pair, lane);
        // the eight channel scales of the unit (the same for every lane), fetched ahead of the terms
        sw_words[u] = make_uint4(0u, 0u, 0u, 0u);
        if (live[u]) {
          if (sw_vec && col[u] + 8 <= p.n) {
            sw_words[u] = __ldg(reinterpret_cast<const uint4*>(p.sw + col[u]));
          } else {
            uint16_t* parts = reinterpret_cast<uint16_t*>(&sw_words[u]);
            for (int j = 0; j < 8; ++j)
              if (col[u] + j < p.n) parts[j] = reinterpret_cast<const uint16_t*>(p.sw)[col[u] + j];
          }
        }
      }
      float4 lo[2], hi[2];
      // eight groups' terms of both units are fetched together, then added in ascending group order
#pragma unroll 1
      for (int g0 = 0; g0 < p.groups; g0 += 8) {
        float4 a[2][8], b[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float4* base = src[u] + static_cast<size_t>(g0) * kPlane;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (live[u] && g0 + i < p.groups) {
              a[u][i] = __ldcg(base + i * kPlane);
              b[u][i] = __ldcg(base + i * kPlane + 32);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (live[u] && g0 + i < p.groups) {
              if (g0 + i == 0) {
                lo[u] = a[u][i];
                hi[u] = b[u][i];
              } else {
                lo[u] = make_float4(__fadd_rn(lo[u].x, a[u][i].x), __fadd_rn(lo[u].y, a[u][i].y), __fadd_rn(lo[u].z, a[u][i].z),
                                    __fadd_rn(lo[u].w, a[u][i].w));
                hi[u] = make_float4(__fadd_rn(hi[u].x, b[u][i].x), __fadd_rn(hi[u].y, b[u][i].y), __fadd_rn(hi[u].z, b[u][i].z),
                                    __fadd_rn(hi[u].w, b[u][i].w));
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!live[u] || out_row[u] >= p.m) continue;
        const float sum[8] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w};
        const uint32_t sw_pairs[4] = {sw_words[u].x, sw_words[u].y, sw_words[u].z, sw_words[u].w};
        uint32_t words[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          // a BF16 is the upper half of the FP32 with the same value
          const float s0 = __uint_as_float(sw_pairs[j >> 1] << 16);
          const float s1 = __uint_as_float(sw_pairs[j >> 1] & 0xffff0000u);
          words[j >> 1] = pack_bf16x2(__fmul_rn(sum[j], s0), __fmul_rn(sum[j + 1], s1));
        }
        __nv_bfloat16* dst = p.out + static_cast<size_t>(out_row[u]) * p.n + col[u];
        if (out_vec && col[u] + 8 <= p.n) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
        } else {
          for (int j = 0; j < 8; ++j)
            if (col[u] + j < p.n)
              reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>((j & 1) ? (words[j >> 1] >> 16) : (words[j >> 1] & 0xffffu));
        }
      }
    }
  }
  // the last warp to leave puts the counters back to zero for the next launch
  __syncwarp();
  if (lane == 0 && atomicAdd(sync + 1, 1u) == expected - 1u) {
    sync[0] = 0u;
    sync[1] = 0u;
  }
}

template <int kCtas, int kMode>
__global__ void __launch_bounds__(GemmConfig<kCtas, kMode>::kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a,
               const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_w_slice,
               const __grid_constant__ OutputMaps out_maps, const GemmParams p) {
  using Cfg = GemmConfig<kCtas, kMode>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  constexpr int kRingBytes = Cfg::kStages * Cfg::kStageBytes;
  uint8_t* staging = smem + kRingBytes;
  uint8_t* bar_region = staging + Cfg::kStagingBytes;
  const uint32_t bar_base = smem_base + kRingBytes + Cfg::kStagingBytes;
  // barrier layout (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_region + 8 * (2 * Cfg::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // grouped form with pieces: the barrier the piece's number is announced on, and the number
  const uint32_t piece_bar = bar_base + 8u * (2 * Cfg::kStages + 5);
  volatile int* piece_slot = reinterpret_cast<volatile int*>(bar_region + 8 * (2 * Cfg::kStages + 6));
  // drawn tiles (see kDrawSlots): barriers at byte 192, the tiles' numbers behind them
  auto draw_bar = [&](int i) { return bar_base + 192u + 8u * i; };
  volatile int* draw_slot = reinterpret_cast<volatile int*>(bar_region + 192 + 8 * kDrawSlots);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kCtas == 2 ? cluster_ctarank() : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), Cfg::kEpiWarps * kCtas);
    }
    if constexpr (kMode == kModeGrouped) mbar_init(piece_bar, 1);
    if (out_maps.state != nullptr)
      for (int i = 0; i < kDrawSlots; ++i) mbar_init(draw_bar(i), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
    if (p.split > 1 || p.wide_tiles > 0 || (kMode == kModeBiased && kCtas == 2)) prefetch_tensormap(&map_w_slice);
    for (int d = 0; d < p.num_outputs; ++d) prefetch_tensormap(&out_maps.map[d]);
  }
  if constexpr (kMode == kModeBiased) {
    if (kCtas == 1 || rank == 1) {
    // Eight rows of ones behind the weight rows of every stage (the swizzle permutes 16-byte
    // chunks within a row, so a constant fill is layout-independent).
    constexpr int kOnesBytes = Cfg::kOnesRows * Cfg::kBlockK;
    for (int i = threadIdx.x; i < Cfg::kStages * (kOnesBytes / 16); i += Cfg::kThreads) {
      const int s = i / (kOnesBytes / 16), c = i % (kOnesBytes / 16);
      uint8_t* dst = smem + s * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBRowsLoad * Cfg::kBlockK;
      reinterpret_cast<uint4*>(dst)[c] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    }
    fence_proxy_async_smem();
  }
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(tmem_slot), 512);
    tmem_relinquish<kCtas>();
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched with programmatic stream serialization: everything above (barriers, TMEM, descriptor
  // prefetch) may overlap the tail of the previous kernel in the stream; global memory is touched
  // only after that kernel has finished.
  pdl_wait();

  // calls completed so far on this set of buffers (the rendezvous at the end counts from it)
  const unsigned long long calls_done = out_maps.state ? ld_relaxed_u64(out_maps.state) : 0ull;

  const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;   // per group
  // Work items: whole tiles, then column slices, walked with a fixed stride. The pieces of the grouped form
  // are not dealt out in advance: a worker that has finished its whole tiles takes the next piece from a
  // counter, so the pieces go to the workers that are ahead. (SM clocks differ by a few percent between
  // parts of the chip under the power cap; with a fixed assignment the pieces of a tile, which have to wait
  // for one another, finished with the slowest worker that held one.)
  const bool pieces = kMode == kModeGrouped && p.piece_items > 0;
  const int total_tiles = pieces ? p.full_tiles : p.total_items;
  // Called by whole warps once their fixed items are done. The first CTA's load warp draws the number and
  // announces it to every other role of the CTA (pair); returns the item, or -1 when no piece is left.
  auto fetch_piece = [&]() -> int {
    if constexpr (kMode != kModeGrouped) {
      return -1;
    } else {
      if (!pieces) return -1;
      int q = 0;
      if (warp == 0 && rank == 0) {
        if (lane == 0) {
          const unsigned workers = gridDim.x / kCtas;
          q = static_cast<int>(atomicAdd(p.piece_sync + kPieceFetchWord, 1u));
          // every worker draws exactly once per launch: the last draw puts the counter back for the next one
          if (static_cast<unsigned>(q) == workers - 1u) p.piece_sync[kPieceFetchWord] = 0u;
          *piece_slot = q;
          if constexpr (kCtas == 2)
            st_shared_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(piece_slot)), 1), static_cast<uint32_t>(q));
          mbar_arrive(piece_bar);
          if constexpr (kCtas == 2) mbar_arrive_cluster(piece_bar, 1);
        }
        q = __shfl_sync(0xffffffffu, q, 0);
      } else {
        if (!__all_sync(0xffffffffu, mbar_wait<kCtas == 2>(piece_bar, 0u, abort_flag))) return -1;
        q = *piece_slot;
      }
      return q < p.piece_items ? p.full_tiles + q : -1;
    }
  };
  const int first_tile = kCtas == 2 ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_stride = kCtas == 2 ? (gridDim.x >> 1) : gridDim.x;
  // The item after `tile` for the calling warp (all of its lanes): the fixed stride, or in the gathering form
  // with a rendezvous the worker's next draw (`draws` counts them per role; a value past the last item ends the
  // walk for every role alike, and an abandoned wait returns one as well).
  const bool drawn = kMode == kModeFused && out_maps.state != nullptr;
  auto next_item = [&](int tile, int& draws) -> int {
    if (!drawn) return tile + tile_stride;
    const int slot = draws % kDrawSlots;                                          // draw number `draws`, from zero
    const uint32_t parity = static_cast<uint32_t>(draws / kDrawSlots) & 1u;       // how often the slot was used before
    ++draws;
    int value = 0;
    if (warp == 0 && rank == 0) {
      if (lane == 0) {
        value = tile_stride + static_cast<int>(atomicAdd(out_maps.state + 2, 1ull));
        draw_slot[slot] = value;
        if constexpr (kCtas == 2)
          st_shared_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(draw_slot + slot)), 1), static_cast<uint32_t>(value));
        mbar_arrive(draw_bar(slot));
        if constexpr (kCtas == 2) mbar_arrive_cluster(draw_bar(slot), 1);
      }
      value = __shfl_sync(0xffffffffu, value, 0);
    } else {
      if (!__all_sync(0xffffffffu, mbar_wait<kCtas == 2>(draw_bar(slot), parity, abort_flag))) return 0x7fffffff;
      value = draw_slot[slot];
    }
    return value;
  };

  if (warp < Cfg::kFirstEpiWarp) {
    // grouped form: the first warpgroup (loads, MMAs, two idle warps) gives registers up for the epilogue's
    if constexpr (kMode == kModeGrouped) setmaxnreg_dec<Cfg::kRegsFrontWarps>();
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      // The producer and MMA loops are run by their whole warp with one elected lane issuing: the
      // loop state then lives in uniform registers, which is where TMA and MMA instructions take
      // their operands. Issued from a single thread inside a divergent branch, every instruction
      // pays tens of cycles of register moves (measured: 47-76 cycles per MMA against 128 cycles
      // of tensor-pipe time for a 128 x 256 x 32 step, before the waits and commits).
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t leader_full0 = kCtas == 2 ? map_to_cta(full_bar(0), 0) : full_bar(0);
      // the raster keeps a group of A rows in L2 while the weights stream past: A lines leave L2 last
      const uint64_t a_policy = l2_policy_evict_last();
      bool ok = true;
      bool drew = false;
      int draws = 0;
      for (int tile = first_tile; ok; tile = next_item(tile, draws)) {
        if (tile >= total_tiles) {
          if (drew || (tile = fetch_piece()) < 0) break;
          drew = true;
        }
        int mt, nt, n_start, n_width, g_begin = 0, g_end = p.groups, leftover = -1, tile_index = tile;
        bool alt;
        if constexpr (kMode == kModeGrouped) grouped_item(p, tile, tile_index, g_begin, g_end, leftover);
        tile_coords(p, tile_index, mt, nt, n_start, n_width, alt);
        const int a_row = mt * (Cfg::kBlockM * kCtas) + rank * Cfg::kBlockM;
        // a pair's CTAs supply half the weight rows each; slices and wide tiles load through their own box
        // (biased pair: the first CTA loads 128 channels through map_w, the second 120 through the other map)
        const int w_row = n_start + rank * (kMode == kModeBiased ? Cfg::kBRowsSmem : n_width / kCtas);
        const CUtensorMap* w_map = (alt || (kMode == kModeBiased && rank == 1)) ? &map_w_slice : &map_w;
        const uint32_t tx = kMode == kModeBiased
                                ? static_cast<uint32_t>(kCtas * Cfg::kABytes + Cfg::kChannelsPerTile * Cfg::kBlockK)
                                : static_cast<uint32_t>(alt ? p.stage_tx_slice : p.stage_tx) * kCtas;
        for (int g = g_begin; ok && g < g_end; ++g) {
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))) { ok = false; break; }
            if (elect_one()) {
              if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), tx);
              const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
              const uint32_t b_dst = a_dst + Cfg::kABytes;
              const uint32_t bar = leader_full0 + 8u * stage;
              const int kx = kb * Cfg::kBlockK;
              if constexpr (kCtas == 2) {
                tma_load_2d_pair_hint(a_dst, &map_a, kx, g * p.m + a_row, bar, a_policy);
                tma_load_2d_pair(b_dst, w_map, g * p.k + kx, w_row, bar);
              } else {
                tma_load_2d_hint(a_dst, &map_a, kx, g * p.m + a_row, bar, a_policy);
                tma_load_2d(b_dst, w_map, g * p.k + kx, w_row, bar);
              }
            }
            __syncwarp();
            if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
      pdl_launch_dependents();       // all of this CTA's loads are issued: the next kernel may set up
      if (!ok) __nanosleep(200000);  // let loads already in flight land before teardown
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (rank == 0) {
        int stage = 0;
        uint32_t phase = 0, acc_iter = 0;
        bool ok = true;
        bool drew = false;
        int draws = 0;
        for (int tile = first_tile; ok; tile = next_item(tile, draws)) {
          if (tile >= total_tiles) {
            if (drew || (tile = fetch_piece()) < 0) break;
            drew = true;
          }
          int mt, nt, n_start, n_width, g_begin = 0, g_end = p.groups, leftover = -1, tile_index = tile;
          bool alt;
          if constexpr (kMode == kModeGrouped) grouped_item(p, tile, tile_index, g_begin, g_end, leftover);
          tile_coords(p, tile_index, mt, nt, n_start, n_width, alt);
          // accumulator columns the MMA produces (the biased form adds its 16 ones columns)
          const uint32_t idesc = idesc_i8(Cfg::kBlockM * kCtas, kMode == kModeBiased ? Cfg::kTileN : n_width,
                                          /*b_unsigned=*/kMode == kModeBiased);
          for (int g = g_begin; ok && g < g_end; ++g, ++acc_iter) {
            const uint32_t buf = acc_iter & 1u, acc_phase = (acc_iter >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait<kCtas == 2>(tmem_empty_bar(buf), acc_phase ^ 1u, abort_flag))) {
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const uint32_t tmem_d = tmem_base + buf * Cfg::kTileN;
            for (int kb = 0; kb < num_kb; ++kb) {
              if (!__all_sync(0xffffffffu, mbar_wait<kCtas == 2>(full_bar(stage), phase, abort_flag))) {
                ok = false;
                break;
              }
              tcgen05_fence_after();
              const uint32_t a_addr = smem_base + stage * Cfg::kStageBytes;
              const uint64_t a_desc = smem_desc_sw128(a_addr);
              const uint64_t b_desc = smem_desc_sw128(a_addr + Cfg::kABytes);
              if (elect_one()) {
  #pragma unroll
                for (int ks = 0; ks < Cfg::kBlockK / 32; ++ks)
                  mma_i8<kCtas>(tmem_d, a_desc + 2u * ks, b_desc + 2u * ks, idesc,
                                (kb | ks) != 0 ? 1u : 0u);
                if constexpr (kCtas == 2) {
                  mma_commit_pair(map_to_cta(empty_bar(stage), 0));
                  mma_commit_pair(map_to_cta(empty_bar(stage), 1));
                } else {
                  mma_commit(empty_bar(stage));
                }
              }
              __syncwarp();
              if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
            }
            if (!ok) break;
            if (elect_one()) {
              if constexpr (kCtas == 2) {
                mma_commit_pair(map_to_cta(tmem_full_bar(buf), 0));
                mma_commit_pair(map_to_cta(tmem_full_bar(buf), 1));
              } else {
                mma_commit(tmem_full_bar(buf));
              }
            }
            __syncwarp();
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    if constexpr (kMode == kModeGrouped) setmaxnreg_inc<Cfg::kRegsEpiWarps>();
    const int epi = warp - Cfg::kFirstEpiWarp;
    const int quarter = warp & 3;                       // TMEM lanes this warp may read
    const int col_base = (epi >> 2) * Cfg::kColsPerEpiWarp;
    constexpr int kChunks = Cfg::kColsPerEpiWarp / 64;  // 64 output columns per staged box
    const bool tma_out = p.num_outputs > 0;
    const bool out_vec = (p.n % 8 == 0) && (reinterpret_cast<uintptr_t>(p.out) % 16 == 0);
    const bool ws_vec = (p.n % 4 == 0) && (reinterpret_cast<uintptr_t>(p.workspace) % 16 == 0);
    uint8_t* my_staging = staging + epi * (Cfg::kStoreBufs + Cfg::kWsBufs) * Cfg::kStoreBoxBytes;
    uint8_t* my_ws_staging = my_staging + Cfg::kStoreBufs * Cfg::kStoreBoxBytes;
    const bool ws_tma = kMode == kModeWorkspace && out_maps.has_ws_map != 0;
    uint32_t acc_iter = 0, store_iter = 0;
    bool ok = true;
    const uint64_t store_policy = l2_policy_evict_first();
    float total[kMode == kModeGrouped ? Cfg::kColsPerEpiWarp : 1];
    int piece_tile = -1, piece_group = 0, piece_mt = 0, piece_n0 = 0, piece_width = 0;
    bool drew = false;
    int draws = 0;
    for (int tile = first_tile; ok; tile = next_item(tile, draws)) {
      if (tile >= total_tiles) {
        if (drew || (tile = fetch_piece()) < 0) break;
        drew = true;
      }
      int mt, nt, n0, n_width;                            // n0 = first output column of this item
      int g_begin = 0, g_end = p.groups, leftover = -1, tile_index = tile;
      bool alt;
      if constexpr (kMode == kModeGrouped) grouped_item(p, tile, tile_index, g_begin, g_end, leftover);
      tile_coords(p, tile_index, mt, nt, n0, n_width, alt);
      const int row0 = mt * (Cfg::kBlockM * kCtas) + rank * Cfg::kBlockM + quarter * 32;
      const int row = row0 + lane;
      // Channel scales of this warp's columns, all fetched here, ahead of the accumulators: lane j of word i
      // holds sw[n0 + col_base + 32 i + j]. Fetched where each 32-column half needs them, every half began with
      // a round trip to L2 (cycle stamps: 1100 cycles per half, 10 k for a tile's epilogue; hidden behind the
      // next tile's MMAs, but not behind the last one's).
      float tile_sw[Cfg::kColsPerEpiWarp / 32];
#pragma unroll
      for (int i = 0; i < Cfg::kColsPerEpiWarp / 32; ++i) {
        const int channel = n0 + col_base + i * 32 + lane;
        tile_sw[i] = channel < p.n ? __bfloat162float(p.sw[channel]) : 0.f;
      }
      if constexpr (kMode == kModeGrouped) {
        // the running sums of the previous item are dead (this item's first group overwrites them): say so
#pragma unroll
        for (int t = 0; t < Cfg::kColsPerEpiWarp; ++t) asm volatile("" : "=f"(total[t]));
      }
      for (int g = g_begin; g < g_end; ++g, ++acc_iter) {
        const uint32_t buf = acc_iter & 1u, acc_phase = (acc_iter >> 1) & 1u;
        // (fetched ahead of the wait: the scale does not depend on the accumulators)
        const float row_scale = row < p.m ? p.sa[static_cast<size_t>(g) * p.m + row] : 0.f;
        if (!__all_sync(0xffffffffu, mbar_wait<kCtas == 2>(tmem_full_bar(buf), acc_phase, abort_flag))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               buf * Cfg::kTileN + col_base;
        int32_t bias = 0;
        if constexpr (kMode == kModeBiased) {
          uint32_t ones[8];
          tmem_ld_32x8(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                           buf * Cfg::kTileN + p.tile_n, ones);
          tmem_ld_wait();
          bias = static_cast<int32_t>(ones[0]) * 128;
        }
        if constexpr (kMode == kModeSwiGLU) {
          // Accumulator columns [0,128) are gate channels, [128,256) the matching up channels. Two output
          // boxes of 64 columns per tile; each half box needs 32 gate and 32 up accumulators.
          const int h0_tile = nt * (Cfg::kTileN / 2);       // first output column of this tile
#pragma unroll
          for (int boxi = 0; boxi < 2; ++boxi) {
            const int c0 = h0_tile + boxi * 64;             // first output column of this box
            const bool store_box = c0 < p.out_n;
            uint8_t* box = my_staging + (store_iter % Cfg::kStoreBufs) * Cfg::kStoreBoxBytes;
            if (store_box && store_iter >= Cfg::kStoreBufs) {
              if (lane == 0) tma_store_wait_read<Cfg::kStoreBufs - 1>();
              __syncwarp();
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int gate_col = boxi * 64 + half * 32;   // accumulator column of the first gate value
              uint32_t vg[32], vu[32];
              tmem_ld_32x32(taddr + gate_col, vg);
              tmem_ld_32x32(taddr + Cfg::kTileN / 2 + gate_col, vu);
              tmem_ld_wait_for(vg);
              tmem_ld_wait_for(vu);
              if (!store_box) continue;
              // channel scales: lane j holds those of gate column j and up column j of this half box
              const float my_gate_sw = tile_sw[boxi * 2 + half], my_up_sw = tile_sw[Cfg::kTileN / 64 + boxi * 2 + half];
              uint32_t packed[16];
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                float h[2];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                  const float gs = __shfl_sync(0xffffffffu, my_gate_sw, j + t);
                  const float us = __shfl_sync(0xffffffffu, my_up_sw, j + t);
                  // what fused_channel_mm would have written (BF16), read back as silu_mul would
                  const float gate = __bfloat162float(__float2bfloat16_rn(
                      __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(vg[j + t])), row_scale), gs)));
                  const float up = __bfloat162float(__float2bfloat16_rn(
                      __fmul_rn(__fmul_rn(__int2float_rn(static_cast<int32_t>(vu[j + t])), row_scale), us)));
                  h[t] = swiglu_one(gate, up);
                }
                packed[j >> 1] = pack_bf16x2(h[0], h[1]);
              }
              uint4* row_base = reinterpret_cast<uint4*>(box + lane * 128);
#pragma unroll
              for (int c = 0; c < 4; ++c)
                row_base[(half * 4 + c) ^ (lane & 7)] =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            if (store_box) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0 && row0 < p.m) {
                tma_store_2d_hint(&out_maps.map[0], smem_u32(box), c0, row0, store_policy);
                tma_store_commit();
              }
              ++store_iter;
            }
          }
        } else {
        const bool last_group = g + 1 == p.groups && leftover < 0;   // a piece never stores the output here
#pragma unroll
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          const int tile_col = col_base + chunk * 64;     // first accumulator column of this 64-wide box
          if (tile_col >= n_width) continue;              // a narrow tile or a slice has fewer boxes
          const int c0 = n0 + tile_col;                   // its first output column
          const bool store_box = (kMode != kModeGrouped || last_group) && c0 < p.n;
          // a box that straddles the item's right edge (its width is a multiple of 32, not of 64) must not
          // be written as a whole 64-wide TMA box: its valid half goes out with direct stores
          const bool tma_box = tma_out && tile_col + 64 <= n_width;
          uint8_t* box = my_staging + (store_iter % Cfg::kStoreBufs) * Cfg::kStoreBoxBytes;
          if (tma_box && store_box && store_iter >= Cfg::kStoreBufs) {
            // the box is reused only after its previous stores have finished reading it
            if (lane == 0) tma_store_wait_read<Cfg::kStoreBufs - 1>();
            __syncwarp();
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int h0 = c0 + half * 32;                // 32 columns per TMEM load
            uint32_t v[32];
            tmem_ld_32x32(taddr + chunk * 64 + half * 32, v);
            tmem_ld_wait();
            if constexpr (kMode == kModeGrouped) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float term = __fmul_rn(__int2float_rn(static_cast<int32_t>(v[j])), row_scale);
                const int t = chunk * 64 + half * 32 + j;
                total[t] = g == g_begin ? term : __fadd_rn(total[t], term);
              }
              if (leftover >= 0 && tile_col + half * 32 < n_width) {
                // a piece: this group's terms of the warp's 32 rows x 32 columns to the workspace, in the
                // order piece_term_index gives (the lanes of a store are adjacent: 512 contiguous bytes)
                float4* plane = reinterpret_cast<float4*>(p.terms) +
                                (static_cast<size_t>(leftover) * p.groups + g) * (Cfg::kBlockM * kCtas * Cfg::kTileN / 4);
                const int row_block = static_cast<int>(rank) * (Cfg::kBlockM / 32) + quarter;
                const int col_block = (tile_col + half * 32) >> 5;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const int t = chunk * 64 + half * 32 + j;
                  __stcg(plane + piece_term_index(row_block, col_block, j >> 2, lane),
                         make_float4(total[t], total[t + 1], total[t + 2], total[t + 3]));
                }
              }
            }
            if (!store_box || h0 >= p.n || tile_col + half * 32 >= n_width) continue;
            // channel scales of these 32 columns: lane j holds sw[h0 + j]
            const float my_sw = tile_sw[chunk * 2 + half];
            const int limit = kMode == kModeBiased
                                  ? min(p.n - h0, n_width - (tile_col + half * 32))
                                  : p.n - h0;
            if constexpr (kMode == kModeBiased) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = static_cast<uint32_t>(static_cast<int32_t>(v[j]) - bias);
            }
            if constexpr (kMode == kModeWorkspace) {
              if (ws_tma) {
                // The accumulators leave as a 32 x 32 INT32 tile store (128-byte rows, same swizzle as the BF16
                // boxes). Two staging boxes alternate; letting at most one store group stay pending before a box
                // is written again is enough: whatever was committed before the latest group has then been read.
                uint8_t* ws_box = my_ws_staging + half * Cfg::kStoreBoxBytes;
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                uint4* ws_row = reinterpret_cast<uint4*>(ws_box + lane * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c)
                  ws_row[c ^ (lane & 7)] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && row0 < p.m) {
                  tma_store_2d(&out_maps.ws_map, smem_u32(ws_box), h0, row0);
                  tma_store_commit();
                }
              } else if (row < p.m) {
                int32_t* ws = p.workspace + static_cast<size_t>(row) * p.n + h0;
                if (ws_vec && limit >= 32) {
#pragma unroll
                  for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<uint4*>(ws + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                } else {
                  for (int j = 0; j < 32; ++j)
                    if (j < limit) ws[j] = static_cast<int32_t>(v[j]);
                }
              }
            }
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float s0 = __shfl_sync(0xffffffffu, my_sw, j);
              const float s1 = __shfl_sync(0xffffffffu, my_sw, j + 1);
              float f0, f1;
              if constexpr (kMode == kModeGrouped) {
                f0 = total[chunk * 64 + half * 32 + j];
                f1 = total[chunk * 64 + half * 32 + j + 1];
              } else {
                f0 = __fmul_rn(__int2float_rn(static_cast<int32_t>(v[j])), row_scale);
                f1 = __fmul_rn(__int2float_rn(static_cast<int32_t>(v[j + 1])), row_scale);
              }
              packed[j >> 1] = pack_bf16x2(__fmul_rn(f0, s0), __fmul_rn(f1, s1));
            }
            if (tma_box) {
              // Stage with the 128-byte swizzle the store's tensor map expects: 16-byte chunk c of
              // box row r lives at chunk c ^ (r & 7).
              uint4* row_base = reinterpret_cast<uint4*>(box + lane * 128);
#pragma unroll
              for (int c = 0; c < 4; ++c)
                row_base[(half * 4 + c) ^ (lane & 7)] =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            } else if (row < p.m) {
              __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * p.n + h0;
              if (out_vec && limit >= 32) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  *reinterpret_cast<uint4*>(dst + 2 * j) =
                      make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
              } else if (out_vec && limit % 8 == 0) {
                // a tile edge inside these 32 columns (widths are multiples of 8): whole 16-byte groups
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                  if (2 * j < limit)
                    *reinterpret_cast<uint4*>(dst + 2 * j) =
                        make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
              } else {
                for (int j = 0; j < 32; ++j)
                  if (j < limit) {
                    const uint32_t word = packed[j >> 1];
                    reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>((j & 1) ? (word >> 16) : (word & 0xffffu));
                  }
              }
            }
          }
          if (tma_box && store_box) {
            // one lane stores the staged box to every destination (columns past N and rows past M
            // are clipped by the tensor map)
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < p.m) {
              // destination 0 is this GPU's own memory: written once, so it should not displace the A
              // rows and W tiles that the next tiles read again; the others are peers' buffers
              tma_store_2d_hint(&out_maps.map[0], smem_u32(box), c0, row0, store_policy);
              for (int d = 1; d < p.num_outputs; ++d)
                tma_store_2d(&out_maps.map[d], smem_u32(box), c0, row0);
              tma_store_commit();
            }
            ++store_iter;
          }
        }
        }
        // this warp is done with the accumulator buffer
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtas == 2) mbar_arrive_cluster(tmem_empty_bar(buf), 0);
          else mbar_arrive(tmem_empty_bar(buf));
        }
      }
      if constexpr (kMode == kModeGrouped) {
        if (leftover >= 0) {   // a piece is always a worker's last item: remember it and finish it below
          piece_tile = leftover;
          piece_group = g_begin;
          piece_mt = mt;
          piece_n0 = n0;
          piece_width = n_width;
        }
      }
    }
    if constexpr (kMode == kModeGrouped) {
      // ---- a piece: wait for the other pieces of its tile, then finish this piece's share of it. Done behind
      // the item loop, where the running sums are dead and their registers free for the terms in flight.
      if (piece_tile >= 0 && ok)
        finish_piece<kCtas, kMode>(p.terms, p.piece_sync, p.sw, p.out, p.m, p.n, p.groups, piece_tile, piece_group, piece_mt,
                                   piece_n0, piece_width, static_cast<int>(rank), epi, lane, out_vec, abort_flag);
    }
    if ((tma_out || ws_tma) && lane == 0) {
      // staged boxes must outlive their stores; before the rendezvous the stores must have landed as well
      if (out_maps.state) tma_store_wait_all(); else tma_store_wait_read<0>();
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<kCtas>(tmem_base, 512);
  }
  if (out_maps.state != nullptr && threadIdx.x == 0) {
    // Cross-GPU rendezvous. Every epilogue warp of this CTA has waited for its tile stores (the
    // __syncthreads above orders that before this thread); the fences make those writes, which went
    // through the async proxy, precede the release of the arrival counts at system scope.
    fence_proxy_async_global();
    __threadfence_system();
    for (int d = 0; d < p.num_outputs; ++d) red_release_sys_add_u64(out_maps.signal[d] + out_maps.source, 1ull);
    // one counter per source rank: a rank that is already a call ahead cannot stand in for a late one
    const unsigned long long target = (calls_done + 1ull) * gridDim.x;
    const unsigned long long start = global_timer_ns();
    bool arrived = true;
    for (int from = 0; arrived && from < p.num_outputs; ++from) {
      for (uint32_t spin = 1; ld_acquire_sys_u64(out_maps.signal[0] + from) < target; ++spin) {
        __nanosleep(64);
        if ((spin & 255u) == 0u && global_timer_ns() - start > kWaitDeadlineNs) {
          atomicOr(&g_ci8_status, kStatusPeerTimeout);   // a peer never arrived: the gathered result is incomplete
          arrived = false;
          break;
        }
      }
    }
    // the last CTA to leave publishes the call count for the next call on these buffers (after a
    // timeout it still counts the call, so the host can read the status word and carry on)
    (void)arrived;
    __threadfence();
    if (atomicAdd(out_maps.state + 1, 1ull) == gridDim.x - 1ull) {
      out_maps.state[1] = 0ull;
      out_maps.state[2] = 0ull;   // every worker has drawn its last tile: the next call draws from zero again
      __threadfence();
      st_relaxed_u64(out_maps.state, calls_done + 1ull);
    }
  }
}

}  // namespace ci8

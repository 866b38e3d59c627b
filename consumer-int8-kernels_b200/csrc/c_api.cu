// Host side of libci8.so: argument checks, tensor-map construction, schedule selection and
// launches behind the C ABI declared in include/ci8.h. No allocation, no synchronisation.
#include "../../include/ci8.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>

#include "allspark_unpack.cuh"
#include "decode_splitk.cuh"
#include "gemm_tcgen05.cuh"
#include "gemv_w8a16.cuh"
#include "q8_block.cuh"
#include "quantize.cuh"

namespace {

using namespace ci8;

constexpr int kInvalid = static_cast<int>(cudaErrorInvalidValue);
constexpr int kMaxDevices = 64;

// ------------------------------------------------------------------ per-device facts
struct DeviceInfo {
  std::atomic<int> sm_count{0};
};
DeviceInfo g_devices[kMaxDevices];

int sm_count() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 148;
  int count = g_devices[device].sm_count.load(std::memory_order_relaxed);
  if (count == 0) {
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    g_devices[device].sm_count.store(count, std::memory_order_relaxed);
  }
  return count;
}

// Raises a kernel's dynamic shared-memory limit once per device (idempotent, capture-safe).
template <typename Kernel>
cudaError_t ensure_smem(Kernel kernel, int bytes, std::atomic<uint64_t>& done_mask) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  const uint64_t bit = uint64_t(1) << (device & 63);
  if (done_mask.load(std::memory_order_acquire) & bit) return cudaSuccess;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err == cudaSuccess) done_mask.fetch_or(bit, std::memory_order_release);
  return err;
}

// ------------------------------------------------------------------ tensor maps
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled_fn() {
  static std::atomic<void*> cached{nullptr};
  void* fn = cached.load(std::memory_order_acquire);
  if (!fn) {
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess)
      return nullptr;
    cached.store(fn, std::memory_order_release);
  }
  return reinterpret_cast<EncodeTiled>(fn);
}

// Row-major byte matrix [rows, cols] -> tiles of box_rows x 128 bytes, 128-byte swizzle,
// out-of-range elements read as zero.
cudaError_t make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiled encode = encode_tiled_fn();
  if (!encode) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {128u, box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

bool aligned(const void* p, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(p) % bytes == 0; }

// ------------------------------------------------------------------ tcgen05 GEMM launch
// BF16 [rows, cols] matrix -> boxes of box_cols x box_rows elements with the 128-byte swizzle.
cudaError_t make_bf16_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                          uint32_t box_rows);
// BF16 [rows, cols] output matrix -> store boxes of 64 columns x 32 rows.
cudaError_t make_output_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols) {
  return make_bf16_map(map, base, rows, cols, 64, 32);
}
cudaError_t make_bf16_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                          uint32_t box_rows) {
  EncodeTiled encode = encode_tiled_fn();
  if (!encode) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Bytes of activations one raster group may hold (they are meant to stay in L2 while the weights stream
// past). CI8_RASTER_MIB overrides the default for experiments; read once.
long long raster_bytes() {
  static const long long bytes = [] {
    const char* text = std::getenv("CI8_RASTER_MIB");
    const long mib = text ? std::strtol(text, nullptr, 10) : 0;
    return static_cast<long long>(mib >= 1 && mib <= 120 ? mib : 36) << 20;
  }();
  return bytes;
}

// Grouped form with a workspace: how many tiles (256 x 256, CTA pairs) the last, partial wave holds when
// cutting them along the groups pays: one piece per worker at most, and a last wave less than half
// full (a fuller one is better left alone). 0 otherwise.
constexpr size_t kPieceHeaderBytes = 1024;                       // the pieces' counters
constexpr size_t kPieceTermBytes = 256 * 256 * sizeof(float);    // one group's terms of one tile
int grouped_leftover_tiles(int m, int n, int groups, long long workers) {
  if (m <= 128 || groups < 2) return 0;
  const long long tiles = static_cast<long long>((m + 255) / 256) * ((n + 255) / 256);
  const long long rest = tiles % workers;
  return (rest > 0 && rest * groups <= workers && 2 * rest <= workers) ? static_cast<int>(rest) : 0;
}

// Fills the tiling of a launch into p (tiles_m, group_m, tile_n, tiles_n, wide_tiles, split, full_tiles,
// total_items, out_n) for `workers` persistent CTAs (CTA pairs for kCtas == 2). p.tile_n > 0 on entry
// forces that width (a schedule); num_outputs > 1 is the gathering form.
template <int kCtas, int kMode>
void plan_tiles(GemmParams& p, int num_outputs, long long workers) {
  using Cfg = GemmConfig<kCtas, kMode>;
  p.tiles_m = (p.m + Cfg::kBlockM * kCtas - 1) / (Cfg::kBlockM * kCtas);
  // Tile width and last-wave slicing. The persistent grid works through the tiles in waves of `workers`
  // equally long tiles, so the time is about waves x (tile width + a per-tile overhead worth ~9 columns).
  // Two remedies for a mostly empty last wave, both chosen here from that model: a narrower tile (224 or
  // 192 accumulator columns) that packs the work into fuller waves, and cutting the last wave's tiles
  // into 2 or 4 column slices when those fit into one pass over the workers (measured: a half slice lasts
  // ~0.6 and a quarter slice ~0.5 of a whole tile, ~0.8 in the grouped form: the MMAs take about N/2 cycles
  // but the slice still streams all of A through a ring sized for whole tiles).
  // The 224-wide tile runs ~3 % below the line (its last 64-column box straddles the tile edge and
  // leaves through direct stores) and cannot be sliced (112 is not a multiple of 32). Ties go to the
  // wider tile. A schedule can force the width; the biased form keeps 248 channels + 8 ones rows,
  // unsliced; the gathering form needs whole 64-column boxes (256 or 192 wide, slices of 128 or 64).
  int tile_n = 256, split = 1;
  double best = 1e300;
  const bool forced = p.tile_n > 0 && num_outputs <= 1;
  p.out_n = kMode == kModeSwiGLU ? p.n / 2 : p.n;
  if (kMode == kModeBiased) {
    tile_n = Cfg::kChannelsPerTile;
  } else if (kMode == kModeSwiGLU) {
    tile_n = 256;   // a tile is 128 gate channels and their 128 up channels: whole, unsliced tiles only
  } else {
    for (int cand = 256; cand >= 192; cand -= 32) {
      if (forced && cand != p.tile_n) continue;
      if (cand % 64 != 0 && num_outputs > 1) continue;
      const long long tiles = static_cast<long long>(p.tiles_m) * ((p.n + cand - 1) / cand);
      const long long full = tiles / workers, rest = tiles % workers;
      for (int s = 1; s <= 4; s *= 2) {
        const int width = cand / s;
        if (s > 1 && (rest == 0 || rest * s > workers || width % 32 != 0 || (num_outputs > 1 && width % 64 != 0))) continue;
        const double tail = rest == 0 ? 0.0 : s == 1 ? 1.0 : kMode == kModeGrouped ? 0.8 : s == 2 ? 0.6 : 0.5;
        const double cost = (static_cast<double>(full) + tail) * (cand + 9) * (cand == 224 ? 1.03 : 1.0);
        if (cost < best * 0.999) { best = cost; tile_n = cand; split = s; }
      }
    }
  }
  // Third remedy, mixed widths: cut every row stripe's channels (in units of 32) into `count` tiles whose
  // widths differ by at most one unit (192 / 224 / 256 columns), with `count` such that the tiles fill
  // whole waves. The load of the busiest worker is found by walking the kernel's own item order. Taken
  // only when it beats the uniform choices by 3 % in the model; one local destination only (a 64-column
  // store box must not straddle tiles of the gathering form), no forced schedule, and only for
  // problems of a few waves (beyond that a partial last wave is noise, and the walk would cost time).
  int mixed_count = 0, mixed_base = 0, mixed_wide = 0;
  // rows of A per raster group: about 32 MiB of activations, so they stay in L2
  // (every raster group streams the whole of W once, so the groups are made equal: 16 row tiles under a cap
  // of 7 become two groups of 8, not 7 + 7 + 2)
  const long long group_rows = raster_bytes() / (static_cast<long long>(p.k) * p.groups);
  int cap_m = static_cast<int>(group_rows / (Cfg::kBlockM * kCtas));
  if (cap_m < 1) cap_m = 1;
  const int raster_groups = (p.tiles_m + cap_m - 1) / cap_m;
  p.group_m = (p.tiles_m + raster_groups - 1) / raster_groups;
  if ((kMode == kModeFused || kMode == kModeWorkspace || kMode == kModeGrouped) && num_outputs <= 1 && !forced &&
      workers <= 256) {
    // the decision depends on the shape only: remember the last one per thread
    struct Memo { int m, n, group_m, workers, count, base, wide; };
    thread_local Memo memo = {0, 0, 0, 0, 0, 0, 0};
    if (memo.m == p.m && memo.n == p.n && memo.group_m == p.group_m && memo.workers == workers) {
      mixed_count = memo.count; mixed_base = memo.base; mixed_wide = memo.wide;
    } else {
      const int units = (p.n + 31) / 32;
      double best_mixed = 1e300;
      for (int count = (units + 7) / 8; count <= units / 6; ++count) {
        const int base = units / count, wide = units % count;
        const long long tiles = static_cast<long long>(p.tiles_m) * count;
        if (wide == 0 || base + 1 > 8 || tiles > 12 * workers) continue;   // uniform widths are covered above
        GemmParams trial = p;
        trial.tile_n = base * 32; trial.tiles_n = count; trial.wide_tiles = wide;
        trial.split = 1; trial.full_tiles = trial.total_items = static_cast<int>(tiles);
        double load[256] = {};
        double busiest = 0.0;
        for (int item = 0; item < trial.total_items; ++item) {
          int mt, nt, n_start, n_width;
          bool alt;
          tile_coords(trial, item, mt, nt, n_start, n_width, alt);
          // a tile that is not a whole number of 64-column boxes pays the 224-wide tile's 3 %
          double& mine = load[item % workers];
          mine += (n_width + 9) * (n_width % 64 ? 1.03 : 1.0);
          if (mine > busiest) busiest = mine;
        }
        if (busiest < best_mixed * 0.999) { best_mixed = busiest; mixed_count = count; mixed_base = base * 32; mixed_wide = wide; }
      }
      if (best_mixed >= best * 0.97) mixed_count = 0;
      memo = Memo{p.m, p.n, p.group_m, static_cast<int>(workers), mixed_count, mixed_base, mixed_wide};
    }
  }
  p.wide_tiles = 0;
  if (mixed_count > 0) {
    tile_n = mixed_base;
    split = 1;
    p.wide_tiles = mixed_wide;
  }
  // Fourth remedy, grouped form only, when the caller has lent a workspace (p.terms): 256-wide tiles, the
  // leftover tiles cut along the groups into pieces that all run at once.
  const int leftover = (kMode == kModeGrouped && kCtas == 2 && p.terms) ? grouped_leftover_tiles(p.m, p.n, p.groups, workers) : 0;
  p.piece_items = 0;
  if (leftover > 0) {
    tile_n = 256;
    split = 1;
    p.wide_tiles = 0;
    mixed_count = 0;
  }
  p.tile_n = tile_n;
  p.tiles_n = mixed_count > 0 ? mixed_count : (p.n + tile_n - 1) / tile_n;
  {
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    p.split = split;
    p.full_tiles = split > 1 ? static_cast<int>(tiles - tiles % workers) : static_cast<int>(tiles);
    p.total_items = p.full_tiles + static_cast<int>(tiles - p.full_tiles) * split;
    if (leftover > 0) {
      p.full_tiles = static_cast<int>(tiles - leftover);
      p.piece_items = leftover * p.groups;
      p.total_items = p.full_tiles + p.piece_items;
    }
  }
}

// `outputs` lists every destination of the BF16 result (this GPU's buffer and, for the gathering
// form, the matching block in each peer's buffer). When the row pitch allows it they are written
// with TMA tile stores; otherwise the single local output takes the direct-store path.
template <int kCtas, int kMode>
cudaError_t launch_gemm(const void* a, const void* w, const GemmParams& base, cudaStream_t stream,
                        void* const* outputs = nullptr, int num_outputs = 0, void* const* signals = nullptr,
                        void* state = nullptr, int source = 0) {
  using Cfg = GemmConfig<kCtas, kMode>;
  static std::atomic<uint64_t> smem_done{0};
  auto kernel = gemm_i8_kernel<kCtas, kMode>;
  cudaError_t err = ensure_smem(kernel, Cfg::kSmemBytes, smem_done);
  if (err != cudaSuccess) return err;

  GemmParams p = base;
  const int sms = sm_count();
  plan_tiles<kCtas, kMode>(p, num_outputs, kCtas == 2 ? sms / 2 : sms);
  const int tile_n = p.tile_n;
  // biased form: the CTA that holds the ones rows loads kBRowsLoad channels; in a pair the first CTA loads
  // kBRowsSmem through map_w and the second kBRowsLoad through the second map
  const int w_box_rows = kMode == kModeBiased ? (kCtas == 2 ? Cfg::kBRowsSmem : Cfg::kBRowsLoad) : tile_n / kCtas;
  p.stage_tx = Cfg::kABytes + w_box_rows * Cfg::kBlockK;
  CUtensorMap map_a, map_w, map_w_slice;
  err = make_map(&map_a, a, static_cast<uint64_t>(p.m) * p.groups, p.k, Cfg::kBlockM);
  if (err != cudaSuccess) return err;
  err = make_map(&map_w, w, p.n, static_cast<uint64_t>(p.k) * p.groups, w_box_rows);
  if (err != cudaSuccess) return err;
  // the second weight box: a column slice of the last wave's tiles, or the wider tiles of the mixed form
  const int slice_box_rows = kMode == kModeBiased ? Cfg::kBRowsLoad
                             : p.wide_tiles > 0   ? (tile_n + 32) / kCtas
                             : p.split > 1        ? tile_n / p.split / kCtas
                                                  : w_box_rows;
  p.stage_tx_slice = Cfg::kABytes + slice_box_rows * Cfg::kBlockK;
  err = make_map(&map_w_slice, w, p.n, static_cast<uint64_t>(p.k) * p.groups, slice_box_rows);
  if (err != cudaSuccess) return err;
  OutputMaps out_maps = {};
  void* local_only[1] = {p.out};
  if (!outputs) {
    outputs = local_only;
    num_outputs = 1;
  }
  bool tile_stores = p.out_n % 8 == 0 && num_outputs <= kMaxOutputs;
  for (int d = 0; d < num_outputs; ++d) tile_stores = tile_stores && aligned(outputs[d], 16);
  p.num_outputs = 0;
  if (tile_stores) {
    for (int d = 0; d < num_outputs; ++d) {
      err = make_output_map(&out_maps.map[d], outputs[d], p.m, p.out_n);
      if (err != cudaSuccess) return err;
    }
    p.num_outputs = num_outputs;
    if (signals && state) {
      // the gathering form closes with the in-kernel rendezvous over these counters
      for (int d = 0; d < num_outputs; ++d) out_maps.signal[d] = static_cast<unsigned long long*>(signals[d]);
      out_maps.state = static_cast<unsigned long long*>(state);
      out_maps.source = source;
    }
  } else if (num_outputs != 1 || kMode == kModeSwiGLU) {
    return cudaErrorInvalidValue;   // several destinations, and the SwiGLU form, need the tile-store path
  }

  if (kMode == kModeWorkspace && p.workspace && p.n % 4 == 0 && aligned(p.workspace, 16)) {
    EncodeTiled encode = encode_tiled_fn();
    if (!encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.n), static_cast<cuuint64_t>(p.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.n) * 4};
    const cuuint32_t box[2] = {32u, 32u};
    const cuuint32_t elem[2] = {1u, 1u};
    const CUresult r = encode(&out_maps.ws_map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, p.workspace, dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    out_maps.has_ws_map = 1;
  }

  const long long tiles = p.total_items;
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  if (kCtas == 2) {
    const long long clusters = tiles < sms / 2 ? tiles : sms / 2;
    config.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.numAttrs = 2;
  } else {
    config.gridDim = dim3(static_cast<unsigned>(tiles < sms ? tiles : sms));
  }
  config.blockDim = dim3(Cfg::kThreads);
  config.dynamicSmemBytes = Cfg::kSmemBytes;
  config.stream = stream;
  return cudaLaunchKernelEx(&config, kernel, map_a, map_w, map_w_slice, out_maps, p);
}

// Launch with programmatic stream serialization: the kernel may become resident while the kernel
// before it in the stream drains; every kernel launched this way calls griddepcontrol.wait before
// its first access to global memory.
template <typename... Params, typename... Args>
cudaError_t launch_serialized(void (*kernel)(Params...), unsigned grid, unsigned block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.gridDim = dim3(grid);
  config.blockDim = dim3(block);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  config.attrs = attr;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// ------------------------------------------------------------------ streaming-kernel (M <= 64) launch
// Picks the split-K factor and the slab width (channels per CTA, a multiple of 16: kind::i8 takes N in
// steps of 16 above 32) from a small time model fitted to measurements on B200, in microseconds:
//   fixed(split) + 4 (waves - 1) + max(weight bytes / HBM rate, waves * K blocks per CTA * time per ring stage)
// where a ring stage (slab x 128 weight bytes + the 2 or 8 KB activation tile) takes at least 0.17 us
// (barrier round trip, TMA and MMA issue) and one SM pulls at most about 75 GB/s. Split-K shortens the
// per-CTA stream but costs a cluster launch and the shared-memory reduction. Clusters of four lose
// a few SMs to placement (a cluster sits inside one GPC). Ties go to the smaller split and slab.
// M <= 16: from this slab width on (four 32-channel chunks) the activation box is loaded four times so
// that eight warps instead of two share the epilogue; measured 29.1 vs 30.6 us on N=34816, K=5120, and
// slower for narrow slabs, whose stages are small against the three extra loads.
constexpr int kReplicateFromSlab = 128;

void choose_decode_shape(int n, int k, int rows, int max_split, int sms, int* split_out, int* slab_out) {
  const int num_kb = (k + 127) / 128;
  const double hbm_us = static_cast<double>(n) * k / 6.4e6;
  double best = 1e300;
  int best_split = 1, best_slab = 128;
  for (int split = 1; split <= max_split; split *= 2) {
    if (split > num_kb) break;
    const long long capacity = split == 4 ? (sms / 4 - 4) * 4 : split == 2 ? (sms / 2) * 2 : sms;
    const double fixed_us = split == 1 ? 4.5 : split == 2 ? 5.0 : 5.8;
    for (int slab = 16; slab <= 256; slab += 16) {
      const long long slabs = (n + slab - 1) / slab;
      const long long ctas = slabs * split;
      const long long waves = (ctas + capacity - 1) / capacity;
      // M <= 16 with a wide slab uses the replicated 64-row tile (see launch_decode)
      const double stage_bytes = (slab + (rows == 16 && slab >= kReplicateFromSlab ? 64 : rows)) * 128.0;
      const double stage_us = stage_bytes / 75e3 > 0.17 ? stage_bytes / 75e3 : 0.17;
      const double stream_us = static_cast<double>(waves) * ((num_kb + split - 1) / split) * stage_us;
      const double cost = fixed_us + 4.0 * (waves - 1) + (stream_us > hbm_us ? stream_us : hbm_us);
      if (cost < best * 0.995) { best = cost; best_split = split; best_slab = slab; }
    }
  }
  *split_out = best_split;
  *slab_out = best_slab;
}

template <int kSplit, bool kBiased, int kRows, int kDataRows = kRows, bool kDynamic = false>
cudaError_t launch_decode_variant(const void* a, const void* w, const DecodeParams& p, cudaStream_t stream) {
  using Cfg = DecodeConfig<kSplit, kRows, kDataRows, kDynamic>;
  static std::atomic<uint64_t> smem_done{0};
  auto kernel = decode_w8a8_kernel<kSplit, kBiased, kRows, kDataRows, kDynamic>;
  cudaError_t err = ensure_smem(kernel, Cfg::kSmemBytes, smem_done);
  if (err != cudaSuccess) return err;
  CUtensorMap map_w, map_a;
  err = make_map(&map_w, w, p.n, p.k, p.slab);
  if (err != cudaSuccess) return err;
  // the dynamic form reads the BF16 activations (64-column boxes); the others the INT8 codes
  err = kDynamic ? make_bf16_map(&map_a, p.x, p.m, p.k, 64, 16) : make_map(&map_a, a, p.m, p.k, Cfg::kDataRows);
  if (err != cudaSuccess) return err;
  const int slabs = (p.n + p.slab - 1) / p.slab;
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attr[2];
  config.gridDim = dim3(static_cast<unsigned>(slabs * kSplit));
  config.blockDim = dim3(Cfg::kThreads);
  config.dynamicSmemBytes = Cfg::kSmemBytes;
  config.stream = stream;
  // the kernel's prologue (barriers, TMEM, descriptor prefetch) may overlap the tail of the kernel
  // before it in the stream; it calls griddepcontrol.wait before touching global memory
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  if (kSplit > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = kSplit;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&config, kernel, map_w, map_a, p);
}

// Rows the streaming kernel takes: up to 16 with any split, up to 64 with a split of at most two
// (the shared-memory reduce buffer grows with the rows).
constexpr int kDecodeMaxRows = 64;

template <bool kBiased>
cudaError_t launch_decode(const void* a, const void* w, DecodeParams p, int forced_split, cudaStream_t stream) {
  const bool wide = p.m > 16;
  const int max_split = wide ? 2 : 4;
  if (forced_split > max_split) return cudaErrorInvalidValue;
  int split = 1, slab = 128;
  choose_decode_shape(p.n, p.k, wide ? 64 : 16, max_split, sm_count(), &split, &slab);
  if (forced_split > 0) {
    split = forced_split;
    const int per = sm_count() / split > 0 ? sm_count() / split : 1;
    slab = ((p.n + per - 1) / per + 15) / 16 * 16;
    if (slab < 16) slab = 16;
    if (slab > 256) slab = 256;
  }
  if (slab < 16 || slab > 256 || slab % 16 != 0) return cudaErrorInvalidValue;   // not an instruction shape
  p.slab = slab;
  if (wide) {
    return split == 1 ? launch_decode_variant<1, kBiased, 64>(a, w, p, stream)
                      : launch_decode_variant<2, kBiased, 64>(a, w, p, stream);
  }
  if (slab >= kReplicateFromSlab) {
    switch (split) {
      case 1: return launch_decode_variant<1, kBiased, 64, 16>(a, w, p, stream);
      case 2: return launch_decode_variant<2, kBiased, 64, 16>(a, w, p, stream);
      default: return launch_decode_variant<4, kBiased, 64, 16>(a, w, p, stream);
    }
  }
  switch (split) {
    case 1: return launch_decode_variant<1, kBiased, 16>(a, w, p, stream);
    case 2: return launch_decode_variant<2, kBiased, 16>(a, w, p, stream);
    default: return launch_decode_variant<4, kBiased, 16>(a, w, p, stream);
  }
}

bool gemm_geometry_ok(int m, int n, int k) {
  return m > 0 && n > 0 && k > 0 && k % 32 == 0 && k <= 65536 &&
         static_cast<long long>(m) * k <= INT32_MAX && static_cast<long long>(n) * k <= INT32_MAX;
}

// ------------------------------------------------------------------ quantizer launch
template <int kTeam, int kPacks, bool kSwiGLU = false>
void launch_quantize_vec(const void* x, int8_t* q, float* s, int rows, int k, int m, int groups, cudaStream_t stream) {
  constexpr int kThreads = kTeam > 256 ? kTeam : 256;
  constexpr int kRowsPerCta = kThreads / kTeam;
  // persistent grid: as many CTAs as fit on the device at once (cached per device), capped by the work
  static std::atomic<int> resident[kMaxDevices];
  int device = 0;
  cudaGetDevice(&device);
  device = device >= 0 && device < kMaxDevices ? device : 0;
  int per_device = resident[device].load(std::memory_order_relaxed);
  if (per_device == 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_rows_vec_kernel<kTeam, kPacks, kSwiGLU>, kThreads, 0) !=
            cudaSuccess || per_sm < 1)
      per_sm = 1;
    per_device = per_sm * sm_count();
    resident[device].store(per_device, std::memory_order_relaxed);
  }
  const int needed = (rows + kRowsPerCta - 1) / kRowsPerCta;
  constexpr bool kPersistent = !kSwiGLU && kPacks >= 4 && kPacks <= 9;
  // (making every CTA of the persistent form walk the same number of rows, 512 CTAs x 4 passes instead of
  // 592 CTAs x 3.46, was measured 20-25 % SLOWER: the kernel lives on the number of loads in flight)
  const int grid = (!kPersistent || needed < per_device) ? needed : per_device;
  launch_serialized(quantize_rows_vec_kernel<kTeam, kPacks, kSwiGLU>, static_cast<unsigned>(grid), kThreads, 0,
                    stream, static_cast<const uint16_t*>(x), q, s, rows, k, m, groups);
}

// rows = output rows; groups == 0 for the plain form.
cudaError_t launch_quantize(const void* x, int8_t* q, float* s, int rows, int k, int m, int groups,
                            cudaStream_t stream) {
  const bool vector_ok = k % 8 == 0 && aligned(x, 16) && aligned(q, 8);
  const int packs = k / 8;
  if (vector_ok && packs <= 32 * 4 && rows >= 64) {
    // narrow rows (K <= 1024): one warp per row, eight rows per CTA
    const int per_lane = (packs + 31) / 32;
#define CI8_WARP(P) launch_quantize_vec<32, P>(x, q, s, rows, k, m, groups, stream)
    if (per_lane <= 1) CI8_WARP(1);
    else if (per_lane <= 2) CI8_WARP(2);
    else CI8_WARP(4);
#undef CI8_WARP
  } else if (vector_ok && packs <= 128 * 8) {
    // rows up to K = 8192: 128 threads per row, two rows per CTA, no idle pack slots at K = 4096 / 5120
    const int per_thread = (packs + 127) / 128;
#define CI8_HALF(P) launch_quantize_vec<128, P>(x, q, s, rows, k, m, groups, stream)
    if (per_thread <= 1) CI8_HALF(1);
    else if (per_thread <= 2) CI8_HALF(2);
    else if (per_thread <= 3) CI8_HALF(3);
    else if (per_thread <= 4) CI8_HALF(4);
    else if (per_thread <= 5) CI8_HALF(5);
    else if (per_thread <= 6) CI8_HALF(6);
    else CI8_HALF(8);
#undef CI8_HALF
  } else if (vector_ok && packs <= 256 * 32) {
    // one 256-thread CTA per row
    const int per_thread = (packs + 255) / 256;
#define CI8_CTA(P) launch_quantize_vec<256, P>(x, q, s, rows, k, m, groups, stream)
    if (per_thread <= 5) CI8_CTA(5);
    else if (per_thread <= 6) CI8_CTA(6);
    else if (per_thread <= 9) CI8_CTA(9);
    else if (per_thread <= 12) CI8_CTA(12);
    else if (per_thread <= 16) CI8_CTA(16);
    else if (per_thread <= 24) CI8_CTA(24);
    else CI8_CTA(32);
#undef CI8_CTA
  } else {
    if (groups > 0) return cudaErrorInvalidValue;   // the grouped form requires aligned buffers
    quantize_rows_generic_kernel<<<rows, 256, 0, stream>>>(static_cast<const uint16_t*>(x), q, s, k);
  }
  return cudaGetLastError();
}

// silu_mul_quantize: rows of [gate(k) | up(k)]; one 256-thread CTA per row.
cudaError_t launch_swiglu_quantize(const void* x, int8_t* q, float* s, int m, int k, cudaStream_t stream) {
  // the SwiGLU is arithmetic-heavy (expf, a division), so rows are spread over 512 threads to keep
  // twice as many warps resident as the plain quantizer would
  const int packs = k / 8;
#define CI8_SWIGLU(T, P) launch_quantize_vec<T, P, true>(x, q, s, m, k, m, 0, stream)
  if (packs <= 256) CI8_SWIGLU(256, 1);
  else if (packs <= 512) CI8_SWIGLU(512, 1);
  else if (packs <= 1024) CI8_SWIGLU(512, 2);
  else if (packs <= 1536) CI8_SWIGLU(512, 3);
  else if (packs <= 2560) CI8_SWIGLU(512, 5);
  else if (packs <= 4608) CI8_SWIGLU(512, 9);
  else CI8_SWIGLU(512, 16);
#undef CI8_SWIGLU
  return cudaGetLastError();
}

template <int kRows>
cudaError_t launch_gemv(const void* x, const int8_t* w, const void* sw, void* out, int m, int n, int k,
                        cudaStream_t stream) {
  constexpr int kChannels = kRows <= 4 ? 4 : 2;
  constexpr int kSmem = kRows * kGemvChunk * 2;
  static std::atomic<uint64_t> smem_done{0};
  auto kernel = gemv_w8a16_kernel<kRows, kChannels>;
  cudaError_t err = ensure_smem(kernel, kSmem, smem_done);
  if (err != cudaSuccess) return err;
  const int per_cta = 8 * kChannels;
  kernel<<<(n + per_cta - 1) / per_cta, 256, kSmem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), w, static_cast<const __nv_bfloat16*>(sw),
      static_cast<__nv_bfloat16*>(out), m, n, k);
  return cudaGetLastError();
}

// channel_mm for operands that are only 4-byte aligned (a view at an odd offset into a larger
// buffer): TMA needs 16-byte aligned bases, the reference's kernel reads 32-bit words and accepts
// such operands, so this plain kernel does too. One warp per (row, eight channels): the lanes walk K
// in 32-bit words, dp4a on the activation word and the eight weight words (code+128 turned into the
// signed code by flipping the top bit of every byte), a shuffle tree, the usual epilogue. Integer
// sums are exact, so the result has the same bits as the tensor-core path. Slow, and only chosen
// when the fast path cannot take the pointers.
__global__ void __launch_bounds__(256)
channel_mm_words_kernel(const int8_t* __restrict__ a, const uint8_t* __restrict__ w, const float* __restrict__ sa,
                        const __nv_bfloat16* __restrict__ sw, __nv_bfloat16* __restrict__ out, int m, int n, int k) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int groups = (n + 7) / 8;
  const int row = static_cast<int>(warp / groups);
  const int c0 = static_cast<int>(warp % groups) * 8;
  if (row >= m) return;
  const int* a_words = reinterpret_cast<const int*>(a + static_cast<size_t>(row) * k);
  int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int word = lane; word < k / 4; word += 32) {
    const int av = __ldg(a_words + word);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 + j < n) {
        const unsigned wv = __ldg(reinterpret_cast<const unsigned*>(w + static_cast<size_t>(c0 + j) * k) + word);
        acc[j] = __dp4a(av, static_cast<int>(wv ^ 0x80808080u), acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], offset);
  if (lane < 8 && c0 + lane < n) {
    int mine = acc[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mine = lane == j ? acc[j] : mine;
    const float scaled = __fmul_rn(__fmul_rn(__int2float_rn(mine), sa[row]), __bfloat162float(sw[c0 + lane]));
    out[static_cast<size_t>(row) * n + c0 + lane] = __float2bfloat16_rn(scaled);
  }
}

// Moves the device status word into a caller-owned word on the stream (and clears it), so that a
// captured graph can carry the check: bits are ORed into *word, which may be device memory or pinned,
// device-mapped host memory that the host polls and clears at its leisure.
__global__ void status_to_word_kernel(unsigned* word) {
  const unsigned bits = atomicExch(&g_ci8_status, 0u);
  if (bits) {
    atomicOr_system(word, bits);
    __threadfence_system();
  }
}

// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever arrives on. The
// wait gives up after `deadline_ns`, raises the status bit and the kernel returns normally.
__global__ void wait_timeout_selftest_kernel(unsigned long long deadline_ns, int* gave_up) {
  __shared__ alignas(8) unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&barrier), 1);
    fence_barrier_init();
    const bool completed = mbar_wait(smem_u32(&barrier), 0u, &abort_flag, deadline_ns);
    *gave_up = completed ? 0 : 1;
  }
}

// The same for a rendezvous between the CTAs of a cluster: CTA 0 of a pair waits on a barrier that CTA 1
// is supposed to arrive on remotely and, in this self-test, never does. The wait gives up after
// `deadline_ns` and raises the cluster status bit; the closing cluster barrier keeps CTA 1 around
// until then, as the split-K kernel's teardown does.
__global__ void __cluster_dims__(2, 1, 1) cluster_timeout_selftest_kernel(unsigned long long deadline_ns, int* gave_up) {
  __shared__ alignas(8) unsigned long long barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&barrier), 1);
    fence_barrier_init();
  }
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (cluster_ctarank() == 0 && threadIdx.x == 0) {
    const bool completed = mbar_wait<true, kStatusClusterTimeout>(smem_u32(&barrier), 0u, &abort_flag, deadline_ns);
    *gave_up = completed ? 0 : 1;
  }
  cluster_arrive();
  cluster_wait();
}

// Cross-GPU rendezvous as a kernel of its own (one thread): everything this GPU's earlier kernels in the
// stream wrote into its peers' memory is complete when this kernel starts; it tells every peer so
// (one arrival counter per source rank in each peer's memory) and waits until every peer has told it
// the same. The call counter lives in `state`, so the kernel can be replayed from a CUDA graph.
struct RendezvousParams {
  unsigned long long* signal[ci8::kMaxOutputs];   // signal[r]: rank r's counters (peer-mapped); [rank] is this GPU's own
  unsigned long long* state;
  int world, rank;
};
__global__ void peer_rendezvous_kernel(const RendezvousParams p) {
  if (threadIdx.x != 0) return;
  const unsigned long long calls_done = ld_relaxed_u64(p.state);
  __threadfence_system();
  for (int d = 1; d < p.world; ++d) red_release_sys_add_u64(p.signal[(p.rank + d) % p.world] + p.rank, 1ull);
  const unsigned long long start = global_timer_ns();
  for (int from = 0; from < p.world; ++from) {
    if (from == p.rank) continue;
    for (uint32_t spin = 1; ld_acquire_sys_u64(p.signal[p.rank] + from) < calls_done + 1ull; ++spin) {
      __nanosleep(32);
      if ((spin & 255u) == 0u && global_timer_ns() - start > kWaitDeadlineNs) {
        atomicOr(&g_ci8_status, kStatusPeerTimeout);
        from = p.world;
        break;
      }
    }
  }
  __threadfence();
  st_relaxed_u64(p.state, calls_done + 1ull);
}

}  // namespace

// ------------------------------------------------------------------ block-32 (Q8_0) launch
template <int kTileN>
cudaError_t launch_q8_block_mm(const int8_t* a, const float* sa, const int8_t* w, const void* sw, void* y, int m, int n,
                               int k, cudaStream_t stream) {
  using Cfg = Q8BlockConfig<kTileN>;
  static std::atomic<uint64_t> smem_done{0};
  cudaError_t err = ensure_smem(q8_block_mm_kernel<kTileN>, Cfg::kSmemBytes, smem_done);
  if (err != cudaSuccess) return err;
  Q8BlockParams p{sa, static_cast<const __half*>(sw), static_cast<__nv_bfloat16*>(y), m, n, k, 0, 0};
  p.tiles_m = (m + Cfg::kBlockM - 1) / Cfg::kBlockM;
  p.tiles_n = (n + Cfg::kTileN - 1) / Cfg::kTileN;
  CUtensorMap map_a, map_w;
  err = make_map(&map_a, a, m, k, Cfg::kBlockM);
  if (err != cudaSuccess) return err;
  err = make_map(&map_w, w, n, k, Cfg::kTileN);
  if (err != cudaSuccess) return err;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  const int sms = sm_count();
  return launch_serialized(q8_block_mm_kernel<kTileN>, static_cast<unsigned>(tiles < sms ? tiles : sms), Cfg::kThreads,
                           Cfg::kSmemBytes, stream, map_a, map_w, p);
}

// Channels per tile of the block-32 kernel: a tile's time is its epilogue's (the FP32 rescale of every 32-deep
// partial sum), and the persistent grid runs the tiles in waves of one per SM. Measured on M=4096, N=1024,
// K=4096: four waves of 64-wide tiles 121 us, seven waves of 32-wide ones 135 us, so a wave of width w costs about
// w + 24 (per stage the barrier round trips, the scale hand-over and the accumulator loads do not shrink with
// the width). Narrow tiles pay where the wide one leaves SMs without work: M=16, N=1024 32.0 -> 19.4 us with
// 16-wide tiles on 64 SMs instead of 64-wide ones on 16. Ties go to the wider tile, which loads A less often.
int q8_block_tile_channels(int m, int n) {
  const long long tiles_m = (m + 127) / 128, sms = sm_count();
  int best = 64;
  long long best_cost = 0;
  for (int width = 64; width >= 16; width /= 2) {
    const long long tiles = tiles_m * ((n + width - 1) / width);
    const long long cost = ((tiles + sms - 1) / sms) * (width + 24);
    if (width == 64 || cost * 100 < best_cost * 97) { best = width; best_cost = cost; }
  }
  return best;
}

cudaError_t launch_q8_block(const void* x, int8_t* a, float* sa, const int8_t* w, const void* sw, void* y, int m,
                            int n, int k, cudaStream_t stream) {
  const long long blocks = static_cast<long long>(m) * (k / 32);
  cudaError_t err = launch_serialized(q8_block_quantize_kernel, static_cast<unsigned>((blocks + 255) / 256), 256, 0, stream,
                                      static_cast<const uint16_t*>(x), a, sa, static_cast<int64_t>(blocks));
  if (err != cudaSuccess) return err;
  switch (q8_block_tile_channels(m, n)) {
    case 16: return launch_q8_block_mm<16>(a, sa, w, sw, y, m, n, k, stream);
    case 32: return launch_q8_block_mm<32>(a, sa, w, sw, y, m, n, k, stream);
    default: return launch_q8_block_mm<64>(a, sa, w, sw, y, m, n, k, stream);
  }
}

// ------------------------------------------------------------------ block-32 with built-in scratch
// Scratch of ci8_q8_block_mm_static: the activation codes (one byte per value) followed, at a fixed
// offset, by their FP32 block scales (one per 32 values). It is part of the library image, so every
// GPU that loads libci8.so carries these 4.5 MiB until the process exits.
constexpr long long kQ8StaticMaxValues = 4ll << 20;                      // m * k of one call
constexpr long long kQ8StaticScaleOffset = kQ8StaticMaxValues;           // bytes; a multiple of 256
constexpr long long kQ8StaticBytes = kQ8StaticMaxValues + kQ8StaticMaxValues / 32 * 4;
static __device__ __align__(256) unsigned char g_q8_static_scratch[kQ8StaticBytes];

// Device address of the scratch on the current device. In host code `g_q8_static_scratch` is only a
// handle for the runtime, not an address a kernel (or a tensor map) could use, so the address is asked
// for once per device, with that device current, and remembered.
cudaError_t q8_static_scratch(unsigned char** out) {
  static std::atomic<unsigned char*> cached[kMaxDevices];
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  unsigned char* address = cached[device].load(std::memory_order_acquire);
  if (!address) {
    void* looked_up = nullptr;
    err = cudaGetSymbolAddress(&looked_up, g_q8_static_scratch);
    if (err != cudaSuccess) return err;
    if (!looked_up) return cudaErrorInvalidSymbol;
    address = static_cast<unsigned char*>(looked_up);
    cached[device].store(address, std::memory_order_release);
  }
  *out = address;
  return cudaSuccess;
}

// ====================================================================== C ABI
extern "C" {

int ci8_abi_version(void) { return 2; }

const char* ci8_error_string(int code) {
  return code == 0 ? "success" : cudaGetErrorString(static_cast<cudaError_t>(code));
}

int ci8_device_status(unsigned* status) {
  if (!status) return kInvalid;
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess) return err;
  err = cudaMemcpyFromSymbol(status, ci8::g_ci8_status, sizeof(unsigned));
  if (err != cudaSuccess) return err;
  const unsigned zero = 0;
  return cudaMemcpyToSymbol(ci8::g_ci8_status, &zero, sizeof(unsigned));
}

int ci8_device_status_async(unsigned* word, ci8_stream_t stream) {
  if (!word || !aligned(word, 4)) return kInvalid;
  status_to_word_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(word);
  return cudaGetLastError();
}

int ci8_quantize_rows(const void* x, int8_t* codes, float* scales, int m, int k, ci8_stream_t stream) {
  if (!x || !codes || !scales || m <= 0 || k <= 0 || static_cast<long long>(m) * k > INT32_MAX) return kInvalid;
  return launch_quantize(x, codes, scales, m, k, m, 0, reinterpret_cast<cudaStream_t>(stream));
}

int ci8_quantize_grouped4096(const void* x, int8_t* codes, float* scales, int m, int groups,
                             ci8_stream_t stream) {
  if (m < 0 || groups <= 0 || static_cast<long long>(m) * groups * 4096 > INT32_MAX) return kInvalid;
  if (m == 0) return 0;
  if (!x || !codes || !scales || !aligned(x, 16) || !aligned(codes, 8) || !aligned(scales, 4)) return kInvalid;
  return launch_quantize(x, codes, scales, m * groups, 4096, m, groups, reinterpret_cast<cudaStream_t>(stream));
}

int ci8_unpack_allspark(const uint8_t* packed, const void* packed_scales, int8_t* weight, void* scales, int n,
                        int k, ci8_stream_t stream) {
  if (!packed || !packed_scales || !weight || !scales || n <= 0 || n % 16 != 0 || k <= 0 || k > 65536 ||
      k % 16 != 0 || static_cast<long long>((n + 31) / 32 * 32) * k > INT32_MAX || !aligned(packed, 16) ||
      !aligned(weight, 16))
    return kInvalid;
  const long long cells = static_cast<long long>((n + 31) / 32 * 8) * (k / 16);
  unpack_allspark_kernel<<<static_cast<unsigned>((cells + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      packed, static_cast<const uint16_t*>(packed_scales), weight, static_cast<uint16_t*>(scales), n, k);
  return cudaGetLastError();
}

int ci8_silu_mul(const void* x, void* out, int m, int k, ci8_stream_t stream) {
  if (m < 0 || k <= 0 || k % 8 != 0 || static_cast<long long>(m) * 2 * k > INT32_MAX) return kInvalid;
  if (m == 0) return 0;
  if (!x || !out || !aligned(x, 16) || !aligned(out, 16)) return kInvalid;
  const int64_t packs = static_cast<int64_t>(m) * (k / 8);
  silu_mul_kernel<<<static_cast<unsigned>((packs + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), packs, k / 8);
  return cudaGetLastError();
}

int ci8_silu_mul_quantize(const void* x, int8_t* codes, float* scales, int m, int k, ci8_stream_t stream) {
  if (m < 0 || k <= 0 || k % 8 != 0 || k > 65536 || static_cast<long long>(m) * 2 * k > INT32_MAX) return kInvalid;
  if (m == 0) return 0;
  if (!x || !codes || !scales || !aligned(x, 16) || !aligned(codes, 8)) return kInvalid;
  return launch_swiglu_quantize(x, codes, scales, m, k, reinterpret_cast<cudaStream_t>(stream));
}

int ci8_fused_channel_mm(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale,
                         void* out, int m, int n, int k, int schedule, ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !out || !gemm_geometry_ok(m, n, k) || schedule < 0 || schedule > 6 ||
      !aligned(a, 16) || !aligned(w, 16) || static_cast<long long>(m) * n > INT32_MAX)
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (m <= kDecodeMaxRows && schedule == 0) {
    DecodeParams p{a, a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out),
                   nullptr, m, n, k, 0};
    return launch_decode<false>(a, w, p, 0, s);
  }
  GemmParams p{a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), nullptr,
               m, n, k, 1, 0, 0, 0, 0, 0, 0};
  // schedule 0: pairs of CTAs once there is more than one 128-row block, tile width chosen by launch_gemm; odd values
  // force the single-CTA tile, even values the two-CTA tile; 1/2 with 256-wide tiles, 3/4 with
  // 224-wide, 5/6 with 192-wide tiles. All give identical bits.
  const bool pair = schedule == 0 ? m > 128 : (schedule % 2 == 0);
  p.tile_n = schedule == 0 ? 0 : schedule <= 2 ? 256 : schedule <= 4 ? 224 : 192;
  return pair ? launch_gemm<2, kModeFused>(a, w, p, s) : launch_gemm<1, kModeFused>(a, w, p, s);
}

int ci8_cutlass_channel_mm(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale,
                           int32_t* workspace, void* out, int m, int n, int k, ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !workspace || !out || !gemm_geometry_ok(m, n, k) || !aligned(a, 16) ||
      !aligned(w, 16) || static_cast<long long>(m) * n > INT32_MAX)
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (m <= kDecodeMaxRows) {
    DecodeParams p{a, a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out),
                   workspace, m, n, k, 0};
    return launch_decode<false>(a, w, p, 0, s);
  }
  GemmParams p{a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), workspace,
               m, n, k, 1, 0, 0, 0, 0, 0, 0};
  return m > 128 ? launch_gemm<2, kModeWorkspace>(a, w, p, s) : launch_gemm<1, kModeWorkspace>(a, w, p, s);
}

int ci8_channel_mm(const int8_t* a, const uint8_t* w, const float* a_scale, const void* w_scale, void* out,
                   int m, int n, int k, ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !out || !gemm_geometry_ok(m, n, k) || !aligned(a, 4) || !aligned(w, 4) ||
      static_cast<long long>(m) * n > INT32_MAX)
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!aligned(a, 16) || !aligned(w, 16)) {
    // operands the TMA paths cannot take (the reference accepts any 4-byte aligned pointer)
    const long long warps = static_cast<long long>(m) * ((n + 7) / 8);
    channel_mm_words_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(
        a, w, a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), m, n, k);
    return cudaGetLastError();
  }
  if (m <= kDecodeMaxRows) {
    DecodeParams p{a, a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out),
                   nullptr, m, n, k, 0};
    return launch_decode<true>(a, w, p, 0, s);
  }
  GemmParams p{a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), nullptr,
               m, n, k, 1, 0, 0, 0, 0, 0, 0};
  return m > 128 ? launch_gemm<2, kModeBiased>(a, w, p, s) : launch_gemm<1, kModeBiased>(a, w, p, s);
}

int ci8_channel_gemv(const void* x, const int8_t* w, const void* w_scale, void* out, int m, int n, int k,
                     ci8_stream_t stream) {
  if (!x || !w || !w_scale || !out || m <= 0 || m > 16 || n <= 0 || k <= 0 || k > 65536 || k % 16 != 0 ||
      static_cast<long long>(n) * k > INT32_MAX || !aligned(w, 16) || !aligned(x, 4))
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (aligned(x, 16) && n >= 2048) {
    // production path: TMA-staged weights, one CTA per slab of channels, one wave
    const int sms = sm_count();
    // slabs in steps of 16 channels, one MMA fragment (a warp of the 9..16-row form, which owns 32, may end
    // up with only its first 16 in use)
    int slab = ((n + sms - 1) / sms + 15) / 16 * 16;
    if (slab < 16) slab = 16;
    if (slab > GemvTmaConfig<1>::kMaxSlab) slab = GemvTmaConfig<1>::kMaxSlab;
    static std::atomic<uint64_t> smem_done1{0}, smem_done2{0};
    cudaError_t err = m <= 8 ? ensure_smem(gemv_w8a16_tma_kernel<1>, GemvTmaConfig<1>::kSmemBytes, smem_done1)
                             : ensure_smem(gemv_w8a16_tma_kernel<2>, GemvTmaConfig<2>::kSmemBytes, smem_done2);
    if (err != cudaSuccess) return err;
    CUtensorMap map_w, map_x;
    err = make_map(&map_w, w, n, k, slab);
    if (err != cudaSuccess) return err;
    err = make_bf16_map(&map_x, x, m, k, 64, 16);
    if (err != cudaSuccess) return err;
    const int ctas = (n + slab - 1) / slab;
    const auto* sb = static_cast<const __nv_bfloat16*>(w_scale);
    auto* ob = static_cast<__nv_bfloat16*>(out);
    if (m <= 8)
      return launch_serialized(gemv_w8a16_tma_kernel<1>, ctas, GemvTmaConfig<1>::kThreads, GemvTmaConfig<1>::kSmemBytes, s,
                               map_w, map_x, sb, ob, m, n, k, slab);
    else
      return launch_serialized(gemv_w8a16_tma_kernel<2>, ctas, GemvTmaConfig<2>::kThreads, GemvTmaConfig<2>::kSmemBytes, s,
                               map_w, map_x, sb, ob, m, n, k, slab);
    return cudaGetLastError();
  }
  if (aligned(x, 16)) {
    // register-fed tensor-core path: 64 channels per CTA, K split over four warps
    const int ctas = (n + kGemvChannelsPerCta - 1) / kGemvChannelsPerCta;
    const auto* xb = static_cast<const __nv_bfloat16*>(x);
    const auto* sb = static_cast<const __nv_bfloat16*>(w_scale);
    auto* ob = static_cast<__nv_bfloat16*>(out);
    if (m <= 8) gemv_w8a16_mma_kernel<1><<<ctas, 256, 0, s>>>(xb, w, sb, ob, m, n, k);
    else gemv_w8a16_mma_kernel<2><<<ctas, 256, 0, s>>>(xb, w, sb, ob, m, n, k);
    return cudaGetLastError();
  }
  if (m == 1) return launch_gemv<1>(x, w, w_scale, out, m, n, k, s);
  if (m == 2) return launch_gemv<2>(x, w, w_scale, out, m, n, k, s);
  if (m <= 4) return launch_gemv<4>(x, w, w_scale, out, m, n, k, s);
  if (m <= 8) return launch_gemv<8>(x, w, w_scale, out, m, n, k, s);
  return launch_gemv<16>(x, w, w_scale, out, m, n, k, s);
}

long long ci8_grouped_workspace_bytes(int m, int n, int groups) {
  if (m <= 0 || n <= 0 || groups <= 0 || groups > 16) return 0;
  const int leftover = grouped_leftover_tiles(m, n, groups, sm_count() / 2);
  return leftover > 0 ? static_cast<long long>(kPieceHeaderBytes + static_cast<size_t>(leftover) * groups * kPieceTermBytes) : 0;
}

int ci8_grouped_channel_mm_ws(const int8_t* codes, const int8_t* w, const float* scales, const void* w_scale,
                              void* out, void* workspace, long long workspace_bytes, int m, int n, int groups,
                              ci8_stream_t stream) {
  if (!codes || !w || !scales || !w_scale || !out || m <= 0 || n <= 0 || groups <= 0 || groups > 16 ||
      static_cast<long long>(m) * groups * 4096 > INT32_MAX || static_cast<long long>(n) * groups * 4096 > INT32_MAX ||
      static_cast<long long>(m) * n > INT32_MAX || !aligned(codes, 16) || !aligned(w, 16) || workspace_bytes < 0 ||
      (workspace && !aligned(workspace, 16)))
    return kInvalid;
  GemmParams p{scales, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), nullptr,
               m, n, 4096, groups, 0, 0, 0, 0, 0, 0};
  // a workspace that is large enough switches on the split of the last wave's tiles along the groups
  const long long needed = ci8_grouped_workspace_bytes(m, n, groups);
  if (workspace && needed > 0 && workspace_bytes >= needed) {
    p.piece_sync = static_cast<unsigned*>(workspace);
    p.terms = reinterpret_cast<float*>(static_cast<char*>(workspace) + kPieceHeaderBytes);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return m > 128 ? launch_gemm<2, kModeGrouped>(codes, w, p, s) : launch_gemm<1, kModeGrouped>(codes, w, p, s);
}

int ci8_grouped_channel_mm(const int8_t* codes, const int8_t* w, const float* scales, const void* w_scale,
                           void* out, int m, int n, int groups, ci8_stream_t stream) {
  return ci8_grouped_channel_mm_ws(codes, w, scales, w_scale, out, nullptr, 0, m, n, groups, stream);
}

namespace {
// Shared by the two gathering entry points. destination d = the [m, n_shard] block number `rank` of
// peer (rank + d) % world: every rank starts with its own buffer and walks the peers in a different
// order, which spreads the NVLink traffic.
int gather_impl(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale, void* const* gathered,
                void* const* signals, void* state, int world, int rank, int m, int n_shard, int k, int schedule,
                ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !gathered || world <= 0 || world > kMaxOutputs || rank < 0 ||
      rank >= world || !gemm_geometry_ok(m, n_shard, k) || n_shard % 8 != 0 || schedule < 0 || schedule > 6 ||
      !aligned(a, 16) || !aligned(w, 16) || static_cast<long long>(m) * n_shard * world > INT32_MAX)
    return kInvalid;
  void* outputs[kMaxOutputs];
  void* counters[kMaxOutputs];
  const size_t block_bytes = static_cast<size_t>(m) * n_shard * 2;
  for (int d = 0; d < world; ++d) {
    void* base = gathered[(rank + d) % world];
    if (!base || !aligned(base, 16)) return kInvalid;
    outputs[d] = static_cast<char*>(base) + block_bytes * rank;
    counters[d] = signals ? signals[(rank + d) % world] : nullptr;
    if (signals && (!counters[d] || !aligned(counters[d], 8))) return kInvalid;
  }
  GemmParams p{a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(outputs[0]), nullptr,
               m, n_shard, k, 1, 0, 0, 0, 0, 0, 0};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool pair = schedule == 0 ? m > 128 : (schedule % 2 == 0);
  void* const* sig = signals ? counters : nullptr;
  return pair ? launch_gemm<2, kModeFused>(a, w, p, s, outputs, world, sig, state, rank)
              : launch_gemm<1, kModeFused>(a, w, p, s, outputs, world, sig, state, rank);
}
}  // namespace

int ci8_fused_channel_mm_gather(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale,
                                void* const* gathered, int world, int rank, int m, int n_shard, int k,
                                int schedule, ci8_stream_t stream) {
  return gather_impl(a, w, a_scale, w_scale, gathered, nullptr, nullptr, world, rank, m, n_shard, k, schedule, stream);
}

int ci8_fused_channel_mm_gather_sync(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale,
                                     void* const* gathered, void* const* signals, void* state, int world, int rank,
                                     int m, int n_shard, int k, int schedule, ci8_stream_t stream) {
  if (!signals || !state || !aligned(state, 8)) return kInvalid;
  return gather_impl(a, w, a_scale, w_scale, gathered, signals, state, world, rank, m, n_shard, k, schedule, stream);
}

int ci8_peer_rendezvous(void* const* signals, void* state, int world, int rank, ci8_stream_t stream) {
  if (!signals || !state || !aligned(state, 8) || world <= 0 || world > kMaxOutputs || rank < 0 || rank >= world)
    return kInvalid;
  RendezvousParams p = {};
  for (int r = 0; r < world; ++r) {
    if (!signals[r] || !aligned(signals[r], 8)) return kInvalid;
    p.signal[r] = static_cast<unsigned long long*>(signals[r]);
  }
  p.state = static_cast<unsigned long long*>(state);
  p.world = world;
  p.rank = rank;
  peer_rendezvous_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError();
}

int ci8_selftest_wait_timeout(unsigned deadline_us, int* gave_up, ci8_stream_t stream) {
  if (!gave_up || deadline_us == 0 || deadline_us > 1000000) return kInvalid;   // at most one second
  wait_timeout_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(deadline_us) * 1000ull, gave_up);
  return cudaGetLastError();
}

int ci8_selftest_cluster_timeout(unsigned deadline_us, int* gave_up, ci8_stream_t stream) {
  if (!gave_up || deadline_us == 0 || deadline_us > 1000000) return kInvalid;   // at most one second
  cluster_timeout_selftest_kernel<<<2, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(deadline_us) * 1000ull, gave_up);
  return cudaGetLastError();
}

int ci8_dynamic_channel_mm(const void* x, const int8_t* w, const void* w_scale, int8_t* codes, float* scales, void* out,
                           int m, int n, int k, ci8_stream_t stream) {
  if (!x || !w || !w_scale || !codes || !scales || !out || !gemm_geometry_ok(m, n, k) || !aligned(x, 16) ||
      !aligned(codes, 16) || !aligned(w, 16) || static_cast<long long>(m) * n > INT32_MAX)
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (m <= 16 && k <= 8192) {
    // one kernel when the streaming kernel would run unsplit: it scans the activations for the row scales
    // and quantizes each K block on its way into the operand tile
    int split = 1, slab = 128;
    choose_decode_shape(n, k, 16, 4, sm_count(), &split, &slab);
    if (split == 1) {
      DecodeParams p{codes, scales, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out),
                     nullptr, m, n, k, slab, codes, scales, static_cast<const uint16_t*>(x)};
      return launch_decode_variant<1, false, 64, 16, true>(codes, w, p, s);
    }
  }
  cudaError_t err = launch_quantize(x, codes, scales, m, k, m, 0, s);
  if (err != cudaSuccess) return err;
  return ci8_fused_channel_mm(codes, w, scales, w_scale, out, m, n, k, 0, stream);
}

int ci8_gate_up_silu_mm(const int8_t* a, const int8_t* w, const float* a_scale, const void* w_scale, void* out, int m,
                        int n, int k, ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !out || !gemm_geometry_ok(m, n, k) || n % 256 != 0 || !aligned(a, 16) ||
      !aligned(w, 16) || !aligned(out, 16) || static_cast<long long>(m) * n > INT32_MAX)
    return kInvalid;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  GemmParams p{a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out), nullptr,
               m, n, k, 1, 0, 0, 0, 0, 0, 0};
  return m > 128 ? launch_gemm<2, kModeSwiGLU>(a, w, p, s) : launch_gemm<1, kModeSwiGLU>(a, w, p, s);
}

int ci8_q8_block_mm(const void* x, int8_t* a, float* sa, const int8_t* w, const void* sw, void* y, int m, int n,
                    int k, ci8_stream_t stream) {
  if (!x || !a || !sa || !w || !sw || !y || m <= 0 || n <= 0 || k <= 0 || k % 32 != 0 || k > 65536 ||
      static_cast<long long>(m) * k > INT32_MAX || static_cast<long long>(n) * k > INT32_MAX ||
      static_cast<long long>(m) * n > INT32_MAX || !aligned(x, 16) || !aligned(a, 16) || !aligned(w, 16) ||
      !aligned(sw, 2) || !aligned(sa, 4))
    return kInvalid;
  return launch_q8_block(x, a, sa, w, sw, y, m, n, k, reinterpret_cast<cudaStream_t>(stream));
}

// The reference's own name for this entry point (benchmarks/cuda/q8_block_int8.cu:150-160), so that its
// validation script, which only accepts that name, can load this library unchanged.
int q8_block_int8(const void* x, int8_t* a, float* sa, const int8_t* w, const void* sw, void* y, int m, int n, int k,
                  ci8_stream_t stream) {
  return ci8_q8_block_mm(x, a, sa, w, sw, y, m, n, k, stream);
}

int ci8_q8_block_mm_static(const void* x, const int8_t* w, const void* sw, void* y, int m, int n, int k,
                           ci8_stream_t stream) {
  if (!x || !w || !sw || !y || m <= 0 || n <= 0 || k <= 0 || k % 32 != 0 || k > 65536 ||
      static_cast<long long>(n) * k > INT32_MAX || static_cast<long long>(m) * n > INT32_MAX || !aligned(x, 16) ||
      !aligned(w, 16) || !aligned(sw, 2))
    return kInvalid;
  if (static_cast<long long>(m) * k > kQ8StaticMaxValues) return kInvalid;   // does not fit the built-in scratch
  unsigned char* scratch = nullptr;
  const cudaError_t err = q8_static_scratch(&scratch);
  if (err != cudaSuccess) return err;
  // every code and scale the product kernel reads is written by the quantizer of the same call first
  // (rows past m are zero-filled by the tensor map), so nothing left over from an earlier call is seen
  return launch_q8_block(x, reinterpret_cast<int8_t*>(scratch), reinterpret_cast<float*>(scratch + kQ8StaticScaleOffset),
                         w, sw, y, m, n, k, reinterpret_cast<cudaStream_t>(stream));
}

int ci8_q8_block_static_max_values(void) { return static_cast<int>(kQ8StaticMaxValues); }

int ci8_q8_block_tile_channels(int m, int n) { return (m > 0 && n > 0) ? q8_block_tile_channels(m, n) : 0; }

int ci8_gemm_tile_plan(int m, int n, int k, int groups, int* plan) {
  if (!plan || m <= 0 || n <= 0 || k <= 0 || groups <= 0) return kInvalid;
  GemmParams p{nullptr, nullptr, nullptr, nullptr, m, n, k, groups, 0, 0, 0, 0, 0, 0};
  const int sms = sm_count();
  const bool pair = m > 128;
  if (groups > 1) {
    if (pair) plan_tiles<2, kModeGrouped>(p, 1, sms / 2); else plan_tiles<1, kModeGrouped>(p, 1, sms);
  } else {
    if (pair) plan_tiles<2, kModeFused>(p, 1, sms / 2); else plan_tiles<1, kModeFused>(p, 1, sms);
  }
  plan[0] = p.tile_n;
  plan[1] = p.tiles_n;
  plan[2] = p.wide_tiles;
  plan[3] = p.split;
  return 0;
}

// Test hook: the streaming kernel with a forced split-K factor (1, 2 or 4; at most 2 above 16 rows);
// weights_biased != 0 selects the UINT8 form. Same contract as ci8_fused_channel_mm / ci8_channel_mm.
int ci8_decode_mm_split(const int8_t* a, const void* w, const float* a_scale, const void* w_scale,
                        int32_t* workspace, void* out, int m, int n, int k, int split, int weights_biased,
                        ci8_stream_t stream) {
  if (!a || !w || !a_scale || !w_scale || !out || !gemm_geometry_ok(m, n, k) || m > kDecodeMaxRows ||
      (split != 1 && split != 2 && split != 4) || split > (k + 127) / 128 || !aligned(a, 16) || !aligned(w, 16))
    return kInvalid;
  DecodeParams p{a, a_scale, static_cast<const __nv_bfloat16*>(w_scale), static_cast<__nv_bfloat16*>(out),
                 workspace, m, n, k, 0};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return weights_biased ? launch_decode<true>(a, w, p, split, s) : launch_decode<false>(a, w, p, split, s);
}

}  // extern "C"

// Small-M (<= 64 rows) W8A8 linear for decode and small batches: an HBM-streaming kernel.
//
// The weight matrix W [N,K] is read exactly once. One CTA owns a slab of C <= 256 output channels
// (a multiple of 16) and streams it through a deep TMA ring; the host chooses C and the split-K
// factor so that the CTAs fill the SMs in one wave. Per 128-byte K block a ring stage holds the
// C x 128 weight tile and the kRows x 128 tile of (zero-padded) activation rows, kRows = 16 or 64.
// The MMA is tcgen05.mma kind::i8 with M = 64, N = C: the activations are the M side and the
// weights the N side. With the 16-row tile only accumulator rows 0..15 mean anything; rows 16..63
// of the A operand are whatever shared memory follows the 2 KB activation tile (integer garbage
// that lands in accumulator rows nobody reads). Measured on B200, one such instruction (K = 32)
// takes about 24-33 cycles for N <= 64 and N/2 cycles from N = 128 up, so four of them per stage
// stay far below the time the stage's bytes take to arrive.
//
// Warp roles (16-row tile): warp 2 issues the TMA loads, warp 1 the MMAs, warps 0 and 4 run the
// epilogue (accumulator rows 0..15 are TMEM lanes 0..15, which only warps 0 and 4 can read); the
// 64-row tile has rows in every lane quarter and uses warps 0..7 for the epilogue. The producer
// and MMA loops are executed by their whole warp with one elected lane issuing: the loop state
// then lives in uniform registers, which is where TMA and MMA instructions take their operands;
// issued from a single thread inside a divergent branch every instruction paid tens of cycles of
// register moves, which capped a stage at about 0.3 us however narrow the slab.
//
// Split-K: a cluster of kSplit CTAs shares a slab, each streaming its own K range; the non-leader
// CTAs push their INT32 partials into the leader's shared memory (DSMEM) and the leader adds them —
// integer addition, so the result does not depend on the split.
//
// UINT8 weights (code+128): the MMA reads them as unsigned, and the epilogue removes
// 128 * sum_k a[row,k], computed by the epilogue warps from the INT8 activations.
//
// The kernel is launched with programmatic stream serialization: its prologue may overlap the
// tail of the kernel before it in the stream, and griddepcontrol.wait stands before the first
// access to global memory.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include "quantize.cuh"
#include "sm100_ptx.cuh"

namespace ci8 {

struct DecodeParams {
  const int8_t* a;            // [M,K] INT8 activations (for the UINT8-weight row sums)
  const float* sa;            // [M]
  const __nv_bfloat16* sw;    // [N]
  __nv_bfloat16* out;         // [M,N]
  int32_t* workspace;         // optional [M,N] INT32 accumulators
  int m, n, k;
  int slab;                   // channels per CTA (multiple of 16, 16..256)
  // dynamic form only: the kernel quantizes the BF16 activations itself (sa is unused, a is written)
  int8_t* codes_out;          // [M,K] INT8 codes, as quantize_rows would write them
  float* scales_out;          // [M] FP32 row scales, likewise
  const uint16_t* x;          // [M,K] BF16 activations
};

// kRowsT: rows of the activation tile in shared memory (16 or 64). kDataRowsT: distinct rows in it
// (M <= kDataRowsT). <64, 16> is the replicated form: the 16-row box is loaded four times, so every
// TMEM lane quarter holds a copy of the 16 result rows and eight warps share the epilogue's chunks.
// kDynamicT: the kernel takes BF16 activations and quantizes them itself (row absmax in the prologue,
// one pack per epilogue-warp lane per stage into the INT8 operand tile); replicated 64-row form only.
template <int kSplit, int kRowsT = 16, int kDataRowsT = kRowsT, bool kDynamicT = false>
struct DecodeConfig {
  static_assert(!kDynamicT || (kRowsT == 64 && kDataRowsT == 16 && kSplit == 1), "dynamic form: replicated tile, no split");
  static constexpr bool kDynamic = kDynamicT;
  static constexpr int kXBytes = kDynamicT ? 16 * 128 * 2 : 0;   // BF16 activation tile of a stage (two 64-column boxes)
  static_assert(kRowsT == 16 || kRowsT == 64, "activation tiles of 16 or 64 rows");
  static_assert(kDataRowsT == 16 || (kDataRowsT == 64 && kRowsT == 64), "16 or 64 distinct rows");
  static_assert(kDataRowsT == 16 || kSplit <= 2, "the 64-row reduce buffer only fits for a split of two");
  static constexpr int kRows = kRowsT;                   // activation rows per tile
  static constexpr int kDataRows = kDataRowsT;           // distinct rows (the TMA box)
  static constexpr bool kReplicated = kRowsT != kDataRowsT;
  static constexpr int kBlockK = 128;
  static constexpr int kMaxSlab = 256;
  static constexpr int kABytes = kRows * kBlockK;        // activation bytes loaded per stage
  static constexpr int kMmaM = 64;                       // smallest M of the instruction
  // a 16-row tile is followed by 48 more operand rows the instruction reads (and nobody uses)
  static constexpr int kAOperandPad = (kMmaM - kRows) * kBlockK;
  // The ring is a fixed region cut into stages of slab*128 + kABytes, as many as fit (at most
  // kMaxStages): a narrow slab gets more, smaller stages, so the bytes in flight stay the same.
  static constexpr int kRingBytes =
      kRows == 16 ? (kSplit == 1 ? 6 : kSplit == 2 ? 5 : 4) * (kMaxSlab * kBlockK + kABytes)
      : kDynamicT   ? 5 * (kMaxSlab * kBlockK + kABytes + kXBytes)
      : kReplicated ? (kSplit == 1 ? 5 : kSplit == 2 ? 4 : 3) * (kMaxSlab * kBlockK + kABytes)
                    : (kSplit == 1 ? 5 * (kMaxSlab * kBlockK + kABytes) : 150 * 1024);
  static constexpr int kMaxStages = 24;
  static constexpr int kReduceBytes = kSplit == 1 ? 0 : (kSplit - 1) * kDataRows * kMaxSlab * 4;
  static constexpr int kTmemColumns = 256;
  // Accumulator row r lives in TMEM lane 32 * (r / 16) + r % 16, and a warp reaches the lane quarter
  // of its index modulo four. 16 rows: warps 0 and 4 run the epilogue, 1 the MMAs, 2 the TMA loads
  // (3 idles). 64 rows: warps 0..7 run the epilogue (two per quarter), 8 the MMAs, 9 the loads.
  static constexpr int kEpilogueWarps = kRows == 16 ? 2 : 8;
  static constexpr int kMmaWarp = kRows == 16 ? 1 : 8;
  static constexpr int kTmaWarp = kRows == 16 ? 2 : 9;
  static constexpr int kThreads = kRows == 16 ? 160 : 320;
  static constexpr int kBarrierBytes = 1024;
  // FP32 channel scales of the slab + row sums per warp + (dynamic form) row scales and their inverses
  static constexpr int kScaleBytes = kMaxSlab * 4 + 8 * 16 * 4 + 2 * 16 * 4;
  static constexpr int kSmemBytes = kRingBytes + kAOperandPad + kReduceBytes + kBarrierBytes + kScaleBytes + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <int kSplit, bool kBiased, int kRows = 16, int kDataRows = kRows, bool kDynamic = false>
__global__ void __launch_bounds__((DecodeConfig<kSplit, kRows, kDataRows, kDynamic>::kThreads), 1)
decode_w8a8_kernel(const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_a, const DecodeParams p) {
  static_assert(!(kDynamic && kBiased), "the dynamic form takes signed weights");
  using Cfg = DecodeConfig<kSplit, kRows, kDataRows, kDynamic>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  constexpr int kReduceOffset = Cfg::kRingBytes + Cfg::kAOperandPad;
  int32_t* reduce_buf = reinterpret_cast<int32_t*>(smem + kReduceOffset);   // [rank-1][kMaxSlab][kRows]: rows adjacent
  uint8_t* bar_region = smem + kReduceOffset + Cfg::kReduceBytes;
  const uint32_t bar_base = smem_base + kReduceOffset + Cfg::kReduceBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kMaxStages + s); };
  const uint32_t done_bar = bar_base + 8u * (2 * Cfg::kMaxStages);
  auto ready_bar = [&](int s) { return bar_base + 8u * (2 * Cfg::kMaxStages + 1 + s); };   // dynamic form
  // split-K: the other CTAs of the cluster arrive here (remotely) once their partial sums are in this
  // CTA's reduce buffer; only the leader's copy is used
  const uint32_t reduce_bar = bar_base + 8u * (3 * Cfg::kMaxStages + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_region + 8 * (3 * Cfg::kMaxStages + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* scale_tab = reinterpret_cast<float*>(bar_region + Cfg::kBarrierBytes);          // [kMaxSlab]
  int32_t* row_sums = reinterpret_cast<int32_t*>(scale_tab + Cfg::kMaxSlab);             // [warp][16]
  float* row_scales = reinterpret_cast<float*>(row_sums + 8 * 16);                        // [16] scale, [16] inverse

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const uint32_t rank = kSplit > 1 ? cluster_ctarank() : 0u;
  const int slab_index = blockIdx.x / kSplit;
  const int n0 = slab_index * p.slab;
  const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;
  const int kb_begin = static_cast<int>((static_cast<long long>(num_kb) * rank) / kSplit);
  const int kb_end = static_cast<int>((static_cast<long long>(num_kb) * (rank + 1)) / kSplit);
  const int w_bytes = p.slab * Cfg::kBlockK;                 // weight tile of one stage (multiple of 1024)
  const int stage_bytes = w_bytes + Cfg::kABytes + Cfg::kXBytes;
  const int num_stages = min(Cfg::kMaxStages, Cfg::kRingBytes / stage_bytes);

  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      if constexpr (kDynamic) mbar_init(ready_bar(s), Cfg::kEpilogueWarps);
    }
    mbar_init(done_bar, 1);
    if constexpr (kSplit > 1) mbar_init(reduce_bar, (kSplit - 1) * Cfg::kEpilogueWarps);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_a);
  }
  if (warp == Cfg::kMmaWarp) {
    tmem_alloc<1>(smem_u32(tmem_slot), Cfg::kTmemColumns);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  // Split-K, first cluster phase: every thread announces that its CTA's barriers are initialised. The
  // matching wait stands in front of the first access to another CTA's shared memory (the epilogue
  // warps) or in the teardown (everybody else), so nobody blocks here.
  if constexpr (kSplit > 1) cluster_arrive();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only shared memory, TMEM and kernel parameters. While the previous kernel in
  // the stream drains (this CTA got its SM when one of that kernel's CTAs left; the whole grid may take a few
  // more microseconds to finish and flush), the weight tiles of the first ring-full of stages are prefetched
  // into L2, in the producer's order: HBM would otherwise sit idle across the kernel boundary, and the first
  // loads after the wait would each pay a DRAM round trip. A prefetch reads nothing into the SM (see
  // tma_prefetch_l2_2d), so it needs no ordering against the previous kernel.
  if (warp == Cfg::kTmaWarp && kb_end > kb_begin) {
    if (elect_one()) {
      const int count = kb_end - kb_begin;
      const int ahead = count < num_stages ? count : num_stages;
      int kb = kb_begin + (slab_index * 5) % count;
      for (int i = 0; i < ahead; ++i) {
        tma_prefetch_l2_2d(&map_w, kb * Cfg::kBlockK, n0);
        if (++kb == kb_end) kb = kb_begin;
      }
    }
    __syncwarp();
  }
  // From here on global memory is read and written, so the previous kernel in the stream must have finished.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == Cfg::kTmaWarp) {
    // ---------------------------------------------------------------- TMA producer
    // The whole warp runs the loop and an elected lane issues: loop state then stays in uniform
    // registers, which is where the TMA and MMA instructions take their operands from (issued
    // from one thread of a divergent branch they cost tens of cycles each in register moves).
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t tx = static_cast<uint32_t>(stage_bytes);
    // Every slab walks its K range from a different starting block (integer accumulation does
    // not care about the order), which spreads the CTAs over the activation lines and DRAM pages.
    const int count = kb_end - kb_begin;
    int kb = count > 0 ? kb_begin + (slab_index * 5) % count : kb_begin;
    for (int i = 0; i < count; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))) {
        __nanosleep(200000);
        break;
      }
      if (elect_one()) {
        const uint32_t w_dst = smem_base + stage * stage_bytes;
        if constexpr (kDynamic) {
          // weights and the BF16 activation tile (two 64-column boxes); the INT8 operand tile is written
          // by the epilogue warps
          mbar_arrive_expect_tx(full_bar(stage), static_cast<uint32_t>(w_bytes + Cfg::kXBytes));
          tma_load_2d(w_dst, &map_w, kb * Cfg::kBlockK, n0, full_bar(stage));
          tma_load_2d(w_dst + w_bytes + Cfg::kABytes, &map_a, kb * Cfg::kBlockK, 0, full_bar(stage));
          tma_load_2d(w_dst + w_bytes + Cfg::kABytes + Cfg::kXBytes / 2, &map_a, kb * Cfg::kBlockK + 64, 0, full_bar(stage));
        } else {
          mbar_arrive_expect_tx(full_bar(stage), tx);
          tma_load_2d(w_dst, &map_w, kb * Cfg::kBlockK, n0, full_bar(stage));
#pragma unroll
          for (int copy = 0; copy < Cfg::kRows / Cfg::kDataRows; ++copy)   // the same box into every lane quarter's rows
            tma_load_2d(w_dst + w_bytes + copy * Cfg::kDataRows * Cfg::kBlockK, &map_a, kb * Cfg::kBlockK, 0, full_bar(stage));
        }
      }
      __syncwarp();
      if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      if (++kb == kb_end) kb = kb_begin;
    }
  } else if (warp == Cfg::kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    // A = activations (signed, M = 64 of which kRows are real), B = weights (N = slab)
    const uint32_t idesc = idesc_i8(Cfg::kMmaM, p.slab, /*b_unsigned=*/kBiased);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = kb_begin; kb < kb_end; ++kb) {
      if (!__all_sync(0xffffffffu, mbar_wait(kDynamic ? ready_bar(stage) : full_bar(stage), phase, abort_flag))) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t w_addr = smem_base + stage * stage_bytes;
      const uint64_t w_desc = smem_desc_sw128(w_addr);
      const uint64_t a_desc = smem_desc_sw128(w_addr + w_bytes);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_i8<1>(tmem_base, a_desc + 2u * ks, w_desc + 2u * ks, idesc, (kb != kb_begin || ks != 0) ? 1u : 0u);
        mma_commit(empty_bar(stage));
      }
      __syncwarp();
      if (++stage == num_stages) { stage = 0; phase ^= 1u; }
    }
    if (ok && elect_one()) mma_commit(done_bar);
    __syncwarp();
  } else if (kRows == 16 ? (warp == 0 || warp == 4) : warp < 8) {
    // ---------------------------------------------------------------- epilogue warps
    // Two warps per TMEM lane quarter take alternate 32-channel chunks; lanes 0..15 of a warp are
    // the accumulator rows 16 * quarter + lane, lanes 16..31 carry rows nobody uses.
    const int e = warp >> 2;
    const int quarter = warp & 3;
    const int row = Cfg::kReplicated ? lane : quarter * 16 + lane;   // meaningful for lane < 16
    // chunks of this warp: first, first + stride, ... (the replicated form spreads them over all eight warps)
    constexpr int kChunkStride = Cfg::kReplicated ? 8 : 2;
    const int first_chunk = Cfg::kReplicated ? quarter * 2 + e : e;
    const bool real_row = lane < 16;
    const uint32_t tmem_lanes = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    int32_t* my_row_sums = row_sums + warp * 16;
    constexpr int kMyChunks = Cfg::kMaxSlab / 32 / kChunkStride;
    if constexpr (kBiased) {
      // sum_k a[row,k] over this CTA's K range: two lanes per activation row (each warp its own copy)
      const int r = (Cfg::kReplicated ? 0 : quarter * 16) + (lane >> 1), part = lane & 1;
      int sum = 0;
      if (r < p.m) {
        const int k_begin = kb_begin * Cfg::kBlockK, k_end = min(kb_end * Cfg::kBlockK, p.k);
        const int8_t* src = p.a + static_cast<size_t>(r) * p.k;
        if (reinterpret_cast<uintptr_t>(p.a) % 16 == 0 && p.k % 16 == 0) {
          for (int kk = k_begin + part * 16; kk < k_end; kk += 32) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + kk);
            sum = __dp4a(static_cast<int>(v.x), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.y), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.z), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.w), 0x01010101, sum);
          }
        } else {
          for (int kk = k_begin + part; kk < k_end; kk += 2) sum += src[kk];
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      if (part == 0) my_row_sums[lane >> 1] = sum;
    }
    // the channel scales do not depend on the accumulation: fetch them while the weights stream
#pragma unroll
    for (int i = 0; i < kMyChunks; ++i) {
      const int c = kChunkStride * i + first_chunk;
      const int channel = n0 + c * 32 + lane;
      scale_tab[c * 32 + lane] = (c * 32 + lane < p.slab && channel < p.n) ? __bfloat162float(p.sw[channel]) : 0.f;
    }
    __syncwarp();
    if constexpr (kDynamic) {
      // ---- row scales: the eight warps scan the BF16 activations once, all 256 threads on one row at a
      // time with every row's loads issued before the first is used (the scan has to finish while the
      // ring still has room for the weights streaming in); exactly the row quantizer's absmax -> scale.
      // Rows past M get scale 1 (their tile rows are zero-filled).
      const int team = warp * 32 + lane;                 // 0..255
      float* partial = reinterpret_cast<float*>(row_sums);   // [16][8] warp maxima (the row sums are a biased-form thing)
      const int packs_in_row = p.k >> 3;
      // four rows at a time, all of a thread's loads for them in flight together (K <= 8192: at most
      // four packs per thread and row)
      constexpr int kScanRows = 4;
#pragma unroll 1
      for (int r0 = 0; r0 < 16; r0 += kScanRows) {
        uint4 v[kScanRows][4];
#pragma unroll
        for (int rr = 0; rr < kScanRows; ++rr)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int pk = team + 256 * j;
            v[rr][j] = (r0 + rr < p.m && pk < packs_in_row)
                           ? __ldg(reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(r0 + rr) * p.k) + pk)
                           : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
        for (int rr = 0; rr < kScanRows; ++rr) {
          uint32_t packed_max = 0u;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            packed_max = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(packed_max, v[rr][j].x), v[rr][j].y),
                                                     v[rr][j].z), v[rr][j].w);
          float maximum = fmaxf(absmax_lo(packed_max), absmax_hi(packed_max));
#pragma unroll
          for (int mask = 16; mask; mask >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, mask));
          if (lane == 0) partial[(r0 + rr) * 8 + warp] = maximum;
        }
        if (r0 + kScanRows >= p.m) {   // remaining rows are beyond M: their maxima are zero
          for (int r = r0 + kScanRows; r < 16; ++r)
            if (lane == 0) partial[r * 8 + warp] = 0.f;
          break;
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");     // the eight epilogue warps only
      if (team < 16) {
        float maximum = partial[team * 8];
#pragma unroll
        for (int i = 1; i < 8; ++i) maximum = fmaxf(maximum, partial[team * 8 + i]);
        const float scale = team < p.m ? fmaxf(__fdiv_rn(maximum, 127.f), 1e-20f) : 1.f;
        row_scales[team] = scale;
        row_scales[16 + team] = __fdiv_rn(1.f, scale);
        if (blockIdx.x == 0 && team < p.m) p.scales_out[team] = scale;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      // ---- per stage: one 16-byte pack of BF16 per lane -> 8 codes into the INT8 operand tile (all
      // four 16-row slots of it), in the 128-byte-swizzled layout the MMA descriptor expects
      const int conv_row = team >> 4, pack_in_row = team & 15;
      const float scale = row_scales[conv_row], inverse = row_scales[16 + conv_row];
      const int count = kb_end - kb_begin;
      int kb = count > 0 ? kb_begin + (slab_index * 5) % count : kb_begin;     // the producer's order
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < count; ++i) {
        if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag))) break;
        uint8_t* stage_base = smem + stage * stage_bytes + w_bytes;
        const uint8_t* x_tile = stage_base + Cfg::kABytes;
        const int box = pack_in_row >> 3, chunk = pack_in_row & 7;
        const uint4 pack = *reinterpret_cast<const uint4*>(x_tile + box * (Cfg::kXBytes / 2) + conv_row * 128 +
                                                           ((chunk ^ (conv_row & 7)) << 4));
        const uint2 codes = quantize_pack(pack, scale, inverse);
        const int out_chunk = pack_in_row >> 1;          // 16-byte chunk of the 128-byte INT8 row
        const int offset = conv_row * 128 + ((out_chunk ^ (conv_row & 7)) << 4) + (pack_in_row & 1) * 8;
#pragma unroll
        for (int copy = 0; copy < Cfg::kRows / Cfg::kDataRows; ++copy)
          *reinterpret_cast<uint2*>(stage_base + copy * Cfg::kDataRows * Cfg::kBlockK + offset) = codes;
        if (blockIdx.x == 0 && conv_row < p.m && kb * Cfg::kBlockK + pack_in_row * 8 < p.k)
          *reinterpret_cast<uint2*>(p.codes_out + static_cast<size_t>(conv_row) * p.k + kb * Cfg::kBlockK + pack_in_row * 8) = codes;
        fence_proxy_async_smem();                        // generic-proxy writes -> visible to the MMA's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar(stage));
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        if (++kb == kb_end) kb = kb_begin;
      }
    }
    const int chunks = (p.slab + 31) / 32;
    const float row_scale = kDynamic ? ((real_row && row < p.m) ? row_scales[row] : 0.f)
                                     : ((real_row && row < p.m) ? p.sa[row] : 0.f);
    const bool have_work = kb_end > kb_begin;
    const bool ok = have_work ? mbar_wait(done_bar, 0u, abort_flag) : true;
    tcgen05_fence_after();
    const bool live = __all_sync(0xffffffffu, ok) && have_work;
    const int32_t bias = (kBiased && real_row) ? 128 * my_row_sums[lane] : 0;
    const bool out_vec = (p.n % 8 == 0) && (reinterpret_cast<uintptr_t>(p.out) % 16 == 0);
    const bool ws_vec = (p.n % 4 == 0) && (reinterpret_cast<uintptr_t>(p.workspace) % 16 == 0);

    // Walks this warp's chunks with the TMEM read of the next chunk in flight while the current
    // one is processed; f(chunk, acc) gets the bias-corrected INT32 accumulators of 32 channels.
    auto for_each_chunk = [&](auto&& f) {
      uint32_t v[2][32];
      if (live && first_chunk < chunks) tmem_ld_32x32(tmem_lanes + first_chunk * 32, v[0]);
#pragma unroll
      for (int i = 0; i < kMyChunks; ++i) {
        const int chunk = kChunkStride * i + first_chunk;
        if (chunk >= chunks) break;
        uint32_t (&cur)[32] = v[i & 1];
        if (live) {
          tmem_ld_wait_for(cur);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) cur[j] = 0u;
        }
        if (i + 1 < kMyChunks && live && chunk + kChunkStride < chunks)
          tmem_ld_32x32(tmem_lanes + (chunk + kChunkStride) * 32, v[(i + 1) & 1]);
        int32_t acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = static_cast<int32_t>(cur[j]) - bias;
        f(chunk, acc);
      }
    };

    bool partials_in = true;
    if constexpr (kSplit > 1) {
      cluster_wait();   // first phase: every CTA of the cluster has initialised its barriers
      if (rank != 0) {
        // push this CTA's partials into the leader's reduce buffer: [rank-1][channel][row]
        const uint32_t remote = map_to_cta(smem_u32(reduce_buf), 0);
        for_each_chunk([&](int chunk, int32_t (&acc)[32]) {
          if (real_row) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const uint32_t offset = (((rank - 1) * Cfg::kMaxSlab + chunk * 32 + j) * Cfg::kDataRows + row) * 4;
              asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + offset), "r"(acc[j]) : "memory");
            }
          }
        });
        // the stores above are released to the leader by this warp's arrival on its barrier
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(reduce_bar, 0);
      } else {
        // The leader waits for every epilogue warp of every other CTA, with a deadline like every other
        // wait: a peer that never delivers raises the cluster status bit and this CTA writes nothing.
        partials_in = __all_sync(0xffffffffu, mbar_wait<true, kStatusClusterTimeout>(reduce_bar, 0u, abort_flag));
      }
    }
    if (rank == 0 && partials_in) {
      for_each_chunk([&](int chunk, int32_t (&acc)[32]) {
        if constexpr (kSplit > 1) {
          if (real_row) {
#pragma unroll
            for (int r = 0; r < kSplit - 1; ++r)
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] += reduce_buf[(r * Cfg::kMaxSlab + chunk * 32 + j) * Cfg::kDataRows + row];
          }
        }
        const int c0 = n0 + chunk * 32;                     // first output channel of this chunk
        if (c0 >= p.n) return;
        const int limit = min(min(32, p.slab - chunk * 32), p.n - c0);
        const float4* scales = reinterpret_cast<const float4*>(scale_tab + chunk * 32);   // broadcast reads
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 s = scales[j >> 2];
          const float f0 = __fmul_rn(__int2float_rn(acc[j]), row_scale);
          const float f1 = __fmul_rn(__int2float_rn(acc[j + 1]), row_scale);
          const float f2 = __fmul_rn(__int2float_rn(acc[j + 2]), row_scale);
          const float f3 = __fmul_rn(__int2float_rn(acc[j + 3]), row_scale);
          __nv_bfloat162 lo = __floats2bfloat162_rn(__fmul_rn(f0, s.x), __fmul_rn(f1, s.y));
          __nv_bfloat162 hi = __floats2bfloat162_rn(__fmul_rn(f2, s.z), __fmul_rn(f3, s.w));
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&lo);
          packed[(j >> 1) + 1] = *reinterpret_cast<uint32_t*>(&hi);
        }
        if (real_row && row < p.m) {
          __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * p.n + c0;
          if (out_vec && limit == 32) {
#pragma unroll
            for (int j = 0; j < 16; j += 4)
              *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (j < limit) {
                const uint32_t word = packed[j >> 1];
                reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>((j & 1) ? (word >> 16) : (word & 0xffffu));
              }
          }
          if (p.workspace) {
            int32_t* ws = p.workspace + static_cast<size_t>(row) * p.n + c0;
            if (ws_vec && limit == 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<int4*>(ws + j) = make_int4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
            } else {
              for (int j = 0; j < 32; ++j)
                if (j < limit) ws[j] = acc[j];
            }
          }
        }
      });
    }
  }
  if constexpr (kSplit > 1) {
    // the epilogue warps completed the first cluster phase above, everybody else does it here
    if (!(kRows == 16 ? (warp == 0 || warp == 4) : warp < 8)) cluster_wait();
    // Second phase: no CTA leaves while a peer may still write into its shared memory or arrive on its
    // barrier. This hardware barrier has no deadline of its own; it is bounded because every wait on a
    // peer's way here is.
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == Cfg::kMmaWarp) {
    tcgen05_fence_after();
    tmem_dealloc<1>(tmem_base, Cfg::kTmemColumns);
  }
}

}  // namespace ci8

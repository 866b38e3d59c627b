// Block-32 (GGUF Q8_0 style) W8A8 linear: activation scales and INT32 accumulation restart every
// 32 K elements; the rescaled partial sums are added in FP32.
//
//   x BF16 [M,K] -> a INT8 [M,K], sa FP32 [M,K/32]        (q8_block_quantize_kernel)
//   y[m,n] = bf16( sum over blocks b ascending of  float(dot_b[m,n]) * (sa[m,b] * float(sw[n,b])) )
// with one FMA per block: t = fma(float(dot_b), sa*sw, t), which is what the reference's
// `sum += float(acc) * (sa * sw)` compiles to (benchmarks/cuda/q8_block_int8.cu:44-62 in the
// reference). w INT8 [N,K] holds Q8_0 codes in [-128,127], sw FP16 [N,K/32] their block scales.
//
// The 32-deep dot products are exactly one tcgen05.mma.kind::i8 instruction (K = 32) each, issued
// with a fresh accumulator: a ring stage holds 128 bytes of K = four blocks, whose four
// 128 x 64 accumulators fill one 256-column half of TMEM while the epilogue warps drain the other
// half. The kernel is bound by the CUDA cores, not by the tensor pipe: every (row, channel, block)
// costs an INT32->FP32 conversion, the scale product and the FMA (the four MMAs of a stage take
// ~200 cycles, draining their accumulators ~1700), which is inherent to per-block FP32 rescaling
// of INT32 partials — the block-scaled tcgen05 kinds take floating-point operands only. (Replacing
// the conversion instruction by an integer add and a packed FP32 subtract of 1.5 * 2^23 was
// measured slower; so was letting the MMA do the add: accumulators pre-set to the bits of 1.5 * 2^23
// with tcgen05.st after every read, MMA accumulating onto them, one packed subtract per two values:
// bit-exact, 143 us against 123 us on M=4096, N=1024, K=4096. Cycle stamps in the epilogue warps put 1160 of the
// 1470 cycles of a stage into the arithmetic itself: 72 instructions per block and warp at two issue cycles each,
// conversion and packed FP32 alike, which is why neither sixteen epilogue warps of 16 channels, with registers
// moved over from the load and MMA warps, nor accumulator loads that run ahead across stage boundaries helped:
// 136 and 127 us.)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "gemm_tcgen05.cuh"
#include "quantize.cuh"
#include "sm100_ptx.cuh"

namespace ci8 {

// One thread per block of 32 values: 64 bytes in, 32 code bytes and one scale out. The arithmetic
// is the row quantizer's (scale = max(absmax/127, 1e-20), round half to even of the IEEE quotient).
__global__ void __launch_bounds__(256)
q8_block_quantize_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales,
                         int64_t blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t block = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (block >= blocks) return;
  const uint4* src = reinterpret_cast<const uint4*>(x) + block * 4;
  uint4 pack[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) pack[i] = __ldg(src + i);
  uint32_t packed_max = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    packed_max = absmax_bf16x2(packed_max, pack[i].x);
    packed_max = absmax_bf16x2(packed_max, pack[i].y);
    packed_max = absmax_bf16x2(packed_max, pack[i].z);
    packed_max = absmax_bf16x2(packed_max, pack[i].w);
  }
  const float maximum = fmaxf(absmax_lo(packed_max), absmax_hi(packed_max));
  const float scale = fmaxf(__fdiv_rn(maximum, 127.f), 1e-20f);
  const float inverse = __fdiv_rn(1.f, scale);
  uint2 codes[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) codes[i] = quantize_pack(pack[i], scale, inverse);
  uint4* dst = reinterpret_cast<uint4*>(q) + block * 2;
  dst[0] = make_uint4(codes[0].x, codes[0].y, codes[1].x, codes[1].y);
  dst[1] = make_uint4(codes[2].x, codes[2].y, codes[3].x, codes[3].y);
  scales[block] = scale;
}

struct Q8BlockParams {
  const float* sa;            // [M, K/32]
  const __half* sw;           // [N, K/32]
  __nv_bfloat16* y;           // [M, N]
  int m, n, k;
  int tiles_m, tiles_n;
};

// kTileNT: output channels per tile, 64, 32 or 16. The time of a tile is its epilogue's, which is proportional
// to the channels; the host takes a narrower tile when the wider one would leave the last wave (or, for a small
// problem, most of the SMs) without work.
template <int kTileNT>
struct Q8BlockConfig {
  static_assert(kTileNT == 64 || kTileNT == 32 || kTileNT == 16, "tile widths: 64, 32 or 16 channels");
  static constexpr int kBlockM = 128;                  // rows of A per tile
  static constexpr int kTileN = kTileNT;               // output channels per tile
  static constexpr int kBlockK = 128;                  // bytes of K per stage = four 32-wide blocks
  static constexpr int kBlocksPerStage = kBlockK / 32;
  static constexpr int kABytes = kBlockM * kBlockK;
  static constexpr int kWBytes = kTileN * kBlockK;
  static constexpr int kStageBytes = kABytes + kWBytes;
  static constexpr int kStages = 6;
  static constexpr int kEpiWarps = 8;                  // two per TMEM lane quarter, half of the tile's channels each
  static constexpr int kWarpColumns = kTileN / 2;      // channels per epilogue warp
  static constexpr int kThreads = (2 + kEpiWarps) * 32;
  static constexpr int kAccColumns = kBlocksPerStage * kTileN;   // at most 256: one half of TMEM per stage
  static constexpr int kScaleBytes = kEpiWarps * kBlocksPerStage * 32 * 4;   // FP32 weight scales per warp
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + kBarrierBytes + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <int kTileN>
__global__ void __launch_bounds__(Q8BlockConfig<kTileN>::kThreads, 1)
q8_block_mm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                   const Q8BlockParams p) {
  using Cfg = Q8BlockConfig<kTileN>;
  extern __shared__ uint8_t q8_smem_raw[];
  const uint32_t raw_addr = smem_u32(q8_smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = q8_smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  constexpr int kRingBytes = Cfg::kStages * Cfg::kStageBytes;
  float* scale_region = reinterpret_cast<float*>(smem + kRingBytes);
  uint8_t* bar_region = smem + kRingBytes + Cfg::kScaleBytes;
  const uint32_t bar_base = smem_base + kRingBytes + Cfg::kScaleBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * Cfg::kStages + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_region + 8 * (2 * Cfg::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), Cfg::kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), 512);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // the codes and scales come from the kernel before this one in the stream

  const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;
  const int blocks_in_row = p.k / 32;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int mt = tile % p.tiles_m, nt = tile / p.tiles_m;   // row tiles fastest: W tile stays in L2
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!__all_sync(0xffffffffu, mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))) { ok = false; break; }
        if (elect_one()) {
          mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
          const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
          tma_load_2d(a_dst, &map_a, kb * Cfg::kBlockK, mt * Cfg::kBlockM, full_bar(stage));
          tma_load_2d(a_dst + Cfg::kABytes, &map_w, kb * Cfg::kBlockK, nt * Cfg::kTileN, full_bar(stage));
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    pdl_launch_dependents();
    if (!ok) __nanosleep(200000);   // let loads already in flight land before teardown
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t phase = 0, iter = 0;
    bool ok = true;
    const uint32_t idesc = idesc_i8(Cfg::kBlockM, Cfg::kTileN, /*b_unsigned=*/false);
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++iter) {
        const uint32_t buf = iter & 1u, buf_phase = (iter >> 1) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait(tmem_empty_bar(buf), buf_phase ^ 1u, abort_flag))) { ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_base + stage * Cfg::kStageBytes;
        const uint64_t a_desc = smem_desc_sw128(a_addr);
        const uint64_t w_desc = smem_desc_sw128(a_addr + Cfg::kABytes);
        if (elect_one()) {
          // one instruction per 32-wide block, each into its own 64 accumulator columns
#pragma unroll
          for (int b = 0; b < Cfg::kBlocksPerStage; ++b)
            mma_i8<1>(tmem_base + buf * Cfg::kAccColumns + b * Cfg::kTileN, a_desc + 2u * b, w_desc + 2u * b, idesc, 0u);
          mma_commit(empty_bar(stage));
          mma_commit(tmem_full_bar(buf));
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: rescale and add
    const int epi = warp - 2;
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    const int half = epi >> 2;                    // which half of the tile's channels
    constexpr int kCols = Cfg::kWarpColumns;
    float* my_scales = scale_region + epi * (Cfg::kBlocksPerStage * 32);   // [block][channel]
    uint32_t iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int mt = tile % p.tiles_m, nt = tile / p.tiles_m;
      const int row = mt * Cfg::kBlockM + quarter * 32 + lane;
      const int col0 = nt * Cfg::kTileN + half * kCols;       // first channel of this warp
      const int my_col = col0 + lane;                         // the channel whose scales this lane fetches
      const bool my_col_live = lane < kCols && my_col < p.n;  // (lanes past the warp's channels fetch nothing)
      float2 sum2[kCols / 2];                                 // sums of channels 2i and 2i + 1
#pragma unroll
      for (int c = 0; c < kCols / 2; ++c) sum2[c] = make_float2(0.f, 0.f);
      // Scales of a stage's four blocks (zero past the end of K, of M or of N). Those of the next
      // stage are fetched while the current one is processed, and kept as the raw loaded words: any
      // arithmetic on them here would wait for the loads.
      float4 next_row_scales;     // sa[row, 4 blocks]
      uint2 next_channel_scales;  // sw[my_col, 4 blocks] as FP16 bit patterns
      const bool vector_scales = blocks_in_row % Cfg::kBlocksPerStage == 0 &&
                                 reinterpret_cast<uintptr_t>(p.sa) % 16 == 0 && reinterpret_cast<uintptr_t>(p.sw) % 8 == 0;
      auto fetch_scales = [&](int kb) {
        const int first = kb * Cfg::kBlocksPerStage;
        next_row_scales = make_float4(0.f, 0.f, 0.f, 0.f);
        next_channel_scales = make_uint2(0u, 0u);
        if (first >= blocks_in_row) return;
        const float* sa_row = p.sa + static_cast<size_t>(row) * blocks_in_row + first;
        const uint16_t* sw_row = reinterpret_cast<const uint16_t*>(p.sw) + static_cast<size_t>(my_col) * blocks_in_row + first;
        if (vector_scales) {
          // the stage's four blocks are adjacent: one 16-byte and one 8-byte load per thread
          if (row < p.m) next_row_scales = __ldg(reinterpret_cast<const float4*>(sa_row));
          if (my_col_live) next_channel_scales = __ldg(reinterpret_cast<const uint2*>(sw_row));
        } else {
          const int live = min(Cfg::kBlocksPerStage, blocks_in_row - first);
          if (row < p.m) {
            next_row_scales.x = __ldg(sa_row);
            if (live > 1) next_row_scales.y = __ldg(sa_row + 1);
            if (live > 2) next_row_scales.z = __ldg(sa_row + 2);
            if (live > 3) next_row_scales.w = __ldg(sa_row + 3);
          }
          if (my_col_live) {
            uint32_t h0 = __ldg(sw_row), h1 = 0u, h2 = 0u, h3 = 0u;
            if (live > 1) h1 = __ldg(sw_row + 1);
            if (live > 2) h2 = __ldg(sw_row + 2);
            if (live > 3) h3 = __ldg(sw_row + 3);
            next_channel_scales = make_uint2(h0 | (h1 << 16), h2 | (h3 << 16));
          }
        }
      };
      fetch_scales(0);
      for (int kb = 0; kb < num_kb; ++kb, ++iter) {
        const uint32_t buf = iter & 1u, buf_phase = (iter >> 1) & 1u;
        const float row_scale[Cfg::kBlocksPerStage] = {next_row_scales.x, next_row_scales.y, next_row_scales.z,
                                                       next_row_scales.w};
        {
          const __half2 lo = *reinterpret_cast<const __half2*>(&next_channel_scales.x);
          const __half2 hi = *reinterpret_cast<const __half2*>(&next_channel_scales.y);
          my_scales[0 * 32 + lane] = __low2float(lo);
          my_scales[1 * 32 + lane] = __high2float(lo);
          my_scales[2 * 32 + lane] = __low2float(hi);
          my_scales[3 * 32 + lane] = __high2float(hi);
        }
        __syncwarp();
        fetch_scales(kb + 1);   // past the last stage every block index is out of range: zeros, no loads
        if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), buf_phase, abort_flag))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * Cfg::kAccColumns + half * kCols;
        uint32_t v[2][kCols];
        tmem_ld_columns(taddr, v[0]);
#pragma unroll
        for (int b = 0; b < Cfg::kBlocksPerStage; ++b) {
          uint32_t (&cur)[kCols] = v[b & 1];
          tmem_ld_wait_for(cur);
          if (b + 1 < Cfg::kBlocksPerStage) tmem_ld_columns(taddr + (b + 1) * Cfg::kTileN, v[(b + 1) & 1]);
          const float4* channel_scales = reinterpret_cast<const float4*>(my_scales + b * 32);   // broadcast reads
          // packed FP32 arithmetic (two IEEE-rounded lanes per instruction): one multiply for two scale
          // products, one FMA for two accumulations
          const float2 rs2 = make_float2(row_scale[b], row_scale[b]);
#pragma unroll
          for (int c = 0; c < kCols; c += 4) {
            const float4 s = channel_scales[c >> 2];
            const float2 f01 = make_float2(__int2float_rn(static_cast<int32_t>(cur[c])), __int2float_rn(static_cast<int32_t>(cur[c + 1])));
            const float2 f23 = make_float2(__int2float_rn(static_cast<int32_t>(cur[c + 2])), __int2float_rn(static_cast<int32_t>(cur[c + 3])));
            sum2[c >> 1] = __ffma2_rn(f01, __fmul2_rn(rs2, make_float2(s.x, s.y)), sum2[c >> 1]);
            sum2[(c >> 1) + 1] = __ffma2_rn(f23, __fmul2_rn(rs2, make_float2(s.z, s.w)), sum2[(c >> 1) + 1]);
          }
        }
        // this warp is done with the accumulator half and with its scale slots
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
      }
      if (!ok) break;
      if (row < p.m) {
        __nv_bfloat16* dst = p.y + static_cast<size_t>(row) * p.n + col0;
        const int limit = p.n - col0;
        if (limit >= kCols && p.n % 8 == 0 && reinterpret_cast<uintptr_t>(p.y) % 16 == 0) {
#pragma unroll
          for (int c = 0; c < kCols / 2; c += 4)
            *reinterpret_cast<uint4*>(dst + 2 * c) =
                make_uint4(pack_bf16x2(sum2[c].x, sum2[c].y), pack_bf16x2(sum2[c + 1].x, sum2[c + 1].y),
                           pack_bf16x2(sum2[c + 2].x, sum2[c + 2].y), pack_bf16x2(sum2[c + 3].x, sum2[c + 3].y));
        } else {
#pragma unroll
          for (int c = 0; c < kCols; ++c)
            if (c < limit) dst[c] = __float2bfloat16_rn((c & 1) ? sum2[c >> 1].y : sum2[c >> 1].x);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

}  // namespace ci8

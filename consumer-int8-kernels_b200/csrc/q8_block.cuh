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
// ~130 cycles, draining their accumulators ~1000), which is inherent to per-block FP32 rescaling
// of INT32 partials — the block-scaled tcgen05 kinds take floating-point operands only.
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
  const float maximum = fmaxf(bf16_lo(packed_max), bf16_hi(packed_max));
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

struct Q8BlockConfig {
  static constexpr int kBlockM = 128;                  // rows of A per tile
  static constexpr int kTileN = 64;                    // output channels per tile
  static constexpr int kBlockK = 128;                  // bytes of K per stage = four 32-wide blocks
  static constexpr int kBlocksPerStage = kBlockK / 32;
  static constexpr int kABytes = kBlockM * kBlockK;
  static constexpr int kWBytes = kTileN * kBlockK;
  static constexpr int kStageBytes = kABytes + kWBytes;
  static constexpr int kStages = 6;
  static constexpr int kEpiWarps = 8;                  // two per TMEM lane quarter, 32 channels each
  static constexpr int kThreads = (2 + kEpiWarps) * 32;
  static constexpr int kAccColumns = kBlocksPerStage * kTileN;   // 256: one half of TMEM per stage
  static constexpr int kScaleBytes = kEpiWarps * kBlocksPerStage * 32 * 4;   // FP32 weight scales per warp
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + kBarrierBytes + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

__global__ void __launch_bounds__(Q8BlockConfig::kThreads, 1)
q8_block_mm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                   const Q8BlockParams p) {
  using Cfg = Q8BlockConfig;
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
    const int half = epi >> 2;                    // which 32 of the tile's 64 channels
    float* my_scales = scale_region + epi * (Cfg::kBlocksPerStage * 32);   // [block][channel]
    uint32_t iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int mt = tile % p.tiles_m, nt = tile / p.tiles_m;
      const int row = mt * Cfg::kBlockM + quarter * 32 + lane;
      const int col0 = nt * Cfg::kTileN + half * 32;          // first channel of this warp
      const int my_col = col0 + lane;                         // the channel whose scales this lane fetches
      float sum[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) sum[c] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++iter) {
        const uint32_t buf = iter & 1u, buf_phase = (iter >> 1) & 1u;
        // scales of this stage's four blocks (zero past the end of K, of M or of N)
        float row_scale[Cfg::kBlocksPerStage];
#pragma unroll
        for (int b = 0; b < Cfg::kBlocksPerStage; ++b) {
          const int block = kb * Cfg::kBlocksPerStage + b;
          const bool live = block < blocks_in_row;
          row_scale[b] = (live && row < p.m) ? __ldg(p.sa + static_cast<size_t>(row) * blocks_in_row + block) : 0.f;
          my_scales[b * 32 + lane] =
              (live && my_col < p.n) ? __half2float(p.sw[static_cast<size_t>(my_col) * blocks_in_row + block]) : 0.f;
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), buf_phase, abort_flag))) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * Cfg::kAccColumns + half * 32;
#pragma unroll
        for (int b = 0; b < Cfg::kBlocksPerStage; ++b) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + b * Cfg::kTileN, v);
          tmem_ld_wait_for(v);
          const float4* channel_scales = reinterpret_cast<const float4*>(my_scales + b * 32);   // broadcast reads
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const float4 s = channel_scales[c >> 2];
            sum[c] = __fmaf_rn(__int2float_rn(static_cast<int32_t>(v[c])), __fmul_rn(row_scale[b], s.x), sum[c]);
            sum[c + 1] = __fmaf_rn(__int2float_rn(static_cast<int32_t>(v[c + 1])), __fmul_rn(row_scale[b], s.y), sum[c + 1]);
            sum[c + 2] = __fmaf_rn(__int2float_rn(static_cast<int32_t>(v[c + 2])), __fmul_rn(row_scale[b], s.z), sum[c + 2]);
            sum[c + 3] = __fmaf_rn(__int2float_rn(static_cast<int32_t>(v[c + 3])), __fmul_rn(row_scale[b], s.w), sum[c + 3]);
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
        if (limit >= 32 && p.n % 8 == 0 && reinterpret_cast<uintptr_t>(p.y) % 16 == 0) {
#pragma unroll
          for (int c = 0; c < 32; c += 8)
            *reinterpret_cast<uint4*>(dst + c) =
                make_uint4(pack_bf16x2(sum[c], sum[c + 1]), pack_bf16x2(sum[c + 2], sum[c + 3]),
                           pack_bf16x2(sum[c + 4], sum[c + 5]), pack_bf16x2(sum[c + 6], sum[c + 7]));
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (c < limit) dst[c] = __float2bfloat16_rn(sum[c]);
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

// W8A16 small-batch linear: BF16 activations times BF16-rounded dequantized INT8 weights with
// FP32 accumulation:  wd[n,k] = bf16(float(code[n,k]) * float(sw[n])),
//                     out[m,n] = bf16(sum_k x[m,k] * wd[n,k]).
// HBM-bound on the weight stream, which is read exactly once.
//
// gemv_w8a16_mma_kernel: the multiply-accumulate runs on the tensor cores with register-fed
// operands (mma.sync m16n8k16, BF16 x BF16 -> FP32); what is left for the CUDA cores is the
// dequantisation, 3.75 instructions per weight byte. A warp owns 32 output channels (two 16-row
// A fragments) and a quarter of K; each lane loads 16 consecutive weight bytes of "its" channel
// per 64-wide K step. The K index inside a 64-wide step is permuted so that those 16 bytes feed
// four MMAs directly (the activations are read with the same permutation, so the dot products
// are unchanged). The four K quarters of a CTA are added through shared memory.
//
// gemv_w8a16_tma_kernel: the same arithmetic with the weights staged through shared memory by TMA
// (the production path); gemv_w8a16_mma_kernel keeps the register-fed loads (small N).
// gemv_w8a16_kernel: plain FMA version for activations that are not 16-byte aligned.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "sm100_ptx.cuh"

namespace ci8 {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four INT8 codes (one 32-bit word, already XORed with 0x80808080 so each byte is code+128) ->
// two BF16 pairs bf16(code * scale). PRMT builds the float f = 2^23 + (code+128); one FMA gives
// f*scale - (2^23+128)*scale = code*scale, exactly: the subtrahend is exact in FP32 because a BF16
// scale has 8 significant bits and (2^16+1)*m fits 24 bits, and |code|*m fits 16 bits, so the FMA
// rounds nothing and equals the reference's float(code)*scale; CVT then rounds pairs to BF16.
struct DequantScale {
  float scale;
  float offset;   // -(2^23 + 128) * scale
};
__device__ __forceinline__ DequantScale make_dequant_scale(float scale) {
  return DequantScale{scale, -__fmul_rn(8388736.f, scale)};
}
__device__ __forceinline__ void dequant4(uint32_t biased, const DequantScale& s, uint32_t& lo, uint32_t& hi) {
  const float c0 = __fmaf_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7650)), s.scale, s.offset);
  const float c1 = __fmaf_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7651)), s.scale, s.offset);
  const float c2 = __fmaf_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7652)), s.scale, s.offset);
  const float c3 = __fmaf_rn(__uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7653)), s.scale, s.offset);
  __nv_bfloat162 p0 = __floats2bfloat162_rn(c0, c1);
  __nv_bfloat162 p1 = __floats2bfloat162_rn(c2, c3);
  lo = *reinterpret_cast<uint32_t*>(&p0);
  hi = *reinterpret_cast<uint32_t*>(&p1);
}

// The same four codes -> two BF16 pairs with packed BF16 arithmetic, 2.5 instructions per weight byte.
// An INT8 code fits BF16's eight significant bits, so once it is a BF16 number, one packed multiply
// by the (BF16) scale is the exact product rounded once: the reference's bf16(float(code) * scale).
// Making it a BF16 number: 0x4300 | (code & 0x7f) is 128 + (code & 0x7f) exactly, and the code is
// that minus 128 (sign bit clear) or minus 256 (sign bit set); 0x4300 | (code & 0x80) is exactly that
// subtrahend (0x4300 = 128, 0x4380 = 256), and the difference of two such numbers is exact.
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// raw: four two's-complement codes; scale2: the channel's BF16 scale in both halves.
__device__ __forceinline__ void dequant4_packed(uint32_t raw, uint32_t scale2, uint32_t& lo, uint32_t& hi) {
  const uint32_t low7 = raw & 0x7f7f7f7fu, sign = raw & 0x80808080u;
  const uint32_t code01 = bf16x2_sub(__byte_perm(low7, 0x43434343u, 0x4140), __byte_perm(sign, 0x43434343u, 0x4140));
  const uint32_t code23 = bf16x2_sub(__byte_perm(low7, 0x43434343u, 0x4342), __byte_perm(sign, 0x43434343u, 0x4342));
  lo = bf16x2_mul(code01, scale2);
  hi = bf16x2_mul(code23, scale2);
}

constexpr int kGemvKSplit = 4;          // K quarters per CTA
constexpr int kGemvChannelsPerCta = 64; // two warps of 32 channels

// kRowBlocks = 1 for M <= 8, 2 for M <= 16. x must be 16-byte aligned, k % 16 == 0.
template <int kRowBlocks>
__global__ void __launch_bounds__(256)
gemv_w8a16_mma_kernel(const __nv_bfloat16* __restrict__ x, const int8_t* __restrict__ w,
                      const __nv_bfloat16* __restrict__ sw, __nv_bfloat16* __restrict__ out,
                      int m, int n, int k) {
  __shared__ float partial[kGemvKSplit - 1][2][2][kRowBlocks][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int channel_block = warp & 1, k_part = warp >> 1;
  const int c_base = blockIdx.x * kGemvChannelsPerCta + channel_block * 32;

  // K range of this warp in 64-wide steps
  const int steps = (k + 63) >> 6;
  const int step_begin = (steps * k_part) / kGemvKSplit;
  const int step_end = (steps * (k_part + 1)) / kGemvKSplit;

  // channels of this lane's A-fragment rows: group j, rows g and g + 8
  const int8_t* w_row[2][2];
  DequantScale scale[2][2];
  bool valid[2][2];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int channel = c_base + j * 16 + h * 8 + g;
      valid[j][h] = channel < n;
      w_row[j][h] = w + static_cast<size_t>(valid[j][h] ? channel : 0) * k;
      scale[j][h] = make_dequant_scale(valid[j][h] ? __bfloat162float(sw[channel]) : 0.f);
    }
  const __nv_bfloat16* x_row[kRowBlocks];
  bool x_valid[kRowBlocks];
#pragma unroll
  for (int rb = 0; rb < kRowBlocks; ++rb) {
    x_valid[rb] = rb * 8 + g < m;
    x_row[rb] = x + static_cast<size_t>(x_valid[rb] ? rb * 8 + g : 0) * k;
  }

  float acc[2][kRowBlocks][4];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int rb = 0; rb < kRowBlocks; ++rb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][rb][i] = 0.f;

  // weight loads run two steps ahead of the arithmetic (register double buffer)
  auto load_weights = [&](int step, uint4 (&dst)[2][2]) {
    const int k0 = step * 64 + t * 16;
    const bool in_k = step < step_end && k0 < k;   // k % 16 == 0, so a piece is whole or absent
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        dst[j][h] = (in_k && valid[j][h]) ? __ldg(reinterpret_cast<const uint4*>(w_row[j][h] + k0))
                                          : make_uint4(0u, 0u, 0u, 0u);   // code 0
  };
  uint4 wv[2][2], w_next[2][2], w_next2[2][2];
  load_weights(step_begin, wv);
  load_weights(step_begin + 1, w_next);
  for (int step = step_begin; step < step_end; ++step) {
    load_weights(step + 2, w_next2);
    const int k0 = step * 64 + t * 16;          // this lane's 16 K positions
    const bool in_k = k0 < k;
    uint4 xv[kRowBlocks][2];
#pragma unroll
    for (int rb = 0; rb < kRowBlocks; ++rb) {
      if (in_k && x_valid[rb]) {
        const uint4* src = reinterpret_cast<const uint4*>(x_row[rb] + k0);
        xv[rb][0] = __ldg(src);
        xv[rb][1] = __ldg(src + 1);
      } else {
        xv[rb][0] = xv[rb][1] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // MMA i consumes weight bytes 4i..4i+3 and activations 4i..4i+3
      uint32_t b[kRowBlocks][2];
#pragma unroll
      for (int rb = 0; rb < kRowBlocks; ++rb) {
        const uint32_t xw[8] = {xv[rb][0].x, xv[rb][0].y, xv[rb][0].z, xv[rb][0].w,
                                xv[rb][1].x, xv[rb][1].y, xv[rb][1].z, xv[rb][1].w};
        b[rb][0] = xw[2 * i];
        b[rb][1] = xw[2 * i + 1];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint32_t w_lo[4] = {wv[j][0].x, wv[j][0].y, wv[j][0].z, wv[j][0].w};
        const uint32_t w_hi[4] = {wv[j][1].x, wv[j][1].y, wv[j][1].z, wv[j][1].w};
        uint32_t a[4];
        dequant4(w_lo[i] ^ 0x80808080u, scale[j][0], a[0], a[2]);   // row g:   k slots (2t,2t+1), (2t+8,2t+9)
        dequant4(w_hi[i] ^ 0x80808080u, scale[j][1], a[1], a[3]);   // row g+8
#pragma unroll
        for (int rb = 0; rb < kRowBlocks; ++rb) mma_bf16_16816(acc[j][rb], a, b[rb][0], b[rb][1]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        wv[j][h] = w_next[j][h];
        w_next[j][h] = w_next2[j][h];
      }
  }

  // add the K quarters: parts 1..3 park their fragments in shared memory, part 0 finishes
  if (k_part > 0) {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int rb = 0; rb < kRowBlocks; ++rb)
#pragma unroll
        for (int i = 0; i < 4; ++i) partial[k_part - 1][channel_block][j][rb][lane][i] = acc[j][rb][i];
  }
  __syncthreads();
  if (k_part == 0) {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int rb = 0; rb < kRowBlocks; ++rb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float total = acc[j][rb][i];
#pragma unroll
          for (int part = 0; part < kGemvKSplit - 1; ++part) total += partial[part][channel_block][j][rb][lane][i];
          // fragment element i: channel row g (+8 for i >= 2), activation row 2t + (i & 1)
          const int channel = c_base + j * 16 + (i >> 1) * 8 + g;
          const int row = rb * 8 + 2 * t + (i & 1);
          if (channel < n && row < m) out[static_cast<size_t>(row) * n + channel] = __float2bfloat16_rn(total);
        }
      }
  }
}

// ------------------------------------------------------------------ TMA-fed tensor-core version
// gemv_w8a16_tma_kernel: the weight stream goes through shared memory. One producer warp issues
// TMA tile loads of a slab of up to 256 channels x 128 K bytes into a 6-stage ring (the same
// 128-byte-swizzled tiles the W8A8 kernels use); eight consumer warps own 32 channels each, read
// their A fragments with ldmatrix (conflict-free on the swizzled tile; a thread receives the four
// codes at K offsets 4t..4t+3 of a 16-wide segment, which feed one MMA through the same K
// permutation as above), dequantise in registers and run mma.sync. The 16 x 128 activation tile of
// each K block rides in the same stage (two swizzled TMA boxes) and is read with conflict-free
// 8-byte shared loads. HBM only sees the weights, once,
// through deep asynchronous copies instead of register-fed loads.
template <int kRowBlocksT = 1>
struct GemvTmaConfig {
  static constexpr int kBlockK = 128;
  static constexpr int kMaxSlab = 256;
  static constexpr int kWeightBytes = kMaxSlab * kBlockK;   // 32 KB of weights per stage
  static constexpr int kXBoxBytes = 16 * 128;               // 16 activation rows x 64 BF16
  static constexpr int kStageBytes = kWeightBytes + 2 * kXBoxBytes;   // + the 128 K positions of x
  static constexpr int kStages = 6;
  // Up to 8 activation rows: sixteen consumer warps of 16 channels each, four per scheduler, so that one warp's
  // shared-memory and conversion latencies are covered by the others (eight warps of 32 channels left the issue
  // slots half empty while the kernel was still 25 % short of the weight stream's rate: 35.8 -> 33.1 us).
  // 9..16 rows: eight warps of 32 channels, which read each activation fragment once for two channel groups
  // (with sixteen warps the doubled fragment loads took back what the extra warps gave).
  static constexpr int kConsumerWarps = kRowBlocksT == 1 ? 16 : 8;
  static constexpr int kGroups = kRowBlocksT == 1 ? 1 : 2;   // 16-channel groups (A fragments) per consumer warp
  static constexpr int kThreads = (1 + kConsumerWarps) * 32;
  static constexpr int kSmemBytes = kStages * kStageBytes + 256 + 1024;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// map_x: BF16 activations [m, k] as boxes of 64 columns x 16 rows (rows past m read as zero).
template <int kRowBlocks>
__global__ void __launch_bounds__(GemvTmaConfig<kRowBlocks>::kThreads, 1)
gemv_w8a16_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const __nv_bfloat16* __restrict__ sw, __nv_bfloat16* __restrict__ out,
                      int m, int n, int k, int slab) {
  using Cfg = GemvTmaConfig<kRowBlocks>;
  extern __shared__ uint8_t gemv_tma_smem[];
  const uint32_t raw_addr = smem_u32(gemv_tma_smem);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  const uint32_t smem_base = raw_addr + pad;
  const uint32_t bar_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(gemv_tma_smem + pad + Cfg::kStages * Cfg::kStageBytes + 8 * 2 * Cfg::kStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * slab;
  const int num_kb = (k + Cfg::kBlockK - 1) / Cfg::kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), Cfg::kConsumerWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  __syncthreads();
  // launched with programmatic stream serialization: the set-up above may overlap the previous
  // kernel's tail; global memory is touched only after that kernel has finished
  pdl_launch_dependents();
  pdl_wait();

  if (warp == Cfg::kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx = static_cast<uint32_t>(slab) * Cfg::kBlockK + 2 * Cfg::kXBoxBytes;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          __nanosleep(200000);
          break;
        }
        mbar_arrive_expect_tx(full_bar(stage), tx);
        const uint32_t dst = smem_base + stage * Cfg::kStageBytes;
        tma_load_2d(dst, &map_w, kb * Cfg::kBlockK, n0, full_bar(stage));
        tma_load_2d(dst + Cfg::kWeightBytes, &map_x, kb * Cfg::kBlockK, 0, full_bar(stage));
        tma_load_2d(dst + Cfg::kWeightBytes + Cfg::kXBoxBytes, &map_x, kb * Cfg::kBlockK + 64, 0, full_bar(stage));
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  const int g = lane >> 2, t = lane & 3;
  const int c_base = warp * 16 * Cfg::kGroups;        // this warp's first channel within the slab
  const bool warp_active = c_base < slab;
  uint32_t scale[Cfg::kGroups][2];     // the channel's BF16 scale in both halves of a word
#pragma unroll
  for (int j = 0; j < Cfg::kGroups; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int channel = n0 + c_base + j * 16 + h * 8 + g;
      const uint32_t bits = (warp_active && channel < n) ? reinterpret_cast<const uint16_t*>(sw)[channel] : 0u;
      scale[j][h] = bits | (bits << 16);
    }
  // ldmatrix lane addressing: matrix = lane / 8 -> (row half = matrix & 1, segment offset = matrix >> 1)
  const int lm_row = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int lm_seg = lane >> 4;

  float acc[Cfg::kGroups][kRowBlocks][4];
#pragma unroll
  for (int j = 0; j < Cfg::kGroups; ++j)
#pragma unroll
    for (int rb = 0; rb < kRowBlocks; ++rb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[j][rb][i] = 0.f;

  int stage = 0;
  uint32_t phase = 0;
  for (int kb = 0; kb < num_kb; ++kb) {
    // the whole warp leaves together: ldmatrix and mma.sync below are warp-collective
    if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag))) break;
    if (warp_active) {
      const uint32_t tile = smem_base + stage * Cfg::kStageBytes;
      const uint32_t x_tile = tile + Cfg::kWeightBytes;
#pragma unroll
      for (int sp = 0; sp < 4; ++sp) {                // segment pair: 16-wide K segments 2sp and 2sp+1
        // B fragments: the four activations at K offsets 4t..4t+3 of each segment, row g (+8), from
        // the swizzled x boxes (16-byte chunk c of row r lives at chunk c ^ (r & 7))
        uint2 b[kRowBlocks][2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int seg = 2 * sp + half;
          const int chunk = (seg & 3) * 2 + (t >> 1);
          const uint32_t base = x_tile + (seg >> 2) * Cfg::kXBoxBytes + g * 128 + ((chunk ^ g) << 4) + (t & 1) * 8;
#pragma unroll
          for (int rb = 0; rb < kRowBlocks; ++rb) b[rb][half] = lds64(base + rb * 8 * 128);
        }
#pragma unroll
        for (int j = 0; j < Cfg::kGroups; ++j) {
          const int row = c_base + j * 16 + lm_row;   // slab row whose 16-byte chunk this lane addresses
          uint32_t frag[4];                           // (rows 0-7, seg), (rows 8-15, seg), (0-7, seg+1), (8-15, seg+1)
          const int seg = 2 * sp + lm_seg;
          ldmatrix_x4(frag, tile + row * 128 + ((seg ^ (row & 7)) << 4));
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t a[4];
            dequant4_packed(frag[2 * half], scale[j][0], a[0], a[2]);
            dequant4_packed(frag[2 * half + 1], scale[j][1], a[1], a[3]);
#pragma unroll
            for (int rb = 0; rb < kRowBlocks; ++rb) mma_bf16_16816(acc[j][rb], a, b[rb][half].x, b[rb][half].y);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));
    if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
  }

  if (warp_active) {
#pragma unroll
    for (int j = 0; j < Cfg::kGroups; ++j)
#pragma unroll
      for (int rb = 0; rb < kRowBlocks; ++rb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int channel = n0 + c_base + j * 16 + (i >> 1) * 8 + g;
          const int row = rb * 8 + 2 * t + (i & 1);
          if (channel < n && c_base + j * 16 + (i >> 1) * 8 + g < slab && row < m)
            out[static_cast<size_t>(row) * n + channel] = __float2bfloat16_rn(acc[j][rb][i]);
        }
  }
}

// ------------------------------------------------------------------ FMA version (any alignment)
constexpr int kGemvChunk = 2048;   // K elements of every activation row staged per step

template <int kRows, int kChannels>
__global__ void __launch_bounds__(256)
gemv_w8a16_kernel(const __nv_bfloat16* __restrict__ x, const int8_t* __restrict__ w,
                  const __nv_bfloat16* __restrict__ sw, __nv_bfloat16* __restrict__ out,
                  int m, int n, int k) {
  extern __shared__ uint8_t gemv_smem[];
  uint32_t* xs = reinterpret_cast<uint32_t*>(gemv_smem);   // [kRows][kGemvChunk/2] bf16 pairs
  constexpr int kPairs = kGemvChunk / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int first = (blockIdx.x * 8 + warp) * kChannels;

  float acc[kChannels][kRows];
  float scale[kChannels];
#pragma unroll
  for (int c = 0; c < kChannels; ++c) {
    scale[c] = first + c < n ? __bfloat162float(sw[first + c]) : 0.f;
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[c][r] = 0.f;
  }

  for (int k0 = 0; k0 < k; k0 += kGemvChunk) {
    const int span = min(kGemvChunk, k - k0);     // multiple of 16
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * kPairs; i += 256) {
      const int row = i / kPairs, col = i % kPairs;
      xs[i] = (row < m && 2 * col < span)
                  ? reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(row) * k + k0)[col]
                  : 0u;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kChannels; ++c) {
      const int channel = first + c;
      if (channel >= n) break;
      const int8_t* row_w = w + static_cast<size_t>(channel) * k + k0;
#pragma unroll 4
      for (int base = lane * 16; base < span; base += 512) {
        const uint4 packed = __ldg(reinterpret_cast<const uint4*>(row_w + base));
        const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
        float wd[16];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float c0 = static_cast<float>(static_cast<int8_t>(words[j >> 2] >> ((j & 3) * 8)));
          const float c1 = static_cast<float>(static_cast<int8_t>(words[j >> 2] >> (((j + 1) & 3) * 8)));
          const __nv_bfloat162 pair =
              __floats2bfloat162_rn(__fmul_rn(c0, scale[c]), __fmul_rn(c1, scale[c]));
          const float2 f = __bfloat1622float2(pair);
          wd[j] = f.x;
          wd[j + 1] = f.y;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const uint4* xv = reinterpret_cast<const uint4*>(xs + r * kPairs + (base >> 1));
          const uint4 x0 = xv[0], x1 = xv[1];
          const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[c][r] = fmaf(__uint_as_float(xw[j] << 16), wd[2 * j], acc[c][r]);
            acc[c][r] = fmaf(__uint_as_float(xw[j] & 0xffff0000u), wd[2 * j + 1], acc[c][r]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kChannels; ++c) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float total = acc[c][r];
#pragma unroll
      for (int delta = 16; delta; delta >>= 1) total += __shfl_xor_sync(0xffffffffu, total, delta);
      if (lane == 0 && r < m && first + c < n)
        out[static_cast<size_t>(r) * n + first + c] = __float2bfloat16_rn(total);
    }
  }
}

}  // namespace ci8

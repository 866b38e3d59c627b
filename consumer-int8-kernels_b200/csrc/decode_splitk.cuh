// Small-M (<= 16 rows) W8A8 linear for decode: an HBM-streaming kernel.
//
// The weight matrix W [N,K] is read exactly once. The roles of the MMA operands are swapped
// with respect to the prefill GEMM: a slab of up to 256 output channels is the M side of
// tcgen05.mma (two M=128 instructions over rows [0,128) and [C-128,C) of the slab), and the
// (zero-padded) 16 activation rows are the N side, so the accumulator in TMEM is
// [channel, row] and 32 TMEM columns suffice. One CTA streams one slab through a deep TMA ring;
// the slab width C is chosen on the host so that the slabs fill the SMs in one wave.
//
// Split-K: a cluster of kSplit CTAs shares a slab, each streaming its own K range; the
// non-leader CTAs push their INT32 partials into the leader's shared memory (DSMEM) and the
// leader adds them — integer addition, so the result does not depend on the split.
//
// UINT8 weights (code+128): the MMA reads them as unsigned, and the epilogue removes
// 128 * sum_k a[row,k], computed by the epilogue warps from the INT8 activations.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"

namespace ci8 {

struct DecodeParams {
  const int8_t* a;            // [M,K] INT8 activations (for the UINT8-weight row sums)
  const float* sa;            // [M]
  const __nv_bfloat16* sw;    // [N]
  __nv_bfloat16* out;         // [M,N]
  int32_t* workspace;         // optional [M,N] INT32 accumulators
  int m, n, k;
  int slab;                   // channels per CTA (multiple of 16, 128..256)
};

template <int kSplit>
struct DecodeConfig {
  static constexpr int kRows = 16;                       // padded activation rows (MMA N)
  static constexpr int kBlockK = 128;
  static constexpr int kMaxSlab = 256;
  static constexpr int kWBytes = kMaxSlab * kBlockK;     // 32 KB
  static constexpr int kABytes = kRows * kBlockK;        // 2 KB
  static constexpr int kStageBytes = kWBytes + kABytes;
  static constexpr int kStages = kSplit == 1 ? 6 : 5;
  static constexpr int kReduceBytes = kSplit == 1 ? 0 : (kSplit - 1) * 2 * 128 * kRows * 4;
  static constexpr int kThreads = 192;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kReduceBytes + kBarrierBytes + 1024;
};

template <int kSplit, bool kBiased>
__global__ void __launch_bounds__(192, 1)
decode_w8a8_kernel(const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_a, const DecodeParams p) {
  using Cfg = DecodeConfig<kSplit>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  int32_t* reduce_buf = reinterpret_cast<int32_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint8_t* bar_region = smem + Cfg::kStages * Cfg::kStageBytes + Cfg::kReduceBytes;
  const uint32_t bar_base = smem_base + Cfg::kStages * Cfg::kStageBytes + Cfg::kReduceBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  const uint32_t done_bar = bar_base + 8u * (2 * Cfg::kStages);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_region + 8 * (2 * Cfg::kStages + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int32_t* row_sums = reinterpret_cast<int32_t*>(tmem_slot + 2);   // [16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = kSplit > 1 ? cluster_ctarank() : 0u;
  const int slab_index = blockIdx.x / kSplit;
  const int n0 = slab_index * p.slab;
  const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;
  const int kb_begin = static_cast<int>((static_cast<long long>(num_kb) * rank) / kSplit);
  const int kb_end = static_cast<int>((static_cast<long long>(num_kb) * (rank + 1)) / kSplit);
  const bool second_half = p.slab > 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(done_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_a);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), 32);
    tmem_relinquish<1>();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx = static_cast<uint32_t>(p.slab) * Cfg::kBlockK + Cfg::kABytes;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          __nanosleep(200000);
          break;
        }
        mbar_arrive_expect_tx(full_bar(stage), tx);
        const uint32_t w_dst = smem_base + stage * Cfg::kStageBytes;
        tma_load_2d(w_dst, &map_w, kb * Cfg::kBlockK, n0, full_bar(stage));
        tma_load_2d(w_dst + Cfg::kWBytes, &map_a, kb * Cfg::kBlockK, 0, full_bar(stage));
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // "A" operand = weights (unsigned when biased), "B" operand = activations (signed).
      constexpr uint32_t kIdesc = idesc_i8(128, Cfg::kRows, /*b_unsigned=*/false, /*a_unsigned=*/kBiased);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t w_addr = smem_base + stage * Cfg::kStageBytes;
        const uint64_t w_desc0 = smem_desc_sw128(w_addr);
        const uint64_t w_desc1 = smem_desc_sw128(w_addr + (p.slab - 128) * Cfg::kBlockK);
        const uint64_t a_desc = smem_desc_sw128(w_addr + Cfg::kWBytes);
        const uint32_t first = kb == kb_begin ? 0u : 1u;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          mma_i8<1>(tmem_base, w_desc0 + 2u * ks, a_desc + 2u * ks, kIdesc, first | (ks != 0));
          if (second_half)
            mma_i8<1>(tmem_base + Cfg::kRows, w_desc1 + 2u * ks, a_desc + 2u * ks, kIdesc,
                      first | (ks != 0));
        }
        mma_commit(empty_bar(stage));
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) mma_commit(done_bar);
    }
  } else {
    // -------------------------------------------------------------- epilogue warps (128 threads)
    const int t = threadIdx.x - 64;              // 0..127
    const int quarter = warp & 3;                // TMEM lane quarter of this warp
    const int tmem_lane = quarter * 32 + lane;   // accumulator row = channel within the half
    if constexpr (kBiased) {
      // sum_k a[row,k] over this CTA's K range: 8 threads per activation row.
      const int row = t >> 3, part = t & 7;
      int sum = 0;
      if (row < p.m) {
        const int k_begin = kb_begin * Cfg::kBlockK, k_end = min(kb_end * Cfg::kBlockK, p.k);
        const int8_t* src = p.a + static_cast<size_t>(row) * p.k;
        if (reinterpret_cast<uintptr_t>(p.a) % 16 == 0 && p.k % 16 == 0) {
          for (int k = k_begin + part * 16; k < k_end; k += 128) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + k);
            sum = __dp4a(static_cast<int>(v.x), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.y), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.z), 0x01010101, sum);
            sum = __dp4a(static_cast<int>(v.w), 0x01010101, sum);
          }
        } else {
          for (int k = k_begin + part; k < k_end; k += 8) sum += src[k];
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      if (part == 0) row_sums[row] = sum;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const bool ok = kb_end > kb_begin
                        ? mbar_wait(done_bar, 0u, abort_flag)
                        : true;
    tcgen05_fence_after();
    int32_t acc[2][16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t v[16];
      if (ok && kb_end > kb_begin && (h == 0 || second_half)) {
        tmem_ld_32x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + h * Cfg::kRows, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        acc[h][j] = static_cast<int32_t>(v[j]);
        if constexpr (kBiased) acc[h][j] -= 128 * row_sums[j];
      }
    }
    if constexpr (kSplit > 1) {
      if (rank != 0) {
        // push partials into the leader's reduce buffer: [rank-1][half][row j][channel lane]
        const uint32_t remote = map_to_cta(smem_u32(reduce_buf), 0);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t offset = ((((rank - 1) * 2 + h) * 16 + j) * 128 + tmem_lane) * 4;
            asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + offset), "r"(acc[h][j]) : "memory");
          }
      }
    }
    if constexpr (kSplit > 1) {
      cluster_arrive();
      cluster_wait();
    }
    if (rank == 0) {
      if constexpr (kSplit > 1) {
#pragma unroll
        for (int r = 0; r < kSplit - 1; ++r)
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              acc[h][j] += reduce_buf[((r * 2 + h) * 16 + j) * 128 + tmem_lane];
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !second_half) break;
        const int local = h == 0 ? tmem_lane : p.slab - 128 + tmem_lane;
        if (h == 1 && local < 128) continue;        // already produced by the first half
        const int channel = n0 + local;
        if (local >= p.slab || channel >= p.n) continue;
        const float channel_scale = __bfloat162float(p.sw[channel]);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j < p.m) {
            const float scaled = __fmul_rn(__int2float_rn(acc[h][j]), p.sa[j]);
            p.out[static_cast<size_t>(j) * p.n + channel] =
                __float2bfloat16_rn(__fmul_rn(scaled, channel_scale));
            if (p.workspace) p.workspace[static_cast<size_t>(j) * p.n + channel] = acc[h][j];
          }
        }
      }
    }
  }
  if constexpr (kSplit > 1) {
    if (warp < 2) {   // the epilogue warps passed the cluster rendezvous above
      cluster_arrive();
      cluster_wait();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc<1>(tmem_base, 32);
  }
}

}  // namespace ci8

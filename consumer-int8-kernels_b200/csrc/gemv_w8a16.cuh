// W8A16 small-batch linear: BF16 activations times BF16-rounded dequantized INT8 weights with
// FP32 accumulation:  wd[n,k] = bf16(float(code[n,k]) * float(sw[n])),
//                     out[m,n] = bf16(sum_k x[m,k] * wd[n,k]).
// HBM-bound on the weight stream, which is read exactly once. A warp owns kChannels output
// channels; each lane reads 16 bytes of weights per 512-wide K step. The activation rows are
// staged in shared memory in K chunks shared by the whole CTA, so the weight stream is the
// only global traffic in the inner loop.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace ci8 {

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

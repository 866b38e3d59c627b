// unpack_allspark: restores row-major signed INT8 weights [N,K] and channel scales [N] from the
// AllSpark "N32K16" storage (UINT8 code+128, rows padded to a multiple of 32) without touching
// the values. HBM-bound byte permutation: 1 byte read + 1 byte written per weight.
//
// Storage, as the reference's inverse defines it (csrc/allspark_layout.cu:8-28 in the reference):
// packed row P = (n / 32) * 8 + n % 8 holds, for every 16-wide K tile t, one 64-byte cell at byte
// offset P*4K + 64t that interleaves the four channels n, n+8, n+16, n+24 of that 32-block:
// 16-byte quarter q (0..3) carries, for channel n + 8c (c = 0..3), the four bytes at 4c..4c+3 of
// the quarter = K positions {2q, 2q+1, 8+2q, 8+2q+1} of the tile.
// One thread owns one cell: four coalesced 16-byte loads, four 16-byte stores (one per channel);
// a warp covers 32 consecutive tiles, so every store instruction writes 512 contiguous bytes.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace ci8 {

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
  return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

__global__ void __launch_bounds__(256)
unpack_allspark_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ packed_scales,
                       int8_t* __restrict__ weight, uint16_t* __restrict__ scales, int n, int k) {
  const int tiles = k >> 4;
  const int64_t cell = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  const int64_t cells = static_cast<int64_t>((n + 31) / 32 * 8) * tiles;
  if (cell >= cells) return;
  const int packed_row = static_cast<int>(cell / tiles);
  const int tile = static_cast<int>(cell - static_cast<int64_t>(packed_row) * tiles);
  const uint4* src = reinterpret_cast<const uint4*>(packed + static_cast<int64_t>(packed_row) * k * 4 + tile * 64);
  const uint4 q0 = __ldg(src), q1 = __ldg(src + 1), q2 = __ldg(src + 2), q3 = __ldg(src + 3);
  const int first = (packed_row >> 3) * 32 + (packed_row & 7);     // channel n of this cell
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int row = first + 8 * c;
    if (row >= n) continue;                                       // padding rows of the last block
    const uint32_t a = word_of(q0, c), b = word_of(q1, c), cc = word_of(q2, c), d = word_of(q3, c);
    uint4 restored;
    restored.x = ((a & 0xffffu) | (b << 16)) ^ 0x80808080u;       // K 0..3   (code + 128 -> signed)
    restored.y = ((cc & 0xffffu) | (d << 16)) ^ 0x80808080u;      // K 4..7
    restored.z = ((a >> 16) | (b & 0xffff0000u)) ^ 0x80808080u;   // K 8..11
    restored.w = ((cc >> 16) | (d & 0xffff0000u)) ^ 0x80808080u;  // K 12..15
    reinterpret_cast<uint4*>(weight + static_cast<int64_t>(row) * k)[tile] = restored;
    if (tile == 0) scales[row] = packed_scales[(row / 32) * 32 + (row % 8) * 4 + (row % 32) / 8];
  }
}

}  // namespace ci8

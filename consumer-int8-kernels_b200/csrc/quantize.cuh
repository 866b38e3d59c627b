// Dynamic per-row activation quantizer: BF16 -> signed INT8 codes + one FP32 scale per row
// (or per row and 4096-channel group).
//
//   scale = max(absmax / 127, 1e-20)                 IEEE division
//   code  = clamp(rint_even(x / scale), -127, 127)   IEEE division, round half to even
//
// HBM-bound (2 bytes read + 1 byte written per element). Each row is read once: a team of
// threads (one warp for narrow rows, one 256-thread CTA otherwise) holds the row in registers as
// 16-byte packs across the absmax reduction, then writes 8-byte packs of codes.
//
// The per-element IEEE division would make the kernel instruction-bound, so the common case
// takes a short path that provably gives the same bits: q' = x * (1/scale) is within 2.3e-5 of
// the correctly rounded quotient for |q| <= 127, so whenever q' is farther than 5e-5 from a
// half-integer, rint(q') equals rint of the IEEE quotient; rounding and the integer conversion
// are one FADD with 1.5*2^23 (the low byte of the sum is the two's-complement code). A pack that
// holds a value too close to a tie, a NaN or an infinity is redone with the IEEE division.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>
#include "sm100_ptx.cuh"

namespace ci8 {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// The reference arithmetic, literally.
__device__ __forceinline__ int quantize_one(float v, float scale) {
  return max(-127, min(127, __float2int_rn(__fdiv_rn(v, scale))));
}
constexpr float kRoundMagic = 12582912.f;   // 1.5 * 2^23
constexpr float kTieGuard = 0.49995f;       // |q' - rint(q')| below this: no tie within the error bound

// Short path for two values with packed FP32 arithmetic (two IEEE-rounded lanes per instruction):
// returns the FMA results whose low bytes are the codes and clears `safe` when a value is not
// provably away from a rounding tie. shifted = RN(v * inverse + 1.5 * 2^23) is the exact product
// rounded to the nearest integer (ties to even); the last FMA gives the exact product's distance
// from that integer. |v * inverse - v / scale| <= 127.5 * 2^-24 and the reference's own rounding of
// v / scale moves it by as much again, so outside the guard band both round alike. NaN compares
// false, so NaN and inf * 0 land on the exact path too.
// `worst` collects the largest |residual| of a pack with one instruction per value (magnitude of the
// larger operand, NaN kept), so the pack needs a single comparison at its end.
__device__ __forceinline__ float max_abs_keep_nan(float a, float b) {
  float r;
  asm("max.NaN.xorsign.abs.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float2 quantize_fast2(float2 v, float2 inverse, float& worst) {
  const float2 magic = make_float2(kRoundMagic, kRoundMagic);
  const float2 shifted = __ffma2_rn(v, inverse, magic);
  const float2 minus_rounded = __ffma2_rn(shifted, make_float2(-1.f, -1.f), magic);   // exact
  const float2 residual = __ffma2_rn(v, inverse, minus_rounded);
  worst = max_abs_keep_nan(max_abs_keep_nan(worst, residual.x), residual.y);
  return shifted;
}
// The same test for one value (used by the repair path to find the offender).
__device__ __forceinline__ bool away_from_tie(float v, float inverse) {
  const float shifted = __fmaf_rn(v, inverse, kRoundMagic);
  const float residual = __fmaf_rn(v, inverse, -__fsub_rn(shifted, kRoundMagic));
  return fabsf(residual) < kTieGuard;
}

// Running maximum of |x| over packed BF16 pairs: one packed instruction per two values (the larger
// magnitude of each half; the sign bits it returns are meaningless and are masked where the maximum is
// read). It returns the other operand when one is NaN, which is what fmaxf does.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t running, uint32_t pair) {
  uint32_t result;
  asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(result) : "r"(running), "r"(pair));
  return result;
}
// The two maxima of a running packed maximum, as non-negative floats.
__device__ __forceinline__ float absmax_lo(uint32_t running) { return __uint_as_float((running << 16) & 0x7fffffffu); }
__device__ __forceinline__ float absmax_hi(uint32_t running) { return __uint_as_float(running & 0x7fff0000u); }

// Eight BF16 values (one 16-byte pack) -> eight codes (8 bytes). BF16 inputs hit exact rounding ties
// far more often than random reals would (x * 127 / absmax is a ratio of small integers): about one
// warp-pack in eight holds one, so the repair redoes only the offending values, each with the
// reference's division, instead of the whole pack.
__device__ __forceinline__ uint2 quantize_pack(const uint4& pack, float scale, float inverse) {
  const float v[8] = {bf16_lo(pack.x), bf16_hi(pack.x), bf16_lo(pack.y), bf16_hi(pack.y),
                      bf16_lo(pack.z), bf16_hi(pack.z), bf16_lo(pack.w), bf16_hi(pack.w)};
  const float2 inverse2 = make_float2(inverse, inverse);
  uint32_t t[8];
  float worst = 0.f;
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    const float2 shifted = quantize_fast2(make_float2(v[j], v[j + 1]), inverse2, worst);
    t[j] = __float_as_uint(shifted.x);
    t[j + 1] = __float_as_uint(shifted.y);
  }
  if (!(fabsf(worst) < kTieGuard)) {   // also taken when a residual is NaN (NaN or infinite inputs)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (!away_from_tie(v[j], inverse)) t[j] = static_cast<uint32_t>(quantize_one(v[j], scale));
  }
  const uint32_t lo = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410);
  const uint32_t hi = __byte_perm(__byte_perm(t[4], t[5], 0x0040), __byte_perm(t[6], t[7], 0x0040), 0x5410);
  return make_uint2(lo, hi);
}

// Rows are walked in INPUT order so that consecutive teams read consecutive memory. Input row i:
//   plain   : output row i
//   grouped : i = r*G + g (input [M,G,4096]) writes output row g*M + r (output [G,M,4096])
__device__ __forceinline__ int64_t output_row_of(int64_t i, int m, int groups) {
  return groups > 0 ? (i % groups) * static_cast<int64_t>(m) + i / groups : i;
}

// SwiGLU of one gate/up pair as the reference computes it (csrc/silu_quant.cu:30-33 in the
// reference): silu = gate / (1 + expf(-gate)) with the fast division, product rounded to BF16.
__device__ __forceinline__ float swiglu_one(float gate, float up) {
  const float silu = __fdividef(gate, 1.f + expf(-gate));
  return __fmul_rn(silu, up);
}
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t gate, uint32_t up) {
  __nv_bfloat162 r = __floats2bfloat162_rn(swiglu_one(bf16_lo(gate), bf16_lo(up)),
                                           swiglu_one(bf16_hi(gate), bf16_hi(up)));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint4 swiglu_pack(const uint4& gate, const uint4& up) {
  return make_uint4(swiglu_pair(gate.x, up.x), swiglu_pair(gate.y, up.y), swiglu_pair(gate.z, up.z),
                    swiglu_pair(gate.w, up.w));
}

// Loads one row as 16-byte packs of BF16. kSwiGLU: the input row is [gate(k) | up(k)] and the
// packs hold bf16(silu(gate) * up), i.e. exactly what a separate silu_mul would have written.
template <int kTeam, int kPacks, bool kSwiGLU = false>
__device__ __forceinline__ void load_row(uint4 (&pack)[kPacks], const uint16_t* x, int64_t row, int64_t rows,
                                         int k, int member) {
  const int64_t pitch = kSwiGLU ? 2 * static_cast<int64_t>(k) : k;
  const uint4* src = reinterpret_cast<const uint4*>(x + (row < rows ? row : 0) * pitch);
  const int packs_in_row = k >> 3;
#pragma unroll
  for (int i = 0; i < kPacks; ++i) {
    const int index = i * kTeam + member;
    const bool live = row < rows && index < packs_in_row;
    if constexpr (kSwiGLU) {
      pack[i] = live ? swiglu_pack(__ldg(src + index), __ldg(src + packs_in_row + index)) : make_uint4(0, 0, 0, 0);
    } else {
      pack[i] = live ? __ldg(src + index) : make_uint4(0, 0, 0, 0);
    }
  }
}

// kTeam threads per row (32, 128, 256 or 512), kPacks 16-byte packs per thread; 256 threads per CTA
// (512 when the team is that wide). Rows of up to 3 packs per thread run one team per row with many small CTAs resident (measured
// faster there); wider rows (4..9 packs) use a persistent grid in which a team strides over the
// rows and loads its next row before it reduces and converts the current one, so loads stay in
// flight during the arithmetic. The code is the same: the launch decides the grid.
// Requires 16-byte aligned rows of x (k % 8 == 0, base aligned) and 8-byte aligned q.
// kSwiGLU fuses silu(gate)*up in front of the quantizer (silu_mul_quantize).
template <int kTeam, int kPacks, bool kSwiGLU = false>
__global__ void __launch_bounds__(kTeam > 256 ? kTeam : 256)
quantize_rows_vec_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ q,
                         float* __restrict__ scales, int rows, int k, int m, int groups) {
  constexpr int kThreads = kTeam > 256 ? kTeam : 256;   // a team wider than 256 threads is one CTA
  constexpr int kRowsPerCta = kThreads / kTeam;
  constexpr int kWarps = kThreads / 32;
  constexpr bool kPrefetch = !kSwiGLU && kPacks >= 4 && kPacks <= 9;
  __shared__ float maxima[2][kWarps];
  const int member = threadIdx.x % kTeam;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  const int packs_in_row = k >> 3;
  int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + threadIdx.x / kTeam;

  // launched with programmatic stream serialization: the next kernel may start its prologue now,
  // and nothing is read before the previous kernel in the stream has finished
  pdl_launch_dependents();
  pdl_wait();

  uint4 pack[kPacks];
  uint4 next[kPrefetch ? kPacks : 1];
  load_row<kTeam, kPacks, kSwiGLU>(pack, x, row, rows, k, member);
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * kRowsPerCta, iter = 0; base < rows;
       base += stride, row += stride, ++iter) {
    if constexpr (kPrefetch) load_row<kTeam, kPacks, kSwiGLU>(next, x, row + stride, rows, k, member);
    uint32_t packed_max = 0u;
#pragma unroll
    for (int i = 0; i < kPacks; ++i) {
      packed_max = absmax_bf16x2(packed_max, pack[i].x);
      packed_max = absmax_bf16x2(packed_max, pack[i].y);
      packed_max = absmax_bf16x2(packed_max, pack[i].z);
      packed_max = absmax_bf16x2(packed_max, pack[i].w);
    }
    float maximum = fmaxf(absmax_lo(packed_max), absmax_hi(packed_max));
#pragma unroll
    for (int mask = 16; mask; mask >>= 1)
      maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, mask));
    if constexpr (kTeam > 32) {
      constexpr int kWarpsPerTeam = kTeam / 32;
      float* slot = maxima[iter & 1] + (threadIdx.x / kTeam) * kWarpsPerTeam;   // alternating slots: one barrier per row
      if ((threadIdx.x & 31) == 0) slot[(threadIdx.x % kTeam) >> 5] = maximum;
      __syncthreads();
      maximum = slot[0];
#pragma unroll
      for (int i = 1; i < kWarpsPerTeam; ++i) maximum = fmaxf(maximum, slot[i]);
    }
    const float scale = fmaxf(__fdiv_rn(maximum, 127.f), 1e-20f);
    const float inverse = __fdiv_rn(1.f, scale);
    if (row < rows) {
      const int64_t out_row = output_row_of(row, m, groups);
      if (member == 0) scales[out_row] = scale;
      uint2* dst = reinterpret_cast<uint2*>(q + out_row * k);
#pragma unroll
      for (int i = 0; i < kPacks; ++i) {
        const int index = i * kTeam + member;
        if (index < packs_in_row) dst[index] = quantize_pack(pack[i], scale, inverse);
      }
    }
    if constexpr (kPrefetch) {
#pragma unroll
      for (int i = 0; i < kPacks; ++i) pack[i] = next[i];
    } else {
      load_row<kTeam, kPacks, kSwiGLU>(pack, x, row + stride, rows, k, member);
    }
  }
}

// silu_mul: out[m, k] = bf16(silu(x[m, :k]) * x[m, k:]); one 16-byte pack of outputs per thread.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int64_t packs, int packs_in_row) {
  const int64_t index = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (index >= packs) return;
  const int64_t row = index / packs_in_row;
  const int col = static_cast<int>(index - row * packs_in_row);
  const uint4* src = reinterpret_cast<const uint4*>(x) + row * 2 * packs_in_row;
  reinterpret_cast<uint4*>(out)[index] = swiglu_pack(__ldg(src + col), __ldg(src + packs_in_row + col));
}

// Any width and alignment: one CTA per row, two passes over the row (the second one hits L1/L2).
__global__ void __launch_bounds__(256)
quantize_rows_generic_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ q,
                             float* __restrict__ scales, int k) {
  __shared__ float maxima[8];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * k;
  float maximum = 0.f;
  for (int c = threadIdx.x; c < k; c += 256)
    maximum = fmaxf(maximum, fabsf(__uint_as_float(static_cast<uint32_t>(x[base + c]) << 16)));
#pragma unroll
  for (int mask = 16; mask; mask >>= 1)
    maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, mask));
  if ((threadIdx.x & 31) == 0) maxima[threadIdx.x >> 5] = maximum;
  __syncthreads();
  maximum = maxima[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) maximum = fmaxf(maximum, maxima[i]);
  const float scale = fmaxf(__fdiv_rn(maximum, 127.f), 1e-20f);
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
  for (int c = threadIdx.x; c < k; c += 256)
    q[base + c] = static_cast<int8_t>(
        quantize_one(__uint_as_float(static_cast<uint32_t>(x[base + c]) << 16), scale));
}

}  // namespace ci8

/*
 * Scalar C restatement of the reference's W8A8 linear arithmetic. TEST INFRASTRUCTURE ONLY:
 * it is a second, independent checker beside oracle/w8a8_ref.py (plain loops, no vector
 * library), used by the test suite and by the CPU-baseline leg of the benchmark. The shipped
 * library never links or loads it.
 *
 * Parity status: PINNED against the reference's known-answer vectors (tests/golden) and
 * against oracle/w8a8_ref.py on seeded inputs (tests/test_oracle.py).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off).
 *
 * Reference anchors (paths inside the reference project):
 *   quantizer  csrc/kernels.cu:13-35        product   csrc/kernels.cu:95-114, tests/test_cuda_ops.py:488,596
 *   epilogue   csrc/kernels.cu:120          grouped   csrc/kernels.cu:47-48
 *   block-32   benchmarks/cuda/q8_block_int8.cu:11-69 (quantizer and per-block rescaled product)
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* Round to nearest even, NaN stays NaN (quiet), as cvt.rn.bf16.f32 does. */
static uint16_t f32_to_bf16(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

/* csrc/kernels.cu:13-35 — absmax, scale = max(absmax/127, 1e-20), round-half-even, clamp ±127. */
void ci8o_quantize_rows(const uint16_t* x, int8_t* q, float* scales, int m, int k) {
  for (int r = 0; r < m; ++r) {
    float maximum = 0.f;
    for (int c = 0; c < k; ++c) maximum = fmaxf(maximum, fabsf(bf16_to_f32(x[(int64_t)r * k + c])));
    const float scale = fmaxf(maximum / 127.f, 1e-20f);
    scales[r] = scale;
    for (int c = 0; c < k; ++c) {
      const float v = bf16_to_f32(x[(int64_t)r * k + c]) / scale;
      int code = 0;
      if (v == v) { /* __float2int_rn(NaN) == 0 */
        const float rounded = nearbyintf(v); /* default mode: ties to even */
        code = rounded > 127.f ? 127 : rounded < -127.f ? -127 : (int)rounded;
      }
      q[(int64_t)r * k + c] = (int8_t)code;
    }
  }
}

/* csrc/kernels.cu:47-48,293-298 — input [M,G,4096], output group-major [G,M,4096], scales [G,M]. */
void ci8o_quantize_grouped4096(const uint16_t* x, int8_t* q, float* scales, int m, int groups) {
  for (int g = 0; g < groups; ++g)
    for (int r = 0; r < m; ++r)
      ci8o_quantize_rows(x + ((int64_t)r * groups + g) * 4096, q + ((int64_t)g * m + r) * 4096,
                         scales + (int64_t)g * m + r, 1, 4096);
}

/* tests/test_cuda_ops.py:488,596 — exact INT32 product; UINT8 weights hold code + 128. */
void ci8o_int_mm(const int8_t* a, const void* w, int w_is_u8, int32_t* acc, int m, int n, int k) {
  const int8_t* ws = (const int8_t*)w;
  const uint8_t* wu = (const uint8_t*)w;
  for (int c = 0; c < n; ++c)
    for (int r = 0; r < m; ++r) {
      int32_t sum = 0;
      for (int i = 0; i < k; ++i) {
        const int wv = w_is_u8 ? (int)wu[(int64_t)c * k + i] - 128 : (int)ws[(int64_t)c * k + i];
        sum += (int)a[(int64_t)r * k + i] * wv;
      }
      acc[(int64_t)r * n + c] = sum;
    }
}

/* csrc/kernels.cu:120 — bf16((float(acc) * sa[row]) * float(sw[col])), two FP32 roundings. */
void ci8o_epilogue(const int32_t* acc, const float* sa, const uint16_t* sw, uint16_t* out, int m, int n) {
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < n; ++c) {
      volatile float scaled = (float)acc[(int64_t)r * n + c] * sa[r];
      out[(int64_t)r * n + c] = f32_to_bf16(scaled * bf16_to_f32(sw[c]));
    }
}

/* Grouped-scale sum: per group INT32 partial * sa[g,row], FP32 adds in ascending group order,
 * then the channel scale, then BF16. acc is [G,M,N]. One group reduces to ci8o_epilogue. */
void ci8o_grouped_epilogue(const int32_t* acc, const float* sa, const uint16_t* sw, uint16_t* out,
                           int groups, int m, int n) {
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < n; ++c) {
      volatile float total = 0.f;
      for (int g = 0; g < groups; ++g) {
        volatile float term = (float)acc[((int64_t)g * m + r) * n + c] * sa[(int64_t)g * m + r];
        total = g ? total + term : term;
      }
      out[(int64_t)r * n + c] = f32_to_bf16(total * bf16_to_f32(sw[c]));
    }
}

/* IEEE binary16 -> binary32 (exact). */
static float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exponent = (h >> 10) & 0x1fu, mantissa = h & 0x3ffu, bits;
  if (exponent == 0) {
    if (mantissa == 0) {
      bits = sign;
    } else {
      int shift = 0;
      while (!(mantissa & 0x400u)) { mantissa <<= 1; ++shift; }
      mantissa &= 0x3ffu;
      bits = sign | ((uint32_t)(113 - shift) << 23) | (mantissa << 13);
    }
  } else if (exponent == 31) {
    bits = sign | 0x7f800000u | (mantissa << 13);
  } else {
    bits = sign | ((exponent + 112) << 23) | (mantissa << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* benchmarks/cuda/q8_block_int8.cu:11-24 — one scale per 32 values, scale = max(absmax/127, 1e-20),
 * code = int8(round_half_even(v / scale)); NaN quotients give 0 as __float2int_rn does. */
void ci8o_q8_block_quantize(const uint16_t* x, int8_t* q, float* scales, int64_t blocks) {
  for (int64_t b = 0; b < blocks; ++b) {
    float maximum = 0.f;
    for (int i = 0; i < 32; ++i) maximum = fmaxf(maximum, fabsf(bf16_to_f32(x[b * 32 + i])));
    const float scale = fmaxf(maximum / 127.f, 1e-20f);
    for (int i = 0; i < 32; ++i) {
      const float quotient = bf16_to_f32(x[b * 32 + i]) / scale;
      q[b * 32 + i] = isnan(quotient) ? 0 : (int8_t)rintf(quotient);
    }
    scales[b] = scale;
  }
}

/* benchmarks/cuda/q8_block_int8.cu:26-69 — per 32-wide block an INT32 dot product, then
 * sum = fma(float(dot), sa * sw, sum) in ascending block order (the contracted form of the
 * reference's `sum += float(acc) * (sa * sw)`), rounded to BF16 at the end. sw is FP16. */
void ci8o_q8_block_mm(const int8_t* a, const int8_t* w, const float* sa, const uint16_t* sw, uint16_t* y, int m,
                      int n, int k) {
  const int blocks = k / 32;
  for (int r = 0; r < m; ++r)
    for (int c = 0; c < n; ++c) {
      float sum = 0.f;
      for (int b = 0; b < blocks; ++b) {
        int32_t dot = 0;
        for (int i = 0; i < 32; ++i)
          dot += (int32_t)a[(int64_t)r * k + b * 32 + i] * (int32_t)w[(int64_t)c * k + b * 32 + i];
        const float scale = sa[(int64_t)r * blocks + b] * f16_to_f32(sw[(int64_t)c * blocks + b]);
        sum = fmaf((float)dot, scale, sum);
      }
      y[(int64_t)r * n + c] = f32_to_bf16(sum);
    }
}

/* Host twin of the reference's raw C entry point (benchmarks/cuda/q8_block_int8.cu:150-160, bound with
 * ctypes at benchmarks/benchmark_q8_block_int8.py:36-39): same name, same argument order, HOST
 * pointers, stream ignored. With it the reference's own validation script can be run against this
 * checker on a machine without a GPU (tests/golden/run_reference_q8_validator.py). */
int q8_block_int8(const void* x, void* a, void* sa, const void* w, const void* sw, void* y, int m, int n, int k,
                  void* stream) {
  (void)stream;
  if (m <= 0 || n <= 0 || k <= 0 || k % 32) return 1;
  ci8o_q8_block_quantize((const uint16_t*)x, (int8_t*)a, (float*)sa, (int64_t)m * (k / 32));
  ci8o_q8_block_mm((const int8_t*)a, (const int8_t*)w, (const float*)sa, (const uint16_t*)sw, (uint16_t*)y, m, n, k);
  return 0;
}

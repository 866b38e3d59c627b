"""CPU oracle for the dynamic-quantization W8A8 linear path. TEST INFRASTRUCTURE ONLY.

This module restates, with torch on the host, the arithmetic that the reference
(AppMana/consumer-int8-kernels) pins for its six linear-path operators. It is the
checker for the CUDA kernels: only the test suite, the smoke check and the CPU
baseline leg of the benchmark may import it. Nothing in the shipped package does.

Parity status: PINNED. Every function below is checked against the known-answer
vectors the reference's own tests hold for this path (tests/golden/*.json, built
by tests/golden/make_golden.py) and, for the weight encoding, against outputs of
the reference's importable ``consumer_int8.quantization`` module.

Reference anchors (paths inside the reference project):
  * activation quantizer   csrc/kernels.cu:27-33,70,81-82 (IEEE divide, round
    half to even via __float2int_rn, clamp to [-127,127], scale floor 1e-20);
    torch restatement at benchmarks/microbench_quantize.py:75-76
  * grouped quantizer      csrc/kernels.cu:47-48,293-298; tests/test_cuda_ops.py:31-38
  * integer product        tests/test_cuda_ops.py:488 (UINT8-128) and :596 (INT8)
  * epilogue               tests/test_cuda_ops.py:489,599; csrc/kernels.cu:120
  * W8A16 GEMV             tests/test_gemv.py:26-29
  * weight encoding        src/consumer_int8/quantization.py:22-32
"""

from __future__ import annotations

import torch

__all__ = [
    "quantize_rows_ref",
    "quantize_grouped4096_ref",
    "int_mm_literal",
    "int_mm_fast",
    "epilogue_ref",
    "fused_channel_mm_ref",
    "channel_mm_ref",
    "channel_gemv_ref",
    "channel_gemv_fp64",
    "grouped_channel_mm_ref",
    "quantize_channel_ref",
    "silu_mul_ref",
    "unpack_allspark_ref",
    "pack_allspark_ref",
]


# --------------------------------------------------------------------------- #
# Activation quantizers
# --------------------------------------------------------------------------- #
def quantize_rows_ref(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M,K] -> (INT8 codes [M,K], FP32 scales [M]).

    Follows csrc/kernels.cu:27-33: ``scale = fmaxf(absmax / 127.f, 1e-20f)`` with a
    true IEEE division, then ``clamp(__float2int_rn(x / scale), -127, 127)`` —
    round half to even, one more IEEE division per element. The divisions are
    done tensor/tensor so that torch cannot turn them into reciprocal multiplies.
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    value = x.float()
    # fmaxf() returns the other operand when one is NaN, so a NaN never enters the row maximum.
    absmax = torch.nan_to_num(value.abs(), nan=0.0, posinf=float("inf")).amax(dim=1)
    scale = torch.maximum(absmax / torch.full_like(absmax, 127.0),
                          torch.full_like(absmax, 1e-20))
    quotient = value / scale[:, None].expand_as(value)
    # fmaxf() drops NaNs and __float2int_rn(NaN) is 0: mirror both.
    quotient = torch.nan_to_num(quotient, nan=0.0, posinf=127.0, neginf=-127.0)
    codes = quotient.round().clamp(-127, 127).to(torch.int8)
    return codes, scale


def quantize_grouped4096_ref(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M,G,4096] -> (INT8 [G,M,4096] group-major, FP32 [G,M]).

    The reference defines the grouped quantizer by equality with the row
    quantizer on each group slice (tests/test_cuda_ops.py:31-38).
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 3 and x.size(2) == 4096
    m, groups, width = x.shape
    flat = x.transpose(0, 1).contiguous().view(groups * m, width)
    if m == 0:
        return (torch.empty(groups, 0, width, dtype=torch.int8),
                torch.empty(groups, 0, dtype=torch.float32))
    codes, scales = quantize_rows_ref(flat)
    return codes.view(groups, m, width), scales.view(groups, m)


# --------------------------------------------------------------------------- #
# Integer product
# --------------------------------------------------------------------------- #
def int_mm_literal(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The reference's literal oracle: ``a.int() @ w.int().T`` (tests/test_cuda_ops.py:596).

    ``w`` may be INT8 (signed codes) or UINT8 (code + 128, tests/test_cuda_ops.py:488).
    """
    wide = w.int() - 128 if w.dtype == torch.uint8 else w.int()
    return a.int() @ wide.T


def int_mm_fast(a: torch.Tensor, w: torch.Tensor, row_chunk: int = 2048) -> torch.Tensor:
    """Exact INT32 product through FP32 GEMMs over K-chunks, for full-size configs.

    Each K-chunk of at most 1024 terms has |sum| <= 1024*128*128 = 2^24, which FP32
    holds exactly whatever the summation order, so every partial product is exact;
    the partials are then added in INT32 (the reference bounds K by 65536 so the
    total fits). Cross-checked against int_mm_literal in the test suite.
    """
    if w.dtype == torch.uint8:
        w = (w.to(torch.int16) - 128).to(torch.int8)
    m, k = a.shape
    n = w.shape[0]
    out = torch.empty(m, n, dtype=torch.int32)
    wf = w.float()
    for r0 in range(0, m, row_chunk):
        af = a[r0:r0 + row_chunk].float()
        acc = torch.zeros(af.shape[0], n, dtype=torch.int32)
        for k0 in range(0, k, 1024):
            acc += (af[:, k0:k0 + 1024] @ wf[:, k0:k0 + 1024].T).to(torch.int32)
        out[r0:r0 + row_chunk] = acc
    return out


# --------------------------------------------------------------------------- #
# Epilogue and the composed operators
# --------------------------------------------------------------------------- #
def epilogue_ref(acc: torch.Tensor, a_scale: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """``bf16((float(acc) * sa[row]) * float(sw[col]))`` — row scale first, channel scale
    second, two FP32 roundings, then one rounding to BF16 (tests/test_cuda_ops.py:489,599)."""
    return (acc.float() * a_scale.float()[:, None] * w_scale.float()[None, :]).bfloat16()


def fused_channel_mm_ref(a, w, a_scale, w_scale, fast: bool = False):
    """fused_channel_mm / cutlass_channel_mm: returns (INT32 accumulators, BF16 out)."""
    assert w.dtype == torch.int8
    acc = int_mm_fast(a, w) if fast else int_mm_literal(a, w)
    return acc, epilogue_ref(acc, a_scale, w_scale)


def channel_mm_ref(a, w_u8, a_scale, w_scale, fast: bool = False):
    """channel_mm: UINT8 weights hold signed code + 128 (csrc/kernels.cu:107)."""
    assert w_u8.dtype == torch.uint8
    acc = int_mm_fast(a, w_u8) if fast else int_mm_literal(a, w_u8)
    return acc, epilogue_ref(acc, a_scale, w_scale)


def channel_gemv_fp64(x: torch.Tensor, w: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """The reference's W8A16 oracle (tests/test_gemv.py:26-29): FP64 linear over the
    BF16-rounded dequantized weights, result rounded to BF16."""
    dequantized = (w.float() * w_scale.float()[:, None]).bfloat16()
    return torch.nn.functional.linear(x.double(), dequantized.double()).bfloat16()


channel_gemv_ref = channel_gemv_fp64


def grouped_channel_mm_ref(codes, scales, w, w_scale, fast: bool = False) -> torch.Tensor:
    """Grouped-scale W8A8: codes [G,M,4096], scales [G,M] (from the grouped quantizer),
    w INT8 [N, G*4096], w_scale BF16 [N] -> BF16 [M,N].

    Per group an exact INT32 product; the groups are rescaled and summed in FP32 in
    ascending group order with separate multiply and add roundings (no FMA), then the
    channel scale is applied and the result is rounded to BF16. With one group this is
    exactly fused_channel_mm_ref. The reference has no single function for this; its
    precedent for FP32-summed rescaled INT32 partials is
    benchmarks/cuda/q8_block_int8.cu:44-62.
    """
    groups, m, width = codes.shape
    n = w.shape[0]
    total = torch.zeros(m, n, dtype=torch.float32)
    for g in range(groups):
        wg = w[:, g * width:(g + 1) * width]
        acc = int_mm_fast(codes[g], wg) if fast else int_mm_literal(codes[g], wg)
        term = acc.float() * scales[g].float()[:, None]
        total = term if g == 0 else total + term
    return (total * w_scale.float()[None, :]).bfloat16()


# --------------------------------------------------------------------------- #
# SwiGLU in front of the down projection (floating point: tolerance, not bit-exact)
# --------------------------------------------------------------------------- #
def silu_mul_ref(x: torch.Tensor) -> torch.Tensor:
    """BF16 [M, 2K] = gate | up  ->  BF16 [M, K] = bf16(silu(gate) * up), evaluated in FP64.

    The reference computes ``gate / (1 + expf(-gate))`` with the GPU's fast division and rounds
    the FP32 product to BF16 (csrc/silu_quant.cu:30-33); its own test compares with a compiled
    torch SwiGLU on the GPU (tests/test_cuda_ops.py:874-911). Transcendentals cannot be restated
    bit-exactly on a CPU, so this checker is used with a tolerance of one BF16 ulp; the integer
    part of that operator (the quantizer behind it) is checked exactly.
    """
    k = x.shape[1] // 2
    gate, up = x[:, :k].double(), x[:, k:].double()
    return (gate / (1.0 + torch.exp(-gate)) * up).to(torch.bfloat16)


# --------------------------------------------------------------------------- #
# Weight encoding (defines the UINT8 + 128 / BF16-scale tensors the path consumes)
# --------------------------------------------------------------------------- #
def quantize_channel_ref(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[N,K] float -> (UINT8 code+128 [N,K], BF16 scale [N]); src/consumer_int8/quantization.py:22-32."""
    value = weight.float()
    scale = value.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny) / 127.0
    codes = (value / scale[:, None]).round().clamp(-128, 127)
    return (codes.to(torch.int16) + 128).to(torch.uint8), scale.to(torch.bfloat16)


# --------------------------------------------------------------------------- #
# AllSpark N32K16 storage (byte permutation). Parity for this operator is UNPINNED: the
# reference's only pin packs with vLLM's allspark_repack_weight (tests/test_cuda_ops.py:440-471),
# which is not available here; the inverse permutation below restates the reference's kernel
# index arithmetic (csrc/allspark_layout.cu:8-28), and pack_allspark_ref is its algebraic inverse.
# --------------------------------------------------------------------------- #
def _cell_index(n: int, k: int):
    """For every (row, tile, j): byte offset into the packed buffer, following the reference."""
    import numpy as np

    rows = np.arange(n)[:, None, None]
    tiles = np.arange(k // 16)[None, :, None]
    j = np.arange(16)[None, None, :]
    packed_row = (rows // 32) * 8 + rows % 8
    base = packed_row * k * 4 + tiles * 64 + ((rows % 32) // 16) * 8 + ((rows % 16) // 8) * 4
    # restored word x = (a & 0xffff) | (b << 16): bytes a0 a1 b0 b1; y: c0 c1 d0 d1; z: a2 a3 b2 b3; w: c2 c3 d2 d3
    quarter = np.array([0, 0, 1, 1, 2, 2, 3, 3, 0, 0, 1, 1, 2, 2, 3, 3])[j]
    byte = np.array([0, 1, 0, 1, 0, 1, 0, 1, 2, 3, 2, 3, 2, 3, 2, 3])[j]
    return base + quarter * 16 + byte


def unpack_allspark_ref(packed: torch.Tensor, packed_scales: torch.Tensor, n: int, k: int):
    """packed UINT8 [ceil(n/32)*32, k] -> (INT8 [n,k] = code - 128, BF16 [n] scales)."""
    import numpy as np

    flat = packed.contiguous().view(-1).numpy()
    index = _cell_index(n, k)
    codes = (flat[index].reshape(n, k).astype(np.int16) - 128).astype(np.int8)
    rows = np.arange(n)
    scale_index = (rows // 32) * 32 + (rows % 8) * 4 + (rows % 32) // 8
    return torch.from_numpy(codes), packed_scales[torch.from_numpy(scale_index)]


def pack_allspark_ref(codes_u8: torch.Tensor, scales: torch.Tensor):
    """UINT8 code+128 [n,k] and BF16 [n] scales -> the packed pair (inverse of unpack_allspark_ref)."""
    import numpy as np

    n, k = codes_u8.shape
    padded = (n + 31) // 32 * 32
    flat = np.zeros(padded * k, dtype=np.uint8)
    flat[_cell_index(n, k).reshape(-1)] = codes_u8.contiguous().numpy().reshape(-1)
    rows = np.arange(n)
    scale_index = (rows // 32) * 32 + (rows % 8) * 4 + (rows % 32) // 8
    packed_scales = torch.zeros(padded, dtype=scales.dtype)
    packed_scales[torch.from_numpy(scale_index)] = scales
    return torch.from_numpy(flat).view(padded, k), packed_scales


def q8_block_quantize_ref(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [M,K] -> (INT8 codes [M,K], FP32 scales [M,K/32]): the row quantizer applied to every
    32 consecutive values (benchmarks/cuda/q8_block_int8.cu:11-24; its oracle in
    benchmarks/benchmark_q8_block_int8.py:90-93 is the same absmax/127 formula)."""
    m, k = x.shape
    codes, scales = quantize_rows_ref(x.reshape(m * (k // 32), 32))
    return codes.reshape(m, k), scales.reshape(m, k // 32)


def q8_block_mm_ref(a: torch.Tensor, w: torch.Tensor, sa: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    """Block-32 W8A8 product: a INT8 [M,K], w INT8 [N,K], sa FP32 [M,K/32], sw FP16 [N,K/32] -> BF16
    [M,N] with sum = fma(float(dot_b), sa_b * sw_b, sum) over ascending blocks
    (benchmarks/cuda/q8_block_int8.cu:44-62 with the multiply-add contracted). The FMA is emulated
    in FP64: the product of an integer below 2^20 and an FP32 scale is exact there, so only the
    final rounding of the sum to FP32 is done twice (FP64, then FP32)."""
    m, k = a.shape
    n = w.shape[0]
    blocks = k // 32
    total = torch.zeros(m, n, dtype=torch.float32)
    a64 = a.reshape(m, blocks, 32).double()
    w64 = w.reshape(n, blocks, 32).double()
    for b in range(blocks):
        dot = a64[:, b] @ w64[:, b].T                                   # exact: |dot| < 2^20
        scale = sa[:, b, None].float() * sw[None, :, b].float()        # one FP32 rounding, as on the GPU
        total = (dot * scale.double() + total.double()).float()
    return total.bfloat16()


def q8_block_mm_loose_ref(a, w, sa, sw) -> torch.Tensor:
    """The formula of the reference's own acceptance test, literally
    (benchmarks/benchmark_q8_block_int8.py:104-109): FP32 multiply and add, no FMA; the test
    there allows rtol 0.008 against it."""
    m, k = a.shape
    n = w.shape[0]
    blocks = k // 32
    total = torch.zeros(m, n)
    for b in range(blocks):
        dot = a.reshape(m, blocks, 32)[:, b].float() @ w.reshape(n, blocks, 32)[:, b].float().T
        total += dot * (sa[:, b, None] * sw[None, :, b].float())
    return total.bfloat16()

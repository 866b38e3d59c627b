"""gate_up_silu_mm: the gate/up projection with the SwiGLU in the GEMM epilogue must produce the bits
of the two operators it replaces, fused_channel_mm followed by silu_mul (reference
csrc/fused_mm.cu:66-93, csrc/silu_quant.cu:64-88), on weights whose gate and up rows were interleaved
in blocks of 128; the intermediate itself is checked against the CPU checker."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status, linear_case
from test_gpu_swiglu import bf16_ulp_distance
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,inner,k", [(1, 128, 64), (100, 256, 512), (129, 384, 544), (300, 1280, 1024),
                                        (1024, 2176, 640)])
def test_fused_swiglu_gemm_equals_the_operator_pair(ops, m, inner, k):
    from consumer_int8.quantization import interleave_gate_up

    a, w, sa, sw = linear_case(m, 2 * inner, k, seed=m + inner)
    sw = (sw.float() * 4).bfloat16()             # gate values of a few units, so the sigmoid is exercised
    ad, wd, sad, swd = a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV)
    gate_up = torch.empty(m, 2 * inner, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(ad, wd, sad, swd, gate_up, 0)
    _, want_gate_up = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    assert_bit_equal(gate_up, want_gate_up, "gate/up intermediate")
    want = torch.empty(m, inner, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(gate_up, want)
    wi, swi = interleave_gate_up(wd, swd)
    got = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gate_up_silu_mm(ad, wi, sad, swi, got)
    assert_bit_equal(got, want, "fused SwiGLU GEMM vs fused_channel_mm + silu_mul")
    # and inside the SwiGLU checker's tolerance (1 BF16 ulp of an FP64 evaluation)
    # (where the gate is moderate: far below zero expf overflows and the product underflows, as in the reference)
    moderate = want_gate_up[:, :inner].float().abs() <= 20
    distance = bf16_ulp_distance(got, ref.silu_mul_ref(want_gate_up))
    assert moderate.any() and int(distance[moderate].max()) <= 1
    assert device_status(ops) == 0


def test_fused_swiglu_gemm_rejects_bad_geometry(ops):
    a = torch.zeros(4, 64, dtype=torch.int8, device=DEV)
    sa = torch.ones(4, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.int8, device=DEV)      # n % 256 != 0
    with pytest.raises(RuntimeError, match="geometry"):
        ops.gate_up_silu_mm(a, w, sa, torch.ones(128, dtype=torch.bfloat16, device=DEV),
                            torch.empty(4, 64, dtype=torch.bfloat16, device=DEV))

"""silu_mul / silu_mul_quantize (the SwiGLU between the gate/up and down projections).

Floating point part: within one BF16 ulp of the FP64 checker. Integer part: silu_mul_quantize must
equal quantize_rows applied to silu_mul's output bit for bit, eagerly and on graph replay — the
form of the reference's own assertion (tests/test_cuda_ops.py:874-911) — and those codes must
equal the CPU quantizer run on the same BF16 values."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in BF16 steps (sign-magnitude patterns mapped onto a monotone integer line)."""
    def ordered(t):
        bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(bits >= 0x8000, 0x8000 - bits, bits)
    return (ordered(a.cpu()) - ordered(b.cpu())).abs()


@pytest.mark.parametrize("rows", [0, 1, 4, 1024, 3904])
@pytest.mark.parametrize("width", [8704, 17408, 64, 2056])
def test_swiglu_and_its_quantization(ops, rows, width):
    torch.manual_seed(775 + rows + width)
    x = torch.randn(rows, 2 * width, device=DEV, dtype=torch.bfloat16) * 3
    if rows:
        x[0].zero_()
    activated = torch.empty(rows, width, device=DEV, dtype=x.dtype)
    codes = torch.empty(rows, width, device=DEV, dtype=torch.int8)
    scales = torch.empty(rows, device=DEV)
    ops.silu_mul(x, activated)
    ops.silu_mul_quantize(x, codes, scales)
    if not rows:
        return

    def check():
        want = ref.silu_mul_ref(x.cpu())
        assert int(bf16_ulp_distance(activated, want).max()) <= 1       # tolerance: one BF16 ulp
        reference_codes = torch.empty_like(codes)
        reference_scales = torch.empty_like(scales)
        ops.quantize_rows(activated, reference_codes, reference_scales)
        assert torch.equal(codes, reference_codes) and torch.equal(scales, reference_scales)
        cpu_codes, cpu_scales = ref.quantize_rows_ref(activated.cpu())
        assert_bit_equal(codes, cpu_codes, "codes vs CPU quantizer")
        assert_bit_equal(scales, cpu_scales, "scales vs CPU quantizer")

    check()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.silu_mul(x, activated)
        ops.silu_mul_quantize(x, codes, scales)
    x.mul_(0.75)
    codes.fill_(-128)
    scales.fill_(float("nan"))
    graph.replay()
    check()


def test_swiglu_extreme_gates(ops):
    """Large negative gates underflow to (signed) zero, large positive gates pass `up` through."""
    width = 64
    x = torch.zeros(2, 2 * width, dtype=torch.bfloat16)
    x[0, :8] = torch.tensor([-100.0, -30.0, -10.0, 0.0, 10.0, 30.0, 100.0, 1e4])
    x[0, width:width + 8] = torch.tensor([2.0, -3.0, 4.0, 5.0, -6.0, 7.0, 0.5, 1.5])
    x[1, :width] = 3.0e38
    x[1, width:] = 1.0
    out = torch.empty(2, width, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(x.to(DEV), out)
    want = ref.silu_mul_ref(x)
    assert torch.isfinite(out[0].float()).all()
    assert int(bf16_ulp_distance(out[0], want[0]).max()) <= 1
    assert torch.equal(out[1].cpu(), want[1])         # silu(huge) * 1 = huge, exactly representable


def test_swiglu_quantization_rejects_unaligned_input_before_vector_load(ops):
    width = 8704
    x = torch.empty(2 * width + 1, device=DEV, dtype=torch.bfloat16)[1:]
    codes = torch.empty(1, width, device=DEV, dtype=torch.int8)
    scales = torch.empty(1, device=DEV)
    with pytest.raises(RuntimeError, match="aligned buffers"):
        ops.silu_mul_quantize(x.view(1, -1), codes, scales)
    with pytest.raises(RuntimeError, match="SwiGLU quantization shape"):
        ops.silu_mul_quantize(torch.empty(1, 2 * width, device=DEV, dtype=torch.bfloat16),
                              torch.empty(1, width - 8, device=DEV, dtype=torch.int8), scales)
    with pytest.raises(RuntimeError, match="SwiGLU shape"):
        ops.silu_mul(torch.empty(2, 100, device=DEV, dtype=torch.bfloat16),
                     torch.empty(2, 52, device=DEV, dtype=torch.bfloat16))

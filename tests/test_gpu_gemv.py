"""channel_gemv (W8A16) against the reference's FP64 oracle, with the reference's tolerances
(tests/test_gemv.py:10-33): atol 0.004, rtol 0.008, relative L2 error below 0.003."""
import pytest
import torch

from gpu_common import DEV
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 13, 16])
@pytest.mark.parametrize("n,k", [(37, 528), (512, 5120), (1000, 17408), (4096, 5120), (2500, 528), (34816, 1040)])
def test_w8a16_small_batch_matches_bf16_dequantized_linear(ops, m, n, k):
    torch.manual_seed(134)
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    weight = torch.randint(-127, 128, (n, k), device=DEV, dtype=torch.int8)
    scale = (torch.rand(n, device=DEV) * 0.002).bfloat16()
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops.channel_gemv(x, weight, scale, out)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.channel_gemv(x, weight, scale, out)
    x.mul_(0.75)
    graph.replay()
    reference = ref.channel_gemv_fp64(x.cpu(), weight.cpu(), scale.cpu())
    actual = out.cpu()
    torch.testing.assert_close(actual, reference, atol=0.004, rtol=0.008)
    error = (actual.float() - reference.float()).norm() / reference.float().norm()
    assert error.item() < 0.003


def test_gemv_rejects_unsupported_geometry(ops):
    x = torch.zeros(17, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 64, dtype=torch.int8, device=DEV)
    scale = torch.ones(8, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="GEMV geometry"):
        ops.channel_gemv(x, w, scale, torch.empty(17, 8, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError, match="GEMV geometry"):      # k % 16
        ops.channel_gemv(x[:1, :40].contiguous(), w[:, :40].contiguous(), scale,
                         torch.empty(1, 8, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("m,n,k", [(3, 100, 528), (8, 64, 2064)])
def test_w8a16_with_activations_that_are_only_4_byte_aligned(ops, m, n, k):
    """The reference only asks for 4-byte aligned activations (csrc/bindings.cpp:303-304); such
    inputs take the FMA kernel instead of the tensor-core one."""
    torch.manual_seed(7)
    storage = torch.randn(m * k + 2, device=DEV, dtype=torch.bfloat16)
    x = storage[2:].view(m, k)                      # 4 bytes past a 16-byte boundary
    assert x.data_ptr() % 16 == 4
    weight = torch.randint(-127, 128, (n, k), device=DEV, dtype=torch.int8)
    scale = (torch.rand(n, device=DEV) * 0.002).bfloat16()
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops.channel_gemv(x, weight, scale, out)
    reference = ref.channel_gemv_fp64(x.cpu(), weight.cpu(), scale.cpu())
    torch.testing.assert_close(out.cpu(), reference, atol=0.004, rtol=0.008)
    aligned = torch.empty_like(out)
    ops.channel_gemv(x.clone(), weight, scale, aligned)
    torch.testing.assert_close(aligned.cpu(), reference, atol=0.004, rtol=0.008)


@pytest.mark.parametrize("n", [64, 2304])     # the register-fed kernel (small N) and the TMA-staged one
def test_dequantised_weights_are_the_reference_rounding_bit_for_bit(ops, n):
    """The operator multiplies activations with bf16(float(code) * float(scale)) (the reference's
    csrc/gemv.cu:23-26). With one-hot activation rows the output IS that multiplicand, so every code from
    -128 to 127 against a spread of scales (tiny, ordinary, large, negative) can be compared exactly with
    ``(w.float() * scale.float()).bfloat16()``."""
    k = 256
    codes = torch.arange(-128, 128, dtype=torch.int16).to(torch.int8)
    weight = codes.repeat(n, 1).contiguous()                        # channel c, position j holds code j - 128
    generator = torch.Generator().manual_seed(5)
    scale = (torch.rand(n, generator=generator) * 0.02 + 1e-4)
    scale[::7] *= 1e-30
    scale[1::7] *= 1e20
    scale[2::7] *= -1.0
    scale = scale.bfloat16()
    want = (weight.float() * scale.float()[:, None]).bfloat16()     # [n, k]
    dw, ds = weight.to(DEV), scale.to(DEV)
    out = torch.empty(16, n, dtype=torch.bfloat16, device=DEV)
    for first in range(0, k, 16):
        x = torch.zeros(16, k, dtype=torch.bfloat16)
        x[torch.arange(16), first + torch.arange(16)] = 1.0          # row i picks position first + i
        ops.channel_gemv(x.to(DEV), dw, ds, out)
        got = out.cpu()                                              # got[i, c] = multiplicand of (c, first + i)
        expected = want[:, first:first + 16].T.contiguous()
        # (code 0 times a negative scale is -0, which the sum with the other, +0, products turns into +0)
        expected = torch.where(expected == 0, torch.zeros_like(expected), expected)
        assert torch.equal(got.view(torch.int16), expected.view(torch.int16)), f"positions {first}..{first + 15}"

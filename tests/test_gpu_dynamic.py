"""dynamic_channel_mm = quantize_rows + fused_channel_mm in one call. For decode shapes it is one
kernel that quantizes the activations on their way into the MMA operand tile; codes, scales and
outputs must be the bits of the two operators it replaces (reference csrc/kernels.cu:13-35,283-292
and csrc/fused_mm.cu:66-93), checked against the CPU checker, eagerly and under graph replay."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(m, k, generator=g) * 3).bfloat16()
    x[:, ::97] *= 50                                     # outlier channels, as in the decode workload
    if m > 2:
        x[1].zero_()                                     # an all-zero row: scale floor 1e-20
    x[0, :4] = torch.tensor([0.0, -127.0, 63.5, 127.0]).bfloat16()   # exact ties
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
    sw = (torch.rand(n, generator=g) / 127).bfloat16()
    return x, w, sw


# unsplit decode shapes (one kernel), split or large-K shapes and M > 16 (two kernels)
@pytest.mark.parametrize("m,n,k", [(1, 34816, 512), (4, 20000, 1024), (16, 37888, 640), (8, 34816, 5120),
                                   (3, 148 * 16, 96), (16, 512, 4096), (5, 1000, 17408), (40, 5120, 1024),
                                   (300, 512, 256)])
def test_dynamic_linear_equals_quantizer_then_gemm(ops, m, n, k):
    x, w, sw = _case(m, n, k, m + n + k)
    xd, wd, swd = x.to(DEV), w.to(DEV), sw.to(DEV)
    codes = torch.full((m, k), 99, dtype=torch.int8, device=DEV)
    scales = torch.full((m,), float("nan"), device=DEV)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.dynamic_channel_mm(xd, wd, swd, codes, scales, out)
    want_codes, want_scales = ref.quantize_rows_ref(x)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    _, want = ref.fused_channel_mm_ref(want_codes, w, want_scales, sw, fast=True)
    assert_bit_equal(out, want, "out")
    assert device_status(ops) == 0


def test_dynamic_linear_graph_replay_on_new_activations(ops):
    m, n, k = 8, 34816, 1024
    x, w, sw = _case(m, n, k, 11)
    xd, wd, swd = x.to(DEV), w.to(DEV), sw.to(DEV)
    codes = torch.empty(m, k, dtype=torch.int8, device=DEV)
    scales = torch.empty(m, device=DEV)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.dynamic_channel_mm(xd, wd, swd, codes, scales, out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(3):
            ops.dynamic_channel_mm(xd, wd, swd, codes, scales, out)
    x2 = (x.float() * -0.37).bfloat16()
    xd.copy_(x2)
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    want_codes, want_scales = ref.quantize_rows_ref(x2)
    assert_bit_equal(codes, want_codes, "codes after replay")
    _, want = ref.fused_channel_mm_ref(want_codes, w, want_scales, sw, fast=True)
    assert_bit_equal(out, want, "out after replay")

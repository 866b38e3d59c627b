"""Block-32 (Q8_0) W8A8 on the GPU through the C ABI, as the reference's benchmark binds its own
entry point (benchmarks/benchmark_q8_block_int8.py:36-39,68-80): codes, scales and BF16 outputs bit
for bit against the CPU checker, the reference's own tolerance checks (:90-113), graph replay on
negated inputs as there (:86-89), and tile / K tails of the tcgen05 kernel."""
import ctypes

import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=g)
    sw = (torch.randn(n, k // 32, generator=g) * 0.01).half()
    x = (torch.randn(m, k, generator=g) * 0.1).bfloat16()
    x[:, :32] = 0
    if k >= 64:
        x[:, 32:64] *= 100
    return x, w, sw


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(ops, x, a, sa, w, sw, y, m, n, k):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return ops.libci8.ci8_q8_block_mm(_ptr(x), _ptr(a), _ptr(sa), _ptr(w), _ptr(sw), _ptr(y), m, n, k, stream)


CASES = [(1, 1, 32), (17, 33, 96), (129, 65, 256), (16, 200, 4096), (300, 130, 1056), (1024, 1024, 1024),
         (384, 800, 128), (384, 812, 64)]


def test_cases_cover_every_tile_width(ops):
    """The kernel comes in tiles of 64, 32 and 16 channels, chosen from the shape and the SM count."""
    widths = {ops.libci8.ci8_q8_block_tile_channels(m, n) for m, n, _ in CASES}
    assert widths == {16, 32, 64}, widths
    assert ops.libci8.ci8_q8_block_tile_channels(0, 4) == 0


@pytest.mark.parametrize("m,n,k", CASES)
def test_block32_matches_checker_bit_for_bit(ops, m, n, k):
    x, w, sw = _case(m, n, k, 7 * m + n)
    dx, dw, dsw = x.to(DEV), w.to(DEV), sw.to(DEV)
    a = torch.full((m, k), 99, dtype=torch.int8, device=DEV)
    sa = torch.full((m, k // 32), float("nan"), device=DEV)
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert _call(ops, dx, a, sa, dw, dsw, y, m, n, k) == 0
    torch.cuda.synchronize()
    want_codes, want_sa = ref.q8_block_quantize_ref(x)
    assert_bit_equal(a, want_codes, "codes")
    assert_bit_equal(sa, want_sa, "scales")
    want = ref.q8_block_mm_ref(want_codes, w, want_sa, sw)
    assert_bit_equal(y, want, "y")
    # the reference's acceptance checks (benchmark_q8_block_int8.py:104-113)
    torch.testing.assert_close(y.cpu(), ref.q8_block_mm_loose_ref(want_codes, w, want_sa, sw), rtol=0.008, atol=1e-5)
    dense = x.float() @ (w.float().reshape(n, k // 32, 32) * sw.float()[..., None]).reshape(n, k).T
    relative = ((y.cpu().float() - dense).norm() / dense.norm().clamp_min(1e-20)).item()
    assert torch.isfinite(y).all() and relative < 0.015
    assert device_status(ops) == 0


def test_block32_graph_replay_on_negated_inputs(ops):
    m, n, k = 129, 65, 256
    x, w, sw = _case(m, n, k, 3)
    dx, dw, dsw = x.to(DEV), w.to(DEV), sw.to(DEV)
    a = torch.empty(m, k, dtype=torch.int8, device=DEV)
    sa = torch.empty(m, k // 32, device=DEV)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    for _ in range(3):
        assert _call(ops, dx, a, sa, dw, dsw, y, m, n, k) == 0
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        assert _call(ops, dx, a, sa, dw, dsw, y, m, n, k) == 0
    for _ in range(2):
        dx.neg_()
        y.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        codes, scales = ref.q8_block_quantize_ref(dx.cpu())
        assert_bit_equal(a, codes, "codes after replay")
        assert_bit_equal(y, ref.q8_block_mm_ref(codes, w, scales, sw), "y after replay")


def test_block32_rejects_bad_arguments(ops):
    t = torch.zeros(64, dtype=torch.int8, device=DEV)
    null = ctypes.c_void_p(0)
    stream = ctypes.c_void_p(0)
    lib = ops.libci8
    assert lib.ci8_q8_block_mm(_ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 1, 1, 48, stream) == 1   # k % 32
    assert lib.ci8_q8_block_mm(null, _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 1, 1, 32, stream) == 1
    assert lib.ci8_q8_block_mm(_ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), _ptr(t), 0, 1, 32, stream) == 1

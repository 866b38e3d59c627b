"""Chains of dependent kernels on one stream: every kernel reads what the previous one wrote.

The kernels are launched with programmatic stream serialization, so a kernel may become resident
while its predecessor still runs; its griddepcontrol.wait must stand before the first access to
global memory. A misplaced wait would let a kernel read stale codes, scales or activations; these
tests run the MLP-shaped chain quantize_rows -> fused_channel_mm -> silu_mul_quantize ->
fused_channel_mm many times, eagerly and as a CUDA graph, over changing inputs, and compare every
intermediate with the CPU checker bit for bit."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


def _chain_reference(x, w1, sw1, w2, sw2):
    codes, scales = ref.quantize_rows_ref(x)
    _, hidden = ref.fused_channel_mm_ref(codes, w1, scales, sw1, True)
    return codes, scales, hidden


def _make(m, k, inner, seed):
    g = torch.Generator().manual_seed(seed)
    w1 = torch.randint(-127, 128, (2 * inner, k), dtype=torch.int8, generator=g)
    w2 = torch.randint(-127, 128, (k, inner), dtype=torch.int8, generator=g)
    sw1 = (torch.rand(2 * inner, generator=g) / 127).bfloat16()
    sw2 = (torch.rand(k, generator=g) / 127).bfloat16()
    xs = [(torch.randn(m, k, generator=g) * (1 + i)).bfloat16() for i in range(3)]
    return w1, sw1, w2, sw2, xs


@pytest.mark.parametrize("m", [1, 16, 160])
def test_dependent_chain_eager_and_graph(ops, m):
    k, inner = 512, 384
    w1, sw1, w2, sw2, xs = _make(m, k, inner, 5 + m)
    dw1, dsw1, dw2, dsw2 = w1.to(DEV), sw1.to(DEV), w2.to(DEV), sw2.to(DEV)
    x = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    codes = torch.empty(m, k, dtype=torch.int8, device=DEV)
    scales = torch.empty(m, device=DEV)
    hidden = torch.empty(m, 2 * inner, dtype=torch.bfloat16, device=DEV)
    codes2 = torch.empty(m, inner, dtype=torch.int8, device=DEV)
    scales2 = torch.empty(m, device=DEV)
    out = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)

    def chain():
        ops.quantize_rows(x, codes, scales)
        ops.fused_channel_mm(codes, dw1, scales, dsw1, hidden, 0)
        ops.silu_mul_quantize(hidden, codes2, scales2)
        ops.fused_channel_mm(codes2, dw2, scales2, dsw2, out, 0)

    def check(source, what):
        want_codes, want_scales, want_hidden = _chain_reference(source, w1, sw1, w2, sw2)
        assert_bit_equal(codes, want_codes, f"{what}: codes")
        assert_bit_equal(scales, want_scales, f"{what}: scales")
        assert_bit_equal(hidden, want_hidden, f"{what}: hidden")
        # the second half of the chain against the GPU's own intermediates (the SwiGLU is
        # floating point, so its codes are checked through the operators' own identity)
        _, want_out = ref.fused_channel_mm_ref(codes2.cpu(), w2, scales2.cpu(), sw2, True)
        assert_bit_equal(out, want_out, f"{what}: out")
        again_codes = torch.empty_like(codes2)
        again_scales = torch.empty_like(scales2)
        ops.silu_mul_quantize(hidden, again_codes, again_scales)
        torch.cuda.synchronize()
        assert_bit_equal(codes2, again_codes, f"{what}: codes2")
        assert_bit_equal(scales2, again_scales, f"{what}: scales2")

    # eager: back-to-back launches, several rounds so that kernels of neighbouring rounds overlap
    for source in xs:
        x.copy_(source.to(DEV))
        for _ in range(5):
            chain()
        torch.cuda.synchronize()
        check(source, "eager")

    # captured: the same chain five times inside one graph, replayed on new inputs
    x.copy_(xs[0].to(DEV))
    chain()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(5):
            chain()
    for source in reversed(xs):
        x.copy_(source.to(DEV))
        graph.replay()
        torch.cuda.synchronize()
        check(source, "graph")
    assert device_status(ops) == 0

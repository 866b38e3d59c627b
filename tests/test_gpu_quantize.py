"""quantize_rows / quantize_grouped4096 on the GPU against the CPU checker, bit for bit.
Shapes, seeds and assertions follow the reference's tests/test_cuda_ops.py:10-52,493-509."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal, guarded
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("width", [4, 3072, 5120, 6144, 8704, 17408])
@pytest.mark.parametrize("rows,misaligned", [(2, False), (1024, False), (1024, True)])
def test_quantize_rows_preserves_zero_rows_and_round_to_even(ops, width, rows, misaligned):
    torch.manual_seed(742)
    storage = torch.randn(rows * width + 1, device=DEV, dtype=torch.bfloat16)
    x = storage[int(misaligned): rows * width + int(misaligned)].view(rows, width)
    x.mul_(100).clamp_(-127, 127)
    x[:, 0] = -127
    x[0, :4] = torch.tensor([0, -127, 63.5, 127], device=DEV)
    x[1].zero_()
    q = torch.empty_like(x, dtype=torch.int8)
    scales = torch.empty(rows, device=DEV)
    ops.quantize_rows(x, q, scales)
    expected_scale = torch.ones_like(scales)
    expected_scale[1] = 1e-20
    torch.testing.assert_close(scales, expected_scale, rtol=0, atol=0)
    torch.testing.assert_close(q, x.float().round().to(torch.int8), rtol=0, atol=0)


@pytest.mark.parametrize("m,k", [(1, 5120), (4, 5120), (8, 4096), (16, 5120), (100, 8), (65, 2048), (64, 8192),
                                 (333, 5128), (7, 65536), (3, 70000), (2048, 4096), (1000, 12288), (128, 17408)])
def test_quantize_rows_matches_checker_on_real_valued_inputs(ops, m, k):
    g = torch.Generator().manual_seed(m + 31 * k)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[: max(1, k // 1000)]] *= 50.0
    x = x.bfloat16()
    if m > 2:
        x[2].zero_()
    q, check_q = guarded((m, k), torch.int8, -128)
    s, check_s = guarded((m,), torch.float32, float("nan"))
    ops.quantize_rows(x.to(DEV), q, s)
    want_q, want_s = ref.quantize_rows_ref(x)
    assert_bit_equal(s, want_s, "scales")
    assert_bit_equal(q, want_q, "codes")
    check_q()
    check_s()


def test_quantize_rows_special_values(ops):
    x = torch.zeros(6, 64, dtype=torch.bfloat16)
    x[0, :4] = torch.tensor([float("inf"), 1.0, -2.0, float("-inf")])
    x[1, :3] = torch.tensor([float("nan"), 3.0, -1.5])
    x[2, :2] = torch.tensor([1e-38, -1e-38])          # below the 1e-20 scale floor times 127
    x[3, :3] = torch.tensor([3.0e38, -1.0e38, 5.0])    # near the top of the BF16 range
    x[4, :4] = torch.tensor([0.5, 1.5, 2.5, 127.0])
    q = torch.empty(6, 64, dtype=torch.int8, device=DEV)
    s = torch.empty(6, device=DEV)
    ops.quantize_rows(x.to(DEV), q, s)
    want_q, want_s = ref.quantize_rows_ref(x)
    assert_bit_equal(s, want_s, "scales")
    assert_bit_equal(q, want_q, "codes")


@pytest.mark.parametrize("rows,groups", [(0, 4), (1, 1), (3, 2), (128, 4), (2048, 4)])
def test_grouped4096_preserves_native_codes_and_graph_replay(ops, rows, groups):
    torch.manual_seed(137)
    x = torch.randn(rows, groups, 4096, device=DEV, dtype=torch.bfloat16)
    if rows:
        x[0].zero_()
    q = torch.empty(groups, rows, 4096, device=DEV, dtype=torch.int8)
    scales = torch.empty(groups, rows, device=DEV, dtype=torch.float32)
    ops.quantize_grouped_rows(x, q, scales)
    if not rows:
        return
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.quantize_grouped4096(x, q, scales)
    x.neg_()
    q.fill_(-128)
    scales.fill_(float("nan"))
    allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
    graph.replay()
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations
    want_q, want_s = ref.quantize_grouped4096_ref(x.cpu())
    assert_bit_equal(q, want_q, "grouped codes")
    assert_bit_equal(scales, want_s, "grouped scales")
    for group in range(groups):
        expected_q, expected_s = torch.empty_like(q[group]), torch.empty_like(scales[group])
        ops.quantize_rows(x[:, group].contiguous(), expected_q, expected_s)
        assert torch.equal(q[group], expected_q)
        assert torch.equal(scales[group], expected_s)


def test_grouped4096_rejects_wrong_shape_alignment_and_aliases(ops):
    x = torch.randn(3, 4, 4096, device=DEV, dtype=torch.bfloat16)
    q = torch.empty(4, 3, 4096, device=DEV, dtype=torch.int8)
    scales = torch.empty(4, 3, device=DEV)
    with pytest.raises(RuntimeError, match="Expected BF16"):
        ops.quantize_grouped4096(x, q.transpose(0, 1).contiguous(), scales)
    storage = torch.empty(x.numel() + 1, device=DEV, dtype=x.dtype)
    with pytest.raises(RuntimeError, match="aligned"):
        ops.quantize_grouped4096(storage[1:].view_as(x), q, scales)
    aliased = x.view(torch.int8).flatten()[: q.numel()].view_as(q)
    with pytest.raises(RuntimeError, match="overlap"):
        ops.quantize_grouped4096(x, aliased, scales)


def test_quantize_rows_rejects_bad_arguments(ops):
    x = torch.randn(4, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="Wrong output shapes"):
        ops.quantize_rows(x, torch.empty(4, 32, dtype=torch.int8, device=DEV), torch.empty(4, device=DEV))
    with pytest.raises(RuntimeError, match="nonempty"):
        ops.quantize_rows(x[:0], torch.empty(0, 64, dtype=torch.int8, device=DEV), torch.empty(0, device=DEV))
    with pytest.raises(RuntimeError, match="dtype"):
        ops.quantize_rows(x.float(), torch.empty(4, 64, dtype=torch.int8, device=DEV), torch.empty(4, device=DEV))

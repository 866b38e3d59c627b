"""Grouped-scale W8A8 (benchmark config 3): quantize_grouped4096 followed by the one-launch
grouped GEMM, bit for bit against the CPU checker; and the reference-faithful composition
(one fused_channel_mm per group, benchmarks/benchmark_grouped_w8a8.py:100-107)."""
import pytest
import torch

from consumer_int8 import workloads
from gpu_common import DEV, assert_bit_equal, device_status, guarded
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,groups", [(128, 256, 1), (130, 260, 2), (300, 512, 3), (1, 8, 4), (513, 1000, 8)])
def test_grouped_channel_mm_matches_checker(ops, m, n, groups):
    inputs = workloads.grouped_inputs(m, n, groups, seed=m + groups)
    x = inputs.x.to(DEV)
    codes = torch.empty(groups, m, 4096, dtype=torch.int8, device=DEV)
    scales = torch.empty(groups, m, device=DEV)
    ops.quantize_grouped4096(x, codes, scales)
    want_codes, want_scales = ref.quantize_grouped4096_ref(inputs.x)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.grouped_channel_mm(codes, inputs.w.to(DEV), scales, inputs.w_scale.to(DEV), out)
    want = ref.grouped_channel_mm_ref(want_codes, want_scales, inputs.w, inputs.w_scale, fast=True)
    assert_bit_equal(out, want, "grouped out")
    check()
    assert device_status(ops) == 0


def test_grouped_mixed_tile_widths_match_checker(ops):
    """A shape whose automatic tiling mixes two tile widths (what the benchmark's M=2048, N=7168 does)."""
    import ctypes

    m, n, groups = 512, 14336, 2
    plan = (ctypes.c_int * 4)()
    assert ops.libci8.ci8_gemm_tile_plan(m, n, 4096, groups, plan) == 0
    assert plan[2] > 0, f"this shape no longer exercises the mixed widths: {list(plan)}"
    inputs = workloads.grouped_inputs(m, n, groups, seed=5)
    codes, scales = ref.quantize_grouped4096_ref(inputs.x)
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.grouped_channel_mm(codes.to(DEV), inputs.w.to(DEV), scales.to(DEV), inputs.w_scale.to(DEV), out)
    want = ref.grouped_channel_mm_ref(codes, scales, inputs.w, inputs.w_scale, fast=True)
    assert_bit_equal(out, want, "grouped out, mixed widths")
    check()
    assert device_status(ops) == 0


@pytest.mark.parametrize("m,n,groups", [(300, 512, 3), (520, 700, 4), (300, 250, 5), (257, 256, 16), (2048, 7168, 2)])
def test_grouped_split_along_the_groups_matches_checker(ops, m, n, groups):
    """With a lent workspace the tiles of a thin last wave run as one piece per group on CTA pairs of their
    own and the pieces add their FP32 terms in ascending group order: same bits as the checker and as
    the plain operator, call after call on the same workspace (its counters return to zero)."""
    need = ops.grouped_workspace_bytes(m, n, groups)
    assert need > 0, "this shape no longer exercises the split along the groups"
    inputs = workloads.grouped_inputs(m, n, groups, seed=m + n)
    codes, scales = ref.quantize_grouped4096_ref(inputs.x)
    want = ref.grouped_channel_mm_ref(codes, scales, inputs.w, inputs.w_scale, fast=True)
    dc, dw, ds, dsw = codes.to(DEV), inputs.w.to(DEV), scales.to(DEV), inputs.w_scale.to(DEV)
    workspace = torch.zeros(need, dtype=torch.uint8, device=DEV)
    for call in range(3):
        out, check = guarded((m, n), torch.bfloat16, float("nan"))
        ops.grouped_channel_mm_ws(dc, dw, ds, dsw, workspace, out)
        assert_bit_equal(out, want, f"split along the groups, call {call}")
        check()
    assert int(workspace[:1024].view(torch.int32).abs().sum()) == 0, "the counters did not return to zero"
    plain = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.grouped_channel_mm(dc, dw, ds, dsw, plain)
    assert_bit_equal(plain, want, "plain operator")
    # a workspace that is too small is ignored, not an error
    ops.grouped_channel_mm_ws(dc, dw, ds, dsw, workspace[:16], plain)
    assert_bit_equal(plain, want, "too small a workspace")
    assert device_status(ops) == 0


def test_grouped_split_takes_channel_scales_at_any_alignment(ops):
    """The pieces read their channel scales eight at a time when the pointer allows it and one by one
    when it does not: a scale vector that starts two bytes into an allocation gives the same bits."""
    m, n, groups = 520, 700, 4
    need = ops.grouped_workspace_bytes(m, n, groups)
    assert need > 0
    inputs = workloads.grouped_inputs(m, n, groups, seed=77)
    codes, scales = ref.quantize_grouped4096_ref(inputs.x)
    want = ref.grouped_channel_mm_ref(codes, scales, inputs.w, inputs.w_scale, fast=True)
    holder = torch.empty(n + 1, dtype=torch.bfloat16, device=DEV)
    holder[1:].copy_(inputs.w_scale)
    shifted = holder[1:]
    assert shifted.data_ptr() % 16 != 0
    workspace = torch.zeros(need, dtype=torch.uint8, device=DEV)
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.grouped_channel_mm_ws(codes.to(DEV), inputs.w.to(DEV), scales.to(DEV), shifted, workspace, out)
    assert_bit_equal(out, want, "split along the groups, unaligned channel scales")
    check()
    assert device_status(ops) == 0


def test_grouped_split_replays_from_a_graph(ops):
    m, n, groups = 520, 700, 4
    need = ops.grouped_workspace_bytes(m, n, groups)
    assert need > 0
    inputs = workloads.grouped_inputs(m, n, groups, seed=8)
    x = inputs.x.to(DEV)
    dw, dsw = inputs.w.to(DEV), inputs.w_scale.to(DEV)
    codes = torch.empty(groups, m, 4096, dtype=torch.int8, device=DEV)
    scales = torch.empty(groups, m, device=DEV)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    workspace = torch.zeros(need, dtype=torch.uint8, device=DEV)

    def run():
        ops.quantize_grouped4096(x, codes, scales)
        ops.grouped_channel_mm_ws(codes, dw, scales, dsw, workspace, out)

    run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for replay in range(2):
        x.neg_()
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        rc, rs = ref.quantize_grouped4096_ref(x.cpu())
        assert_bit_equal(out, ref.grouped_channel_mm_ref(rc, rs, inputs.w, inputs.w_scale, fast=True), f"replay {replay}")
    assert device_status(ops) == 0


def test_one_group_equals_fused_channel_mm(ops):
    inputs = workloads.grouped_inputs(200, 512, 1, seed=2)
    codes, scales = ref.quantize_grouped4096_ref(inputs.x)
    grouped = torch.empty(200, 512, dtype=torch.bfloat16, device=DEV)
    fused = torch.empty_like(grouped)
    ops.grouped_channel_mm(codes.to(DEV), inputs.w.to(DEV), scales.to(DEV), inputs.w_scale.to(DEV), grouped)
    ops.fused_channel_mm(codes[0].to(DEV), inputs.w.to(DEV), scales[0].to(DEV), inputs.w_scale.to(DEV), fused)
    assert_bit_equal(grouped, fused, "one group")


def test_per_group_fused_calls_on_group_slices(ops):
    """What the reference does today: G independent GEMMs on codes[g] against that group's
    columns of the weight (here each group's slice is made contiguous, as the reference's
    per-group weight tensors are)."""
    m, n, groups = 96, 256, 4
    inputs = workloads.grouped_inputs(m, n, groups, seed=11)
    codes, scales = ref.quantize_grouped4096_ref(inputs.x)
    for g in range(groups):
        wg = inputs.w[:, g * 4096:(g + 1) * 4096].contiguous()
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.fused_channel_mm(codes[g].to(DEV), wg.to(DEV), scales[g].to(DEV), inputs.w_scale.to(DEV), out, 0)
        _, want = ref.fused_channel_mm_ref(codes[g], wg, scales[g], inputs.w_scale, fast=True)
        assert_bit_equal(out, want, f"group {g}")


def test_grouped_rejects_bad_geometry(ops):
    codes = torch.zeros(2, 4, 4096, dtype=torch.int8, device=DEV)
    w = torch.zeros(8, 4096, dtype=torch.int8, device=DEV)       # K for one group only
    with pytest.raises(RuntimeError, match="geometry"):
        ops.grouped_channel_mm(codes, w, torch.ones(2, 4, device=DEV), torch.ones(8, dtype=torch.bfloat16, device=DEV),
                               torch.empty(4, 8, dtype=torch.bfloat16, device=DEV))

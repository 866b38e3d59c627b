"""The benchmark configurations at their full sizes.

Exact comparison with the CPU checker on a seeded sample of output rows (rows are independent,
so a row sample of A against the full W is an exact check of those rows), plus
size-independent properties over the whole output: schedule invariance (one-CTA and two-CTA
tiles give identical bits), agreement of the fused and workspace operators, sign symmetry
(negating the activations negates every output), and row-permutation equivariance."""
import pytest
import torch

from consumer_int8 import workloads
from gpu_common import DEV, assert_bit_equal, device_status
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


def quantize_on_gpu(ops, x):
    codes = torch.empty(x.shape, dtype=torch.int8, device=DEV)
    scales = torch.empty(x.shape[0], device=DEV)
    ops.quantize_rows(x, codes, scales)
    return codes, scales


@pytest.mark.parametrize("name,m,n,k", [("gate_up", 4096, 34816, 5120), ("down", 4096, 5120, 17408)])
def test_prefill_configs(ops, name, m, n, k):
    inputs = workloads.linear_inputs(m, n, k, seed=0)
    x, w, sw = inputs.x.to(DEV), inputs.w.to(DEV), inputs.w_scale.to(DEV)
    codes, scales = quantize_on_gpu(ops, x)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(codes, w, scales, sw, out, 0)

    # quantizer: exact on every row
    want_codes, want_scales = ref.quantize_rows_ref(inputs.x)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    # GEMM: exact on a row sample
    rows = torch.randperm(m, generator=torch.Generator().manual_seed(1))[:48].sort().values
    _, want = ref.fused_channel_mm_ref(want_codes[rows], inputs.w, want_scales[rows], inputs.w_scale, fast=True)
    assert_bit_equal(out[rows.to(DEV)], want, "sampled rows")

    # whole-output properties
    other = torch.empty_like(out)
    ops.fused_channel_mm(codes, w, scales, sw, other, 1)
    assert torch.equal(out, other), "one-CTA and two-CTA schedules differ"
    workspace = torch.empty(m, n, dtype=torch.int32, device=DEV)
    ops.cutlass_channel_mm(codes, w, scales, sw, workspace, other)
    assert torch.equal(out, other), "fused and workspace operators differ"
    acc_rows = ref.int_mm_fast(want_codes[rows], inputs.w)
    assert_bit_equal(workspace[rows.to(DEV)], acc_rows, "sampled accumulators")
    del workspace
    # the UINT8 code+128 form of the same weights (two-CTA biased tiles at this size)
    other.fill_(float("nan"))
    w_u8 = inputs.w_u8.to(DEV)
    ops.channel_mm(codes, w_u8, scales, sw, other)
    assert_bit_equal(other[rows.to(DEV)], want, "channel_mm sampled rows")
    assert torch.equal(out, other), "channel_mm and fused_channel_mm differ"
    del w_u8
    ops.fused_channel_mm(codes.neg(), w, scales, sw, other, 0)
    assert torch.equal(out.float(), -other.float()), "sign symmetry"
    perm = torch.randperm(m, device=DEV, generator=torch.Generator(device=DEV).manual_seed(2))
    ops.fused_channel_mm(codes[perm].contiguous(), w, scales[perm].contiguous(), sw, other, 0)
    assert torch.equal(out[perm], other), "row permutation"
    assert device_status(ops) == 0


@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_decode_config(ops, m):
    n, k = 34816, 5120
    inputs = workloads.linear_inputs(m, n, k, seed=0)
    codes, scales = quantize_on_gpu(ops, inputs.x.to(DEV))
    want_codes, want_scales = ref.quantize_rows_ref(inputs.x)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    _, want = ref.fused_channel_mm_ref(want_codes, inputs.w, want_scales, inputs.w_scale, fast=True)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(codes, inputs.w.to(DEV), scales, inputs.w_scale.to(DEV), out)
    assert_bit_equal(out, want, "fused_channel_mm")
    out.fill_(float("nan"))
    ops.channel_mm(codes, inputs.w_u8.to(DEV), scales, inputs.w_scale.to(DEV), out)
    assert_bit_equal(out, want, "channel_mm")
    if m <= 16:
        ops.channel_gemv(inputs.x.to(DEV), inputs.w.to(DEV), inputs.w_scale.to(DEV), out)
        gemv_want = ref.channel_gemv_fp64(inputs.x, inputs.w, inputs.w_scale)
        # W8A16 has BF16 activations, so compare with the FP64 oracle of that contract; outputs here
        # are O(10..100), so the reference's absolute tolerance is scaled by the output magnitude
        error = (out.cpu().float() - gemv_want.float()).norm() / gemv_want.float().norm()
        assert error.item() < 0.003


def test_grouped_config(ops):
    m, n, groups = 2048, 7168, 8
    inputs = workloads.grouped_inputs(m, n, groups, seed=0)
    codes = torch.empty(groups, m, 4096, dtype=torch.int8, device=DEV)
    scales = torch.empty(groups, m, device=DEV)
    ops.quantize_grouped4096(inputs.x.to(DEV), codes, scales)
    want_codes, want_scales = ref.quantize_grouped4096_ref(inputs.x)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.grouped_channel_mm(codes, inputs.w.to(DEV), scales, inputs.w_scale.to(DEV), out)
    rows = torch.randperm(m, generator=torch.Generator().manual_seed(3))[:64].sort().values
    want = ref.grouped_channel_mm_ref(want_codes[:, rows].contiguous(), want_scales[:, rows].contiguous(),
                                      inputs.w, inputs.w_scale, fast=True)
    assert_bit_equal(out[rows.to(DEV)], want, "sampled rows")
    # the same with a lent workspace: the two tiles of the fourth wave run split along the groups
    need = ops.grouped_workspace_bytes(m, n, groups)
    if need:
        workspace = torch.zeros(need, dtype=torch.uint8, device=DEV)
        split = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        for _ in range(2):
            ops.grouped_channel_mm_ws(codes, inputs.w.to(DEV), scales, inputs.w_scale.to(DEV), workspace, split)
        assert torch.equal(out, split), "the split along the groups changed the result"
    assert device_status(ops) == 0


def test_sharded_config_single_gpu_slice(ops):
    """Config 4 on one GPU: the N-shard of rank r is an ordinary GEMM on w[r*N/G:(r+1)*N/G];
    the concatenation of the shards equals the unsharded result."""
    m, n, k = 16384, 34816, 5120
    inputs = workloads.linear_inputs(m, n, k, seed=0)
    codes, scales = quantize_on_gpu(ops, inputs.x.to(DEV))
    w, sw = inputs.w.to(DEV), inputs.w_scale.to(DEV)
    full = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(codes, w, scales, sw, full, 0)
    world = 8
    shard = n // world
    for rank in (0, 3, 7):
        part = torch.empty(m, shard, dtype=torch.bfloat16, device=DEV)
        ops.fused_channel_mm(codes, w[rank * shard:(rank + 1) * shard], scales, sw[rank * shard:(rank + 1) * shard], part, 0)
        assert torch.equal(part, full[:, rank * shard:(rank + 1) * shard])
    rows = torch.randperm(m, generator=torch.Generator().manual_seed(4))[:32].sort().values
    want_codes, want_scales = ref.quantize_rows_ref(inputs.x[rows])
    _, want = ref.fused_channel_mm_ref(want_codes, inputs.w, want_scales, inputs.w_scale, fast=True)
    assert_bit_equal(full[rows.to(DEV)], want, "sampled rows")


def test_mlp_chain_fused_forms_at_full_size(ops):
    """The prefill MLP chain through the fused forms, at config 2's sizes: gate_up_silu_mm must equal
    fused_channel_mm + silu_mul over the whole [4096, 17408] output, and dynamic_channel_mm the
    quantizer + GEMM pair on the decode shape (a row sample of both is checked against the CPU checker
    through the unfused operators in test_prefill_configs and test_decode_config)."""
    from consumer_int8.quantization import interleave_gate_up

    m, n, k = 4096, 34816, 5120
    inputs = workloads.linear_inputs(m, n, k, seed=3)
    x, w, sw = inputs.x.to(DEV), inputs.w.to(DEV), (inputs.w_scale.float() * 4).bfloat16().to(DEV)
    codes, scales = quantize_on_gpu(ops, x)
    gate_up = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(codes, w, scales, sw, gate_up, 0)
    want = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    ops.silu_mul(gate_up, want)
    del gate_up
    wi, swi = interleave_gate_up(w, sw)
    got = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gate_up_silu_mm(codes, wi, scales, swi, got)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "fused SwiGLU GEMM differs from the pair"
    del wi, swi, got, want

    rows = 16
    out_pair = torch.empty(rows, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(codes[:rows], w, scales[:rows], sw, out_pair, 0)
    codes2 = torch.empty(rows, k, dtype=torch.int8, device=DEV)
    scales2 = torch.empty(rows, device=DEV)
    out_dynamic = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.dynamic_channel_mm(x[:rows], w, sw, codes2, scales2, out_dynamic)
    assert torch.equal(codes2, codes[:rows]) and torch.equal(scales2, scales[:rows])
    assert torch.equal(out_dynamic.view(torch.int16), out_pair.view(torch.int16)), "dynamic linear differs from the pair"
    assert device_status(ops) == 0

"""The CPU oracle against the reference's golden vectors, and its two restatements against
each other. No GPU needed."""
import ctypes
import hashlib
import json
from pathlib import Path

import pytest
import torch

from oracle import w8a8_ref as ref

GOLDEN = Path(__file__).resolve().parent / "golden"
ROOT = Path(__file__).resolve().parents[1]


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def ptr(t: torch.Tensor):
    return ctypes.c_void_p(t.data_ptr())


def test_activation_quantizer_known_answers():
    kat = json.loads((GOLDEN / "activation_kat.json").read_text())
    for row in kat["rows"]:
        if "x_bits" in row:
            x = torch.tensor(row["x_bits"], dtype=torch.int16).view(torch.bfloat16)
        else:
            x = torch.tensor([row["x"]], dtype=torch.float32).bfloat16()
        codes, scale = ref.quantize_rows_ref(x)
        assert codes.tolist() == (row["codes"] if "x_bits" in row else [row["codes"]]), row["name"]
        assert torch.equal(scale, torch.full_like(scale, row["scale"])), row["name"]


def test_weight_encoding_matches_reference_outputs():
    golden = json.loads((GOLDEN / "weight_encoding.json").read_text())
    for case in golden["cases"]:
        if case["name"] == "kat":
            weight = torch.tensor(case["weight"])
            codes, scale = ref.quantize_channel_ref(weight)
            assert codes.tolist() == case["codes"] == [[128, 1, 192, 255], [128, 128, 128, 128]]
            assert scale.view(torch.int16).tolist() == case["scale_bits"]
            continue
        g = torch.Generator().manual_seed(case["seed"])
        n, k = case["n"], case["k"]
        weight = torch.randn(n, k, generator=g) * (10.0 ** torch.randint(-3, 3, (n, 1), generator=g).float())
        weight[0] = 0
        codes, scale = ref.quantize_channel_ref(weight)
        assert sha(codes) == case["codes_sha256"]
        assert sha(scale) == case["scale_sha256"]
        assert codes[1, :16].tolist() == case["first_row_codes"]


def test_linear_known_answers():
    golden = json.loads((GOLDEN / "linear_kat.json").read_text())
    for case in golden["cases"]:
        g = torch.Generator().manual_seed(case["seed"])
        m, n, k = case["m"], case["n"], case["k"]
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=g)
        if case["biased"]:
            w = torch.randint(1, 256, (n, k), dtype=torch.uint8, generator=g)
        else:
            w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
        sa = torch.rand(m, generator=g) / 127
        sw = (torch.rand(n, generator=g) / 127).bfloat16()
        for fast in (False, True):
            fn = ref.channel_mm_ref if case["biased"] else ref.fused_channel_mm_ref
            acc, out = fn(a, w, sa, sw, fast=fast)
            assert sha(acc) == case["acc_sha256"]
            assert sha(out) == case["out_sha256"]
            assert acc[0, :8].tolist() == case["acc_first"]
    for case in golden["gemv"]:
        g = torch.Generator().manual_seed(case["seed"])
        m, n, k = case["m"], case["n"], case["k"]
        x = torch.randn(m, k, generator=g).bfloat16()
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
        scale = (torch.rand(n, generator=g) * 0.002).bfloat16()
        assert sha(ref.channel_gemv_fp64(x, w, scale)) == case["out_sha256"]


@pytest.mark.parametrize("m,k", [(3, 4), (5, 100), (4, 4096), (2, 5120)])
def test_c_checker_matches_torch_checker_quantizer(c_oracle, m, k):
    g = torch.Generator().manual_seed(m * 1000 + k)
    x = (torch.randn(m, k, generator=g) * 7).bfloat16()
    x[0].zero_()
    x[-1, : min(4, k)] = torch.tensor([0, -127, 63.5, 127][: min(4, k)]).bfloat16()
    codes, scale = ref.quantize_rows_ref(x)
    c_codes = torch.empty_like(codes)
    c_scale = torch.empty_like(scale)
    c_oracle.ci8o_quantize_rows(ptr(x), ptr(c_codes), ptr(c_scale), m, k)
    assert torch.equal(codes, c_codes)
    assert torch.equal(scale, c_scale)


def test_c_checker_matches_torch_checker_grouped_and_linear(c_oracle):
    g = torch.Generator().manual_seed(9)
    m, groups, n = 5, 2, 24
    x = (torch.randn(m, groups, 4096, generator=g) * torch.tensor([0.2, 6.0])[None, :, None]).bfloat16()
    codes, scales = ref.quantize_grouped4096_ref(x)
    c_codes, c_scales = torch.empty_like(codes), torch.empty_like(scales)
    c_oracle.ci8o_quantize_grouped4096(ptr(x), ptr(c_codes), ptr(c_scales), m, groups)
    assert torch.equal(codes, c_codes) and torch.equal(scales, c_scales)
    for group in range(groups):  # the reference's own definition (tests/test_cuda_ops.py:31-38)
        row_codes, row_scales = ref.quantize_rows_ref(x[:, group].contiguous())
        assert torch.equal(codes[group], row_codes) and torch.equal(scales[group], row_scales)

    w = torch.randint(-127, 128, (n, groups * 4096), dtype=torch.int8, generator=g)
    sw = (torch.rand(n, generator=g) * 0.019 + 0.001).bfloat16()
    want = ref.grouped_channel_mm_ref(codes, scales, w, sw)
    assert torch.equal(want, ref.grouped_channel_mm_ref(codes, scales, w, sw, fast=True))
    acc = torch.empty(groups, m, n, dtype=torch.int32)
    for group in range(groups):
        part = torch.empty(m, n, dtype=torch.int32)
        wg = w[:, group * 4096:(group + 1) * 4096].contiguous()
        c_oracle.ci8o_int_mm(ptr(codes[group].contiguous()), ptr(wg), 0, ptr(part), m, n, 4096)
        assert torch.equal(part, ref.int_mm_literal(codes[group], wg))
        acc[group] = part
    out = torch.empty(m, n, dtype=torch.bfloat16)
    c_oracle.ci8o_grouped_epilogue(ptr(acc), ptr(scales), ptr(sw), ptr(out), groups, m, n)
    assert torch.equal(out, want)
    # one group reduces to the plain fused operator
    one = ref.grouped_channel_mm_ref(codes[:1], scales[:1], w[:, :4096].contiguous(), sw)
    _, fused = ref.fused_channel_mm_ref(codes[0], w[:, :4096].contiguous(), scales[0], sw)
    assert torch.equal(one, fused)


def test_c_checker_biased_weights_and_epilogue(c_oracle):
    g = torch.Generator().manual_seed(17)
    m, n, k = 17, 37, 128
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=g)
    w = torch.randint(1, 256, (n, k), dtype=torch.uint8, generator=g)
    sa = torch.rand(m, generator=g) / 127
    sw = (torch.rand(n, generator=g) / 127).bfloat16()
    acc, out = ref.channel_mm_ref(a, w, sa, sw)
    c_acc = torch.empty_like(acc)
    c_out = torch.empty_like(out)
    c_oracle.ci8o_int_mm(ptr(a), ptr(w), 1, ptr(c_acc), m, n, k)
    c_oracle.ci8o_epilogue(ptr(c_acc), ptr(sa), ptr(sw), ptr(c_out), m, n)
    assert torch.equal(acc, c_acc) and torch.equal(out, c_out)


def test_fast_product_is_exact_at_worst_case_magnitudes():
    a = torch.full((3, 65536), -127, dtype=torch.int8)
    w = torch.full((2, 65536), -128, dtype=torch.int8)
    assert torch.equal(ref.int_mm_fast(a, w), torch.full((3, 2), 65536 * 127 * 128, dtype=torch.int32))


def test_config0_plumbing_runs_on_the_host():
    """The CPU-runnable benchmark case: M=8, K=4096, N=4096, seed 0 -> BF16 [8,4096]."""
    from consumer_int8 import workloads

    inputs = workloads.linear_inputs(8, 4096, 4096, seed=0, outliers=False)
    codes, scales = ref.quantize_rows_ref(inputs.x)
    _, out = ref.channel_mm_ref(codes, inputs.w_u8, scales, inputs.w_scale, fast=True)
    assert out.shape == (8, 4096) and out.dtype == torch.bfloat16
    assert torch.isfinite(out.float()).all()
    _, signed = ref.fused_channel_mm_ref(codes, inputs.w, scales, inputs.w_scale, fast=True)
    assert torch.equal(out, signed)


def test_allspark_unpack_restatement_follows_the_reference_index_arithmetic():
    """The vectorised restatement against a literal scalar walk of the reference's kernel
    (csrc/allspark_layout.cu:10-27) on a small case, and pack/unpack as mutual inverses."""
    import numpy as np

    n, k = 48, 32
    g = torch.Generator().manual_seed(5)
    packed = torch.randint(0, 256, (64, k), dtype=torch.uint8, generator=g)
    packed_scales = torch.randn(64, generator=g).bfloat16()
    words = packed.contiguous().view(-1).numpy().view("<u4")
    want = np.zeros((n, k), dtype=np.int8)
    for row in range(n):
        for tile in range(k // 16):
            packed_row = (row // 32) * 8 + row % 8
            offset = packed_row * k * 4 + tile * 64 + ((row % 32) // 16) * 8 + ((row % 16) // 8) * 4
            a, b, c, d = (int(words[offset // 4 + i]) for i in (0, 4, 8, 12))
            restored = [((a & 0xFFFF) | (b << 16)) & 0xFFFFFFFF, ((c & 0xFFFF) | (d << 16)) & 0xFFFFFFFF,
                        (a >> 16) | (b & 0xFFFF0000), (c >> 16) | (d & 0xFFFF0000)]
            raw = np.array([w ^ 0x80808080 for w in restored], dtype="<u4").view(np.int8)
            want[row, tile * 16:(tile + 1) * 16] = raw
    codes, scales = ref.unpack_allspark_ref(packed, packed_scales, n, k)
    assert np.array_equal(codes.numpy(), want)
    for row in (0, 7, 8, 31, 32, 47):
        assert scales[row] == packed_scales[(row // 32) * 32 + (row % 8) * 4 + (row % 32) // 8]
    repacked, repacked_scales = ref.pack_allspark_ref((codes.short() + 128).to(torch.uint8), scales)
    again, again_scales = ref.unpack_allspark_ref(repacked, repacked_scales, n, k)
    assert torch.equal(again, codes) and torch.equal(again_scales.view(torch.int16), scales.view(torch.int16))


def _q8_case(m, n, k, seed):
    """Inputs shaped like the reference's benchmark (benchmarks/benchmark_q8_block_int8.py:57-66): Q8_0
    codes over the whole INT8 range, FP16 block scales ~0.01, activations ~0.1 with one all-zero
    block and one block a hundred times larger."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=g)
    sw = (torch.randn(n, k // 32, generator=g) * 0.01).half()
    x = (torch.randn(m, k, generator=g) * 0.1).bfloat16()
    x[:, :32] = 0
    if k >= 64:
        x[:, 32:64] *= 100
    return x, w, sw


@pytest.mark.parametrize("m,n,k", [(1, 1, 32), (17, 33, 96), (129, 65, 256), (8, 40, 1024)])
def test_block32_checkers_agree_and_sit_inside_the_reference_tolerance(c_oracle, m, n, k):
    x, w, sw = _q8_case(m, n, k, 100 + m)
    codes, sa = ref.q8_block_quantize_ref(x)
    c_codes, c_sa = torch.empty_like(codes), torch.empty_like(sa)
    c_oracle.ci8o_q8_block_quantize(ptr(x), ptr(c_codes), ptr(c_sa), ctypes.c_int64(m * (k // 32)))
    assert torch.equal(codes, c_codes) and torch.equal(sa, c_sa)
    # the reference's own assertions on the quantizer (benchmark_q8_block_int8.py:90-101)
    blocks = x.float().reshape(m, k // 32, 32)
    expected_scale = (blocks.abs().amax(-1) / 127).clamp_min(1e-20)
    torch.testing.assert_close(sa, expected_scale, rtol=1e-6, atol=0)
    assert ((codes.reshape(m, k // 32, 32).float() - blocks / expected_scale[..., None]).abs() <= 0.50002).all()
    y = ref.q8_block_mm_ref(codes, w, sa, sw)
    c_y = torch.empty_like(y)
    c_oracle.ci8o_q8_block_mm(ptr(codes), ptr(w), ptr(sa), ptr(sw), ptr(c_y), m, n, k)
    assert torch.equal(y.view(torch.int16), c_y.view(torch.int16))
    torch.testing.assert_close(y, ref.q8_block_mm_loose_ref(codes, w, sa, sw), rtol=0.008, atol=1e-5)


def test_reference_block32_validator_passed_against_the_c_checker():
    """The reference's own validation script for the block-32 path (benchmarks/benchmark_q8_block_int8.py)
    was run, unmodified, against the C checker's host twin of its entry point; the record of that run is
    a fixture. With CI8_REFERENCE_ROOT pointing at a checkout of the reference the run is repeated here
    and must reproduce the record."""
    import json
    import os

    record = json.loads((ROOT / "tests" / "golden" / "q8_block_validator.json").read_text())
    assert record["passed"] is True and record["reference_script"] == "benchmarks/benchmark_q8_block_int8.py"
    shapes = {(s["m"], s["n"], s["k"]): s for s in record["shapes"]}
    assert set(shapes) == {(1, 1, 32), (17, 33, 96), (129, 65, 256)}      # the script's default shapes
    for s in shapes.values():
        assert s["entry"] == "q8_block_int8" and all(e < 0.015 for e in s["relative_l2"])
    reference = os.environ.get("CI8_REFERENCE_ROOT")
    if reference:
        import importlib.util
        import subprocess

        subprocess.run(["make", "-s", "-C", str(ROOT / "oracle")], check=True)
        spec = importlib.util.spec_from_file_location("run_reference_q8_validator",
                                                      ROOT / "tests" / "golden" / "run_reference_q8_validator.py")
        runner = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(runner)
        again = runner.run(Path(reference), ROOT / "oracle" / "libci8_oracle.so")
        assert again["reference_script_sha256"] == record["reference_script_sha256"]
        assert again["shapes"] == record["shapes"]

"""fused_channel_mm / cutlass_channel_mm / channel_mm on the GPU against the CPU checker:
INT32 accumulators and BF16 outputs bit for bit. Shapes and assertions follow the reference's
tests/test_cuda_ops.py:474-490,563-600; further cases cover tile, K and N tails of the
tcgen05 kernel, the decode kernel's split-K factors, and graph replay on mutated inputs."""
import ctypes

import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status, guarded, linear_case, to_u8
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(1, 5120, 5120), (4, 2560, 3072), (17, 37, 128)])
def test_channel_mm_matches_integer_product_with_output_tails(ops, m, n, k):
    generator = torch.Generator(device=DEV).manual_seed(17)
    a = torch.randint(-127, 128, (m, k), device=DEV, dtype=torch.int8, generator=generator)
    w = torch.randint(1, 256, (n, k), device=DEV, dtype=torch.uint8, generator=generator)
    sa = torch.rand(m, device=DEV, generator=generator) / 127
    sw = (torch.rand(n, device=DEV, generator=generator) / 127).bfloat16()
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops.channel_mm(a, w, sa, sw, out)
    integer = a.cpu().int() @ (w.cpu().int() - 128).T
    expected = (integer.float().to(DEV) * sa[:, None] * sw.float()[None, :]).bfloat16()
    torch.testing.assert_close(out, expected, rtol=0, atol=0)
    _, want = ref.channel_mm_ref(a.cpu(), w.cpu(), sa.cpu(), sw.cpu())
    assert_bit_equal(out, want, "channel_mm vs checker")


def test_channel_mm_rejects_unaligned_k_before_launch(ops):
    with pytest.raises(RuntimeError, match="geometry"):
        ops.channel_mm(
            torch.zeros(1, 33, dtype=torch.int8, device=DEV),
            torch.zeros(4, 33, dtype=torch.uint8, device=DEV),
            torch.ones(1, device=DEV),
            torch.ones(4, dtype=torch.bfloat16, device=DEV),
            torch.empty(1, 4, dtype=torch.bfloat16, device=DEV),
        )


def test_tiled_operators_reject_bad_geometry_and_schedule(ops):
    a = torch.zeros(2, 64, dtype=torch.int8, device=DEV)
    sa = torch.ones(2, device=DEV)
    out6 = torch.empty(2, 6, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="geometry"):      # n % 4 != 0
        ops.fused_channel_mm(a, torch.zeros(6, 64, dtype=torch.int8, device=DEV), sa,
                             torch.ones(6, dtype=torch.bfloat16, device=DEV), out6)
    w = torch.zeros(8, 64, dtype=torch.int8, device=DEV)
    sw = torch.ones(8, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(2, 8, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="schedule"):
        ops.fused_channel_mm(a, w, sa, sw, out, 7)
    with pytest.raises(RuntimeError, match="workspace"):
        ops.cutlass_channel_mm(a, w, sa, sw, torch.empty(2, 4, dtype=torch.int32, device=DEV), out)
    with pytest.raises(RuntimeError, match="dtype"):
        ops.fused_channel_mm(a, w.to(torch.uint8), sa, sw, out)


@pytest.mark.parametrize("m", [1, 17, 64, 256, 1024, 1041, 2048, 2057])
@pytest.mark.parametrize("fused", [None, 0, 1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("n,k", [(128, 512), (132, 544)])
def test_gemm_schedules_match_integer_products_and_capture(ops, m, fused, n, k):
    torch.manual_seed(m * 7 + n)
    a = torch.randint(-127, 128, (m, k), device=DEV, dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), device=DEV, dtype=torch.int8)
    sa = torch.rand(m, device=DEV) / 127
    sw = (torch.rand(n, device=DEV) / 127).bfloat16()
    workspace = torch.empty(m, n, device=DEV, dtype=torch.int32)
    out = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)

    def run():
        if fused is not None:
            ops.fused_channel_mm(a, w, sa, sw, out, fused)
        else:
            ops.cutlass_channel_mm(a, w, sa, sw, workspace, out)

    run()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    out.fill_(float("nan"))
    workspace.fill_(-1)
    graph.replay()
    integer = a.cpu().int() @ w.cpu().int().T
    if fused is None:
        torch.testing.assert_close(workspace.cpu(), integer, atol=0, rtol=0)
    expected = (integer.float().to(DEV) * sa[:, None] * sw.float()[None, :]).bfloat16()
    torch.testing.assert_close(out, expected, atol=0, rtol=0)
    assert device_status(ops) == 0


# Tails of the 128x256x128 (and 256x256 pair) tiling, K not a multiple of the 128-byte stage,
# more tiles than SMs, several K stages around the ring.
TILE_CASES = [(128, 256, 128), (129, 260, 160), (255, 508, 96), (300, 1000, 1056), (513, 4, 32),
              (777, 2052, 4096), (4096, 512, 256), (100, 40000, 64), (3000, 3000, 3008),
              # more tiles than CTAs with a small last wave: schedule 0 picks a narrower tile there
              (2048, 7168, 256), (2048, 7136, 160), (4096, 5120, 256), (1300, 30000, 96)]


@pytest.mark.parametrize("m,n,k", TILE_CASES)
@pytest.mark.parametrize("schedule", [0, 1, 2, 3, 4, 5, 6])
def test_fused_channel_mm_tile_and_k_tails(ops, m, n, k, schedule):
    a, w, sa, sw = linear_case(m, n, k, seed=m + n + k)
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.fused_channel_mm(a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV), out, schedule)
    _, want = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    assert_bit_equal(out, want, f"fused schedule {schedule}")
    check()
    assert device_status(ops) == 0


@pytest.mark.parametrize("m,n,k", [(3, 37, 128), (70, 200, 256), (300, 520, 1024)])
@pytest.mark.parametrize("shift_a,shift_w", [(4, 0), (0, 4), (8, 12)])
def test_channel_mm_accepts_operands_that_are_only_four_byte_aligned(ops, m, n, k, shift_a, shift_w):
    """The reference reads its operands as 32-bit words (csrc/kernels.cu:99,105) and checks no
    alignment, so views at a 4-byte offset into a larger buffer must work here as well."""
    a, w, sa, sw = linear_case(m, n, k, seed=m + n)
    a_store = torch.zeros(m * k + 64, dtype=torch.int8, device=DEV)
    w_store = torch.zeros(n * k + 64, dtype=torch.uint8, device=DEV)
    da = a_store[shift_a:shift_a + m * k].view(m, k)
    dw = w_store[shift_w:shift_w + n * k].view(n, k)
    da.copy_(a)
    dw.copy_(to_u8(w))
    assert da.data_ptr() % 16 == shift_a % 16 and dw.data_ptr() % 16 == shift_w % 16
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.channel_mm(da, dw, sa.to(DEV), sw.to(DEV), out)
    _, want = ref.channel_mm_ref(a, to_u8(w), sa, sw)
    assert_bit_equal(out, want, "channel_mm on 4-byte aligned views")
    check()


def _tile_plan(ops, m, n, k, groups=1):
    plan = (ctypes.c_int * 4)()
    assert ops.libci8.ci8_gemm_tile_plan(m, n, k, groups, plan) == 0
    return dict(tile_n=plan[0], tiles_n=plan[1], wide_tiles=plan[2], split=plan[3])


# Shapes whose automatic tiling mixes two tile widths (some channel tiles 32 columns wider than the
# rest, so that the tiles fill whole waves); N tails and a ragged last unit included.
MIXED_CASES = [(2048, 7168, 256), (2048, 7136, 160), (512, 14336, 256), (700, 14300, 96)]


@pytest.mark.parametrize("m,n,k", MIXED_CASES)
def test_mixed_tile_widths_match_checker(ops, m, n, k):
    plan = _tile_plan(ops, m, n, k)
    assert plan["wide_tiles"] > 0 and plan["split"] == 1, f"this shape no longer exercises the mixed widths: {plan}"
    a, w, sa, sw = linear_case(m, n, k, seed=m + n + k)
    da, dw, dsa, dsw = a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV)
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.fused_channel_mm(da, dw, dsa, dsw, out, 0)
    acc, want = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    assert_bit_equal(out, want, f"fused, mixed widths {plan}")
    check()
    workspace, check_ws = guarded((m, n), torch.int32, -1)
    out2, check2 = guarded((m, n), torch.bfloat16, float("nan"))
    ops.cutlass_channel_mm(da, dw, dsa, dsw, workspace, out2)
    assert_bit_equal(workspace, acc, "accumulators, mixed widths")
    assert_bit_equal(out2, want, "workspace form, mixed widths")
    check_ws()
    check2()
    assert device_status(ops) == 0


@pytest.mark.parametrize("m,n,k", [(17, 37, 128), (128, 240, 128), (130, 241, 160), (300, 500, 1024),
                                   (64, 5120, 5120), (1000, 1000, 992), (2048, 4096, 4096),
                                   # edges of the 248-channel tile, one CTA (m <= 128) and a CTA pair, with and
                                   # without an output pitch that allows TMA tile stores (n % 8)
                                   (100, 248, 128), (128, 249, 160), (129, 248, 96), (257, 504, 256), (300, 2000, 96),
                                   (513, 377, 64), (4096, 1000, 64), (256, 128, 32), (1300, 30000, 96)])
def test_channel_mm_biased_weights_on_the_tensor_core_path(ops, m, n, k):
    a, w, sa, sw = linear_case(m, n, k, seed=3 * m + n)
    # extreme rows: the 128*sum(a) correction is largest when every activation is +-127
    a[0] = 127
    a[-1] = -127
    wu = to_u8(w)
    wu[0] = 255
    wu[-1] = 0
    out, check = guarded((m, n), torch.bfloat16, float("nan"))
    ops.channel_mm(a.to(DEV), wu.to(DEV), sa.to(DEV), sw.to(DEV), out)
    _, want = ref.channel_mm_ref(a, wu, sa, sw, fast=True)
    assert_bit_equal(out, want, "channel_mm")
    check()


@pytest.mark.parametrize("m,n,k", [(17, 128, 512), (200, 132, 544), (1041, 260, 1056), (16, 132, 544), (3, 4, 32),
                                   # 65..128 rows: the one-CTA tile with its INT32 tile stores; a pitch that rules them out
                                   (100, 260, 160), (128, 512, 256), (90, 1000, 96), (300, 1004, 96)])
def test_cutlass_channel_mm_writes_exact_accumulators(ops, m, n, k):
    a, w, sa, sw = linear_case(m, n, k, seed=m * n)
    out, check_out = guarded((m, n), torch.bfloat16, float("nan"))
    ws, check_ws = guarded((m, n), torch.int32, -7)
    ops.cutlass_channel_mm(a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV), ws, out)
    acc, want = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    assert_bit_equal(ws, acc, "INT32 accumulators")
    assert_bit_equal(out, want, "BF16 out")
    check_out()
    check_ws()


def test_worst_case_accumulator_magnitude(ops):
    """K = 65536 with every product at its extreme: |acc| = 65536*127*127 (signed weights) and
    the biased form's intermediate 65536*127*255 still fit in INT32."""
    m, n, k = 20, 8, 65536
    a = torch.full((m, k), 127, dtype=torch.int8)
    a[1] = -127
    w = torch.full((n, k), -127, dtype=torch.int8)
    w[1] = 127
    sa = torch.full((m,), 1.0 / 127)
    sw = torch.full((n,), 1.0 / 127).bfloat16()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ws = torch.empty(m, n, dtype=torch.int32, device=DEV)
    ops.cutlass_channel_mm(a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV), ws, out)
    acc, want = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    assert int(acc.abs().max()) == 65536 * 127 * 127
    assert_bit_equal(ws, acc, "accumulators")
    assert_bit_equal(out, want, "out")
    ops.channel_mm(a.to(DEV), to_u8(w).to(DEV), sa.to(DEV), sw.to(DEV), out)
    assert_bit_equal(out, want, "biased out")
    for rows in (16, 3):    # the decode kernel, same extremes
        ops.channel_mm(a[:rows].to(DEV), to_u8(w).to(DEV), sa[:rows].to(DEV), sw.to(DEV), out[:rows])
        assert_bit_equal(out[:rows], want[:rows], "decode biased out")


# ------------------------------------------------------------------ streaming kernel (M <= 64)
DECODE_CASES = [(1, 128, 128), (1, 128, 512), (4, 256, 512), (16, 240, 1024), (8, 132, 544), (3, 37, 128),
                (16, 5120, 5120), (5, 1000, 17408), (2, 34816, 320),
                # 17..64 rows: the 64-row activation tile (every TMEM lane quarter holds real rows)
                (17, 128, 256), (32, 240, 1024), (33, 37, 128), (48, 132, 544), (64, 5120, 5120), (63, 1000, 4352)]


@pytest.mark.parametrize("m,n,k", DECODE_CASES)
@pytest.mark.parametrize("biased", [False, True])
def test_decode_kernel_is_split_invariant(ops, m, n, k, biased):
    a, w, sa, sw = linear_case(m, n, k, seed=m + 2 * n + 3 * k)
    acc, want = ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)
    weights = (to_u8(w) if biased else w).to(DEV)
    ad, sad, swd = a.to(DEV), sa.to(DEV), sw.to(DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for split in (1, 2, 4):
        if split > (k + 127) // 128 or (m > 16 and split > 2):
            continue
        out, check_out = guarded((m, n), torch.bfloat16, float("nan"))
        ws, check_ws = guarded((m, n), torch.int32, -7)
        rc = ops.libci8.ci8_decode_mm_split(
            ctypes.c_void_p(ad.data_ptr()), ctypes.c_void_p(weights.data_ptr()), ctypes.c_void_p(sad.data_ptr()),
            ctypes.c_void_p(swd.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(out.data_ptr()),
            m, n, k, split, int(biased), stream)
        assert rc == 0
        assert_bit_equal(ws, acc, f"accumulators, split {split}")
        assert_bit_equal(out, want, f"out, split {split}")
        check_out()
        check_ws()
    # and through the operators, with the split chosen from the shape
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    if biased:
        ops.channel_mm(ad, weights, sad, swd, out)
    elif n % 4 == 0:
        ops.fused_channel_mm(ad, weights, sad, swd, out)
    else:
        return
    assert_bit_equal(out, want, "operator")
    assert device_status(ops) == 0


def test_decode_graph_replay_on_new_activations(ops):
    m, n, k = 8, 5120, 5120
    a, w, sa, sw = linear_case(m, n, k, seed=5)
    ad, wd, sad, swd = a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(ad, wd, sad, swd, out)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.fused_channel_mm(ad, wd, sad, swd, out)
    a2 = torch.randint(-127, 128, (m, k), dtype=torch.int8)
    ad.copy_(a2)
    sad.mul_(0.5)
    out.fill_(float("nan"))
    allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
    graph.replay()
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations
    _, want = ref.fused_channel_mm_ref(a2, w, sa * 0.5, sw, fast=True)
    assert_bit_equal(out, want, "replayed decode")


def test_quantize_then_mm_pipeline_matches_checker(ops):
    """The composed path of benchmark config 0 (M=8, K=4096, N=4096, seed 0) on the GPU."""
    from consumer_int8 import workloads

    inputs = workloads.linear_inputs(8, 4096, 4096, seed=0, outliers=False)
    x = inputs.x.to(DEV)
    codes = torch.empty(8, 4096, dtype=torch.int8, device=DEV)
    scales = torch.empty(8, device=DEV)
    out = torch.empty(8, 4096, dtype=torch.bfloat16, device=DEV)
    ops.quantize_rows(x, codes, scales)
    ops.channel_mm(codes, inputs.w_u8.to(DEV), scales, inputs.w_scale.to(DEV), out)
    want_codes, want_scales = ref.quantize_rows_ref(inputs.x)
    _, want = ref.channel_mm_ref(want_codes, inputs.w_u8, want_scales, inputs.w_scale, fast=True)
    assert_bit_equal(codes, want_codes, "codes")
    assert_bit_equal(scales, want_scales, "scales")
    assert_bit_equal(out, want, "out")
    ops.fused_channel_mm(codes, inputs.w.to(DEV), scales, inputs.w_scale.to(DEV), out)
    assert_bit_equal(out, want, "signed-weight out")


def test_a_wait_that_runs_out_sets_the_status_word_and_leaves_the_context_usable(ops):
    """Failure detection without faulting the GPU: a kernel waits on a barrier that nothing ever
    arrives on; its bounded wait gives up after 20 ms, the status word reads 1, and the very next
    launches on the same context are correct."""
    assert device_status(ops) == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert ops.libci8.ci8_selftest_wait_timeout(20000, ctypes.c_void_p(gave_up.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert gave_up.item() == 1
    assert device_status(ops) == 1          # bit 0: a wait ran past its deadline
    assert device_status(ops) == 0          # reading clears it
    a, w, sa, sw = linear_case(200, 256, 512, seed=1)
    out = torch.empty(200, 256, dtype=torch.bfloat16, device=DEV)
    ops.fused_channel_mm(a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV), out)
    _, want = ref.fused_channel_mm_ref(a, w, sa, sw)
    assert_bit_equal(out, want, "GEMM after a timed-out wait")
    assert device_status(ops) == 0


def test_a_cluster_rendezvous_that_runs_out_sets_its_own_status_bit(ops):
    """The split-K kernel's leader waits for its peers' partial sums on a barrier they arrive on from
    another CTA. Here a two-CTA cluster runs in which the peer never arrives: the leader gives up
    after 20 ms, status bit 1 (value 2) is raised, both CTAs leave, and a split-K product on the same
    context right afterwards is bit-exact."""
    assert device_status(ops) == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert ops.libci8.ci8_selftest_cluster_timeout(20000, ctypes.c_void_p(gave_up.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert gave_up.item() == 1
    assert device_status(ops) == 2          # bit 1: a rendezvous between CTAs ran past its deadline
    assert device_status(ops) == 0
    m, n, k = 8, 640, 2048
    a, w, sa, sw = linear_case(m, n, k, seed=4)
    _, want = ref.fused_channel_mm_ref(a, w, sa, sw)
    for split in (2, 4):
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        da, dw, dsa, dsw = a.to(DEV), w.to(DEV), sa.to(DEV), sw.to(DEV)
        rc = ops.libci8.ci8_decode_mm_split(*(ctypes.c_void_p(t.data_ptr()) for t in (da, dw, dsa, dsw)), ctypes.c_void_p(0),
                                            ctypes.c_void_p(out.data_ptr()), m, n, k, split, 0, stream)
        assert rc == 0
        assert_bit_equal(out, want, f"split-K {split} after a timed-out rendezvous")
    assert device_status(ops) == 0


def test_status_word_can_be_collected_inside_a_captured_graph(ops):
    """ci8_device_status synchronises and cannot be captured; ci8_device_status_async moves the word into a
    caller-owned word on the stream instead. Captured behind a wait that runs out, a replay leaves the
    bit in that word and the library's own word clear."""
    assert device_status(ops) == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = ops.libci8
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        stream = ctypes.c_void_p(side.cuda_stream)
        assert lib.ci8_device_status_async(ctypes.c_void_p(word.data_ptr()), stream) == 0     # warm-up, nothing to report
        torch.cuda.synchronize()
        assert word.item() == 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            assert lib.ci8_selftest_wait_timeout(5000, ctypes.c_void_p(gave_up.data_ptr()), stream) == 0
            assert lib.ci8_device_status_async(ctypes.c_void_p(word.data_ptr()), stream) == 0
        graph.replay()
        torch.cuda.synchronize()
    assert gave_up.item() == 1 and word.item() == 1
    assert device_status(ops) == 0           # the library's word was cleared by the collecting kernel
    assert lib.ci8_device_status_async(ctypes.c_void_p(0), ctypes.c_void_p(0)) == 1

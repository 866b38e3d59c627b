"""unpack_allspark: the GPU kernel against the CPU restatement of the reference's index arithmetic,
on cells packed by the algebraic inverse; shapes of the reference's test
(tests/test_cuda_ops.py:440-471), graph replay on repacked inputs."""
import pytest
import torch

from gpu_common import DEV, assert_bit_equal, guarded
from oracle import w8a8_ref as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(16, 16), (48, 80), (128, 512), (5120, 3072), (34816, 5120)])
def test_allspark_unpack_preserves_every_code_and_scale_in_graph(ops, n, k):
    generator = torch.Generator().manual_seed(319)
    codes = torch.randint(0, 256, (n, k), dtype=torch.uint8, generator=generator)
    scales = torch.randn(n, generator=generator).bfloat16()
    packed_cpu, packed_scales_cpu = ref.pack_allspark_ref(codes, scales)
    packed, packed_scales = packed_cpu.to(DEV), packed_scales_cpu.to(DEV)
    restored, check_w = guarded((n, k), torch.int8, 77)
    restored_scales, check_s = guarded((n,), torch.bfloat16, float("nan"))
    graph = torch.cuda.CUDAGraph()
    ops.unpack_allspark(packed, packed_scales, restored, restored_scales)
    with torch.cuda.graph(graph):
        ops.unpack_allspark(packed, packed_scales, restored, restored_scales)
    for _ in range(2):
        restored.zero_()
        restored_scales.zero_()
        graph.replay()
        want_codes, want_scales = ref.unpack_allspark_ref(packed.cpu(), packed_scales.cpu(), n, k)
        assert_bit_equal(restored, want_codes, "codes vs checker")
        assert_bit_equal(restored_scales, want_scales, "scales vs checker")
        assert torch.equal(restored.cpu(), (codes.short() - 128).to(torch.int8))     # lossless round trip
        assert torch.equal(restored_scales.cpu().view(torch.int16), scales.view(torch.int16))
        check_w()
        check_s()
        codes.bitwise_xor_(255)
        scales.neg_()
        changed, changed_scales = ref.pack_allspark_ref(codes, scales)
        packed.copy_(changed)
        packed_scales.copy_(changed_scales)


def test_unpacked_weights_feed_the_gemm(ops):
    """unpack_allspark -> quantize_rows -> fused_channel_mm, the chain of
    benchmarks/microbench.py:46-53 in the reference, equals channel_mm on the UINT8 codes."""
    from consumer_int8 import workloads

    inputs = workloads.linear_inputs(64, 256, 512, seed=9)
    packed, packed_scales = ref.pack_allspark_ref(inputs.w_u8, inputs.w_scale)
    weight = torch.empty(256, 512, dtype=torch.int8, device=DEV)
    scales = torch.empty(256, dtype=torch.bfloat16, device=DEV)
    ops.unpack_allspark(packed.to(DEV), packed_scales.to(DEV), weight, scales)
    codes = torch.empty(64, 512, dtype=torch.int8, device=DEV)
    row_scales = torch.empty(64, device=DEV)
    ops.quantize_rows(inputs.x.to(DEV), codes, row_scales)
    out, direct = (torch.empty(64, 256, dtype=torch.bfloat16, device=DEV) for _ in range(2))
    ops.fused_channel_mm(codes, weight, row_scales, scales, out)
    ops.channel_mm(codes, inputs.w_u8.to(DEV), row_scales, inputs.w_scale.to(DEV), direct)
    assert torch.equal(out, direct)


def test_unpack_rejects_wrong_geometry(ops):
    packed = torch.zeros(32, 32, dtype=torch.uint8, device=DEV)
    packed_scales = torch.zeros(32, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="AllSpark N32K16"):
        ops.unpack_allspark(packed, packed_scales, torch.empty(24, 32, dtype=torch.int8, device=DEV),
                            torch.empty(24, dtype=torch.bfloat16, device=DEV))


_VLLM_PROBE = """
import torch
from vllm import _custom_ops as vops
probe = torch.zeros(32, 16, dtype=torch.uint8, device="cuda")
vops.allspark_repack_weight(probe.T.contiguous(), torch.ones(1, 32, dtype=torch.bfloat16, device="cuda"), None, False)
torch.cuda.synchronize()
torch.zeros(1, device="cuda").add_(1)   # a launch error of the call above ("no kernel image") surfaces here
torch.cuda.synchronize()
"""
_vllm_verdict = None


def _vllm_packer():
    """vLLM's own AllSpark packer, which is what the reference's test packs with
    (tests/test_cuda_ops.py:440-471). Whether the installed vLLM can run it on this GPU is found out in a
    child process, once, so that a failing launch cannot touch this process; the test skips if it cannot."""
    global _vllm_verdict
    if _vllm_verdict is None:
        import subprocess
        import sys

        try:
            child = subprocess.run([sys.executable, "-c", _VLLM_PROBE], capture_output=True, text=True, timeout=300)
            lines = [line.strip() for line in (child.stderr or "").splitlines() if "error" in line.lower()]
            _vllm_verdict = "ok" if child.returncode == 0 else (lines[0][:160] if lines else f"exit code {child.returncode}")
        except Exception as error:
            _vllm_verdict = f"{type(error).__name__}"
    if _vllm_verdict != "ok":
        pytest.skip(f"vLLM's allspark_repack_weight does not run here: {_vllm_verdict}")
    from vllm import _custom_ops as vops

    return vops.allspark_repack_weight


@pytest.mark.parametrize("n,k", [(16, 16), (48, 80), (128, 512), (5120, 3072)])
def test_allspark_unpack_inverts_vllms_own_packer(ops, n, k):
    """The reference's test, with the reference's packer: codes and scales packed by vLLM's
    allspark_repack_weight come back bit for bit, from a captured graph, twice, on repacked inputs."""
    repack = _vllm_packer()
    generator = torch.Generator(device=DEV).manual_seed(319)
    codes = torch.randint(0, 256, (n, k), device=DEV, dtype=torch.uint8, generator=generator)
    scales = torch.randn(n, device=DEV, dtype=torch.bfloat16, generator=generator)
    packed, packed_scales, _ = repack(codes.T.contiguous(), scales[None], None, False)
    packed_scales = packed_scales.flatten()
    restored = torch.empty_like(codes, dtype=torch.int8)
    restored_scales = torch.empty_like(scales)
    ops.unpack_allspark(packed, packed_scales, restored, restored_scales)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.unpack_allspark(packed, packed_scales, restored, restored_scales)
    for _ in range(2):
        restored.zero_()
        restored_scales.zero_()
        graph.replay()
        torch.testing.assert_close(restored, (codes.short() - 128).char(), atol=0, rtol=0)
        torch.testing.assert_close(restored_scales, scales, atol=0, rtol=0)
        # the CPU checker and its packer agree with vLLM's layout as well
        want_packed, want_packed_scales = ref.pack_allspark_ref(codes.cpu(), scales.cpu())
        if n % 32 == 0:      # (with padding rows the two packers may fill the padding differently)
            assert torch.equal(packed.cpu().reshape(-1), want_packed.reshape(-1)), "the checker's packer and vLLM's differ"
            assert torch.equal(packed_scales.cpu().view(torch.int16), want_packed_scales.view(torch.int16))
        codes.bitwise_xor_(255)
        scales.neg_()
        changed, changed_scales, _ = repack(codes.T.contiguous(), scales[None], None, False)
        packed.copy_(changed)
        packed_scales.copy_(changed_scales.flatten())

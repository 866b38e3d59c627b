"""The drop-in boundary without a GPU: the C-ABI library loads and exports every symbol that
include/ci8.h declares, the operator module registers the reference's schemas, and nothing
computes on the CPU (there is no fallback)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]

SCHEMAS = {  # the reference's csrc/bindings.cpp:599,603-606,610
    "fused_channel_mm": "consumer_int8::fused_channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) out, int schedule=0) -> ()",
    "quantize_rows": "consumer_int8::quantize_rows(Tensor input, Tensor(a!) codes, Tensor(b!) scales) -> ()",
    "quantize_grouped4096": "consumer_int8::quantize_grouped4096(Tensor input, Tensor(a!) codes, Tensor(b!) scales) -> ()",
    "channel_mm": "consumer_int8::channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) out) -> ()",
    "channel_gemv": "consumer_int8::channel_gemv(Tensor x, Tensor w, Tensor scale, Tensor(a!) out) -> ()",
    "cutlass_channel_mm": "consumer_int8::cutlass_channel_mm(Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor(a!) workspace, Tensor(b!) out) -> ()",
}


def declared_symbols() -> list[str]:
    header = (ROOT / "include" / "ci8.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return re.findall(r"\b((?:ci8_|q8_block_)[a-z0-9_]+)\s*\(", header)


def test_library_exports_every_declared_symbol(ops):
    names = declared_symbols()
    assert len(names) >= 10 and "ci8_fused_channel_mm" in names and "ci8_quantize_rows" in names
    lib = ctypes.CDLL(str(ROOT / "consumer-int8-kernels_b200" / "consumer_int8" / "libci8.so"))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/ci8.h but not exported"
    assert lib.ci8_abi_version() == 2
    lib.ci8_error_string.restype = ctypes.c_char_p
    assert lib.ci8_error_string(0) == b"success"
    assert b"invalid" in lib.ci8_error_string(1).lower()


def test_arguments_are_rejected_before_any_launch(ops):
    """Bad sizes come back as cudaErrorInvalidValue (1) without touching a device."""
    lib = ops.libci8
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: the size checks fail first
    assert lib.ci8_quantize_rows(null, null, null, 4, 4, null) == 1
    assert lib.ci8_quantize_rows(one, one, one, 0, 4, null) == 1
    assert lib.ci8_quantize_grouped4096(one, one, one, -1, 4, null) == 1
    assert lib.ci8_quantize_grouped4096(one, one, one, 0, 4, null) == 0      # empty M is a no-op
    assert lib.ci8_fused_channel_mm(one, one, one, one, one, 1, 4, 33, 0, null) == 1   # k % 32
    assert lib.ci8_fused_channel_mm(one, one, one, one, one, 1, 4, 32, 7, null) == 1   # schedule
    assert lib.ci8_fused_channel_mm(one, one, one, one, one, 1, 4, 65568, 0, null) == 1  # k > 65536
    assert lib.ci8_channel_mm(one, one, one, one, one, 1, 4, 33, null) == 1
    assert lib.ci8_channel_mm(ctypes.c_void_p(6), one, one, one, one, 1, 4, 32, null) == 1  # not even 4-byte aligned
    assert lib.ci8_channel_gemv(one, one, one, one, 17, 4, 32, null) == 1      # m > 16
    assert lib.ci8_channel_gemv(one, one, one, one, 1, 4, 24, null) == 1       # k % 16
    assert lib.ci8_cutlass_channel_mm(one, one, one, one, null, one, 1, 4, 32, null) == 1
    assert lib.ci8_grouped_channel_mm(one, one, one, one, one, 4, 4, 0, null) == 1
    assert lib.ci8_decode_mm_split(one, one, one, one, null, one, 65, 4, 32, 1, 0, null) == 1     # m > 64
    assert lib.ci8_decode_mm_split(one, one, one, one, null, one, 17, 4, 512, 4, 0, null) == 1    # split 4 above 16 rows
    assert lib.ci8_q8_block_mm(one, one, one, one, one, one, 1, 4, 48, null) == 1           # k % 32
    assert lib.ci8_q8_block_mm(one, one, one, one, one, null, 1, 4, 32, null) == 1          # null output


def test_operator_surface_matches_the_reference(ops):
    for name, schema in SCHEMAS.items():
        handle = getattr(ops, name)
        assert handle is getattr(torch.ops.consumer_int8, name)
        assert str(handle.default._schema) == schema
    assert ops.quantize_grouped_rows is ops.quantize_grouped4096     # README name
    assert "grouped_channel_mm" in str(ops.grouped_channel_mm.default._schema)


def test_no_cpu_fallback(ops):
    x = torch.zeros(2, 32, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        ops.quantize_rows(x, torch.zeros(2, 32, dtype=torch.int8), torch.zeros(2))
    with pytest.raises((NotImplementedError, RuntimeError)):
        ops.fused_channel_mm(torch.zeros(2, 32, dtype=torch.int8), torch.zeros(4, 32, dtype=torch.int8),
                             torch.ones(2), torch.ones(4, dtype=torch.bfloat16),
                             torch.zeros(2, 4, dtype=torch.bfloat16))


def test_fake_kernels_trace_without_a_device(ops):
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        x = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")
        codes = torch.empty(4, 64, dtype=torch.int8, device="cuda")
        scales = torch.empty(4, device="cuda")
        assert ops.quantize_rows(x, codes, scales) is None
        w = torch.empty(8, 64, dtype=torch.int8, device="cuda")
        sw = torch.empty(8, dtype=torch.bfloat16, device="cuda")
        out = torch.empty(4, 8, dtype=torch.bfloat16, device="cuda")
        assert ops.fused_channel_mm(codes, w, scales, sw, out) is None
        assert ops.channel_gemv(x, w, sw, out) is None


def test_product_code_never_touches_the_checker():
    """Nothing under the package may import, load or name the oracle."""
    package = ROOT / "consumer-int8-kernels_b200"
    for path in package.rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".cpp", ".h"}:
            text = path.read_text()
            assert "oracle" not in text.lower(), path

"""Regenerates the golden fixtures in this directory. Run once, in a checkout where the
reference project is available; the fixtures (small JSON files) are committed, this script is
how they were made, and nothing at test time reads the reference tree.

  python tests/golden/make_golden.py /path/to/reference

weight_encoding.json   outputs of the reference's own, importable, pure-torch
                       ``consumer_int8.quantization.quantize_channel`` /
                       ``dequantize_channel`` (src/consumer_int8/quantization.py:22-51) on
                       seeded inputs, plus the known-answer vector of
                       tests/test_quantization.py:16-24.
activation_kat.json    the closed-form known answers the reference's GPU tests assert for the
                       activation quantizer (tests/test_cuda_ops.py:493-509): integer-valued
                       rows with scale exactly 1, the x.5 ties that must round to even, the
                       all-zero row with scale 1e-20.
linear_kat.json        small seeded cases of the integer product and the epilogue, evaluated
                       with the literal expressions of tests/test_cuda_ops.py:488-489,596-599
                       (``a.int() @ w.int().T``; ``(acc.float()*sa[:,None]*sw.float()[None,:])
                       .bfloat16()``) and of tests/test_gemv.py:26-29.
"""
import hashlib
import importlib.util
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def load_reference_quantization(root: Path):
    spec = importlib.util.spec_from_file_location(
        "reference_quantization", root / "src" / "consumer_int8" / "quantization.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def weight_encoding(root: Path) -> dict:
    q = load_reference_quantization(root)
    cases = []
    kat = torch.tensor([[0.0, -127.0, 63.5, 127.0], [0.0, 0.0, 0.0, 0.0]])
    codes, scale = q.quantize_channel(kat)
    cases.append(dict(name="kat", weight=kat.tolist(), codes=codes.tolist(),
                      scale_bits=scale.view(torch.int16).tolist()))
    for seed, (n, k) in enumerate([(7, 32), (16, 72), (33, 128), (64, 544)]):
        g = torch.Generator().manual_seed(100 + seed)
        weight = torch.randn(n, k, generator=g) * (10.0 ** torch.randint(-3, 3, (n, 1), generator=g).float())
        weight[0] = 0
        codes, scale = q.quantize_channel(weight)
        restored = q.dequantize_channel(codes, scale)
        g_codes, g_scale = q.quantize_group32(weight)
        cases.append(dict(name=f"seed{100 + seed}", seed=100 + seed, n=n, k=k, codes_sha256=sha(codes),
                          scale_sha256=sha(scale), dequantized_sha256=sha(restored),
                          first_row_codes=codes[1, :16].tolist(),
                          first_scales_bits=scale.view(torch.int16)[:8].tolist(),
                          group32_codes_sha256=sha(g_codes), group32_scale_sha256=sha(g_scale),
                          group32_dequantized_sha256=sha(q.dequantize_group32(g_codes, g_scale))))
    return dict(source="reference src/consumer_int8/quantization.py (imported)", cases=cases)


def activation_kat() -> dict:
    rows = [
        dict(name="reference_row", x=[0.0, -127.0, 63.5, 127.0], codes=[0, -127, 64, 127], scale=1.0),
        dict(name="ties_to_even", x=[127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 62.5, 63.5, -63.5, 126.5, -126.5],
             codes=[127, 0, 2, 2, 0, -2, -2, 62, 64, -64, 126, -126], scale=1.0),
        dict(name="zero_row", x=[0.0] * 8, codes=[0] * 8, scale=1e-20),
        dict(name="first_column_minus_127", x=[-127.0, 3.0, -4.0, 100.0], codes=[-127, 3, -4, 100], scale=1.0),
    ]
    # a seeded integer-valued matrix as in tests/test_cuda_ops.py:497-509 (scale == 1, codes == round(x))
    g = torch.Generator().manual_seed(742)
    x = (torch.randn(4, 64, generator=g).bfloat16() * 100).clamp(-127, 127)
    x[:, 0] = -127
    expected = x.float().round().to(torch.int8)
    rows.append(dict(name="seeded_integer_valued", seed=742, x_bits=x.view(torch.int16).tolist(),
                     codes=expected.tolist(), scale=1.0))
    return dict(source="reference tests/test_cuda_ops.py:493-509", rows=rows)


def linear_kat() -> dict:
    cases = []
    for m, n, k, biased in [(1, 64, 128, True), (4, 48, 96, True), (17, 37, 128, True),
                            (1, 128, 512, False), (17, 132, 544, False), (64, 128, 512, False)]:
        g = torch.Generator().manual_seed(17)
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=g)
        if biased:
            w = torch.randint(1, 256, (n, k), dtype=torch.uint8, generator=g)
            integer = a.int() @ (w.int() - 128).T
        else:
            w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
            integer = a.int() @ w.int().T
        sa = torch.rand(m, generator=g) / 127
        sw = (torch.rand(n, generator=g) / 127).bfloat16()
        expected = (integer.float() * sa[:, None] * sw.float()[None, :]).bfloat16()
        cases.append(dict(m=m, n=n, k=k, biased=biased, seed=17, acc_sha256=sha(integer),
                          out_sha256=sha(expected), acc_first=integer[0, :8].tolist(),
                          out_first_bits=expected.view(torch.int16)[0, :8].tolist()))
    gemv = []
    for m, n, k in [(1, 37, 528), (3, 37, 528), (8, 64, 512)]:
        g = torch.Generator().manual_seed(134)
        x = torch.randn(m, k, generator=g).bfloat16()
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
        scale = (torch.rand(n, generator=g) * 0.002).bfloat16()
        dequantized = (w.float() * scale[:, None].float()).bfloat16()
        out = torch.nn.functional.linear(x.double(), dequantized.double()).bfloat16()
        gemv.append(dict(m=m, n=n, k=k, seed=134, out_sha256=sha(out),
                         out_first_bits=out.view(torch.int16)[0, :8].tolist()))
    return dict(source="reference tests/test_cuda_ops.py:474-490,574-600; tests/test_gemv.py:26-29",
                cases=cases, gemv=gemv)


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    root = Path(sys.argv[1])
    (HERE / "weight_encoding.json").write_text(json.dumps(weight_encoding(root), indent=1) + "\n")
    (HERE / "activation_kat.json").write_text(json.dumps(activation_kat(), indent=1) + "\n")
    (HERE / "linear_kat.json").write_text(json.dumps(linear_kat(), indent=1) + "\n")


if __name__ == "__main__":
    main()

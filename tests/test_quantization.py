"""The weight encodings against the reference's outputs (tests/golden/weight_encoding.json, made
by importing the reference's own module) and its known answers (tests/test_quantization.py:16-42)."""
import hashlib
import json
from pathlib import Path

import pytest
import torch

from consumer_int8.quantization import (dequantize_channel, dequantize_group32, quantize_channel,
                                        quantize_group32, signed_codes)

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "weight_encoding.json").read_text())


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_channel_codes_match_bias_and_scale_convention():
    weight = torch.tensor([[0.0, -127.0, 63.5, 127.0], [0.0, 0.0, 0.0, 0.0]])
    codes, scale = quantize_channel(weight)
    assert codes.dtype == torch.uint8 and scale.dtype == torch.bfloat16
    assert codes.tolist() == [[128, 1, 192, 255], [128, 128, 128, 128]]
    assert scale[0] == 1
    assert signed_codes(codes).tolist() == [[0, -127, 64, 127], [0, 0, 0, 0]]
    assert torch.isfinite(dequantize_channel(codes, scale)).all()
    torch.testing.assert_close(dequantize_channel(codes, scale)[1], weight[1])


@pytest.mark.parametrize("case", [c for c in GOLDEN["cases"] if c["name"] != "kat"], ids=lambda c: c["name"])
def test_encodings_reproduce_the_reference_outputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    n, k = case["n"], case["k"]
    weight = torch.randn(n, k, generator=g) * (10.0 ** torch.randint(-3, 3, (n, 1), generator=g).float())
    weight[0] = 0
    codes, scale = quantize_channel(weight)
    assert sha(codes) == case["codes_sha256"] and sha(scale) == case["scale_sha256"]
    assert sha(dequantize_channel(codes, scale)) == case["dequantized_sha256"]
    g_codes, g_scale = quantize_group32(weight)
    assert sha(g_codes) == case["group32_codes_sha256"] and sha(g_scale) == case["group32_scale_sha256"]
    assert sha(dequantize_group32(g_codes, g_scale)) == case["group32_dequantized_sha256"]


@pytest.mark.parametrize("k", [32, 72, 128, 4304])
def test_group32_roundtrip_keeps_unaligned_tail(k):
    weight = torch.randn(7, k, generator=torch.Generator().manual_seed(4))
    weight[0] = 0
    codes, scale = quantize_group32(weight)
    restored = dequantize_group32(codes, scale)
    assert codes.shape == weight.shape and scale.shape == (7, (k + 31) // 32)
    bound = scale.repeat_interleave(32, dim=1)[:, :k] / 2 + 1e-6
    assert ((restored - weight).abs() <= bound).all()


@pytest.mark.parametrize("quantize", [quantize_channel, quantize_group32])
def test_nonfinite_and_malformed_weights_are_rejected(quantize):
    with pytest.raises(ValueError, match="non-finite"):
        quantize(torch.tensor([[float("nan")]]))
    with pytest.raises(ValueError, match="nonempty floating-point"):
        quantize(torch.zeros(0, 4))
    with pytest.raises(ValueError, match="nonempty floating-point"):
        quantize(torch.zeros(2, 4, dtype=torch.int32))

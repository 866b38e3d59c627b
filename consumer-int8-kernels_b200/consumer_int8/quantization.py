"""Offline weight encodings consumed by the W8A8 linear path (CPU or GPU torch tensors).

Mirrors the reference's ``consumer_int8.quantization`` (src/consumer_int8/quantization.py:22-51):

* channel encoding — one scale per output channel: ``scale = max(absmax, FLT_MIN) / 127``,
  ``code = clamp(round(w / scale), -128, 127)`` stored as UINT8 ``code + 128`` together with the
  scale rounded to BF16 (quantize first, then round the scale). ``channel_mm`` consumes the
  UINT8 form directly; ``fused_channel_mm`` / ``channel_gemv`` take ``signed_codes`` of it.
* group-32 encoding — signed INT8 codes with one FP32 scale per 32 input channels (the last
  group may be short); all-zero groups get scale 1.

The checkpoint rewriting tool built on these (the reference's ``checkpoint.py``) is not part of
this package.
"""

from __future__ import annotations

import torch

GROUP = 32


def _as_matrix(weight: torch.Tensor) -> torch.Tensor:
    if weight.ndim != 2 or not weight.is_floating_point() or weight.numel() == 0:
        raise ValueError("Expected a nonempty floating-point weight matrix")
    value = weight.float()
    if not bool(torch.isfinite(value).all()):
        raise ValueError("Weight contains non-finite values")
    return value


def quantize_channel(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] float -> (UINT8 [N, K] holding code + 128, BF16 [N] channel scales)."""
    value = _as_matrix(weight)
    floor = torch.finfo(torch.float32).tiny
    scale = value.abs().amax(dim=1).clamp_min(floor) / 127.0
    codes = torch.round(value / scale.unsqueeze(1)).clamp_(-128, 127)
    stored = scale.to(torch.bfloat16)          # the codes were computed with the unrounded scale
    if not bool(torch.isfinite(stored).all()) or bool((stored == 0).any()):
        raise ValueError("Channel scales are not representable as nonzero BF16")
    return (codes.to(torch.int16) + 128).to(torch.uint8), stored


def signed_codes(codes: torch.Tensor) -> torch.Tensor:
    """UINT8 code + 128 -> the signed INT8 codes ``fused_channel_mm`` and ``channel_gemv`` take."""
    if codes.dtype != torch.uint8:
        raise ValueError("Expected UINT8 codes")
    return (codes.to(torch.int16) - 128).to(torch.int8)


def dequantize_channel(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (codes.float() - 128.0) * scale.float().unsqueeze(1)


def quantize_group32(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] float -> (INT8 [N, K], FP32 [N, ceil(K / 32)] group scales)."""
    value = _as_matrix(weight)
    n, k = value.shape
    padded = torch.nn.functional.pad(value, (0, -k % GROUP)).view(n, -1, GROUP)
    scale = padded.abs().amax(dim=2) / 127.0
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    codes = torch.round(padded / scale.unsqueeze(2)).clamp_(-127, 127).to(torch.int8)
    return codes.view(n, -1)[:, :k].contiguous(), scale


def dequantize_group32(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return codes.float() * scale.repeat_interleave(GROUP, dim=1)[:, : codes.shape[1]]


def interleave_gate_up(weight: torch.Tensor, scale: torch.Tensor, block: int = 128):
    """Row order for ``ops.gate_up_silu_mm``: the fused gate/up projection ``[gate(I) | up(I)]`` rows
    (the layout ``silu_mul`` reads, reference csrc/silu_quant.cu:64-88) are regrouped so that rows
    ``[2*block*t, 2*block*t + block)`` are gate channels ``[block*t, block*(t+1))`` and the next
    ``block`` rows the up channels of the same range; ``scale`` is permuted alike. No counterpart in
    the reference (it keeps the two operators separate); done once, offline, per weight matrix."""
    n = weight.shape[0]
    inner = n // 2
    assert n % 2 == 0 and inner % block == 0 and scale.shape[0] == n
    index = torch.arange(inner, device=weight.device).reshape(inner // block, 1, block)
    order = torch.cat([index, index + inner], dim=1).reshape(-1)
    return weight[order].contiguous(), scale[order].contiguous()

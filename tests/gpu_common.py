"""Helpers shared by the GPU parity tests."""
import ctypes

import torch

DEV = "cuda"


def bits(t: torch.Tensor) -> torch.Tensor:
    """Bit pattern view for exact comparisons of BF16 / FP32 tensors (NaN-safe)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t


def assert_bit_equal(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    g, w = bits(got), bits(want)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    bad = g != w
    count = int(bad.sum())
    if count:
        index = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {count}/{bad.numel()} elements differ; first at {index}: "
            f"got {got.detach().cpu()[tuple(index)].item()} want {want.detach().cpu()[tuple(index)].item()}")


def device_status(ops) -> int:
    word = ctypes.c_uint(0)
    assert ops.libci8.ci8_device_status(ctypes.byref(word)) == 0
    return word.value


def linear_case(m, n, k, seed=0, device_generator=False):
    """a INT8 [m,k], w INT8 [n,k], sa FP32 [m], sw BF16 [n] as in the reference's tests
    (tests/test_cuda_ops.py:476-484,578-581), generated on the CPU."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, generator=g)
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g)
    sa = torch.rand(m, generator=g) / 127
    sw = (torch.rand(n, generator=g) / 127).bfloat16()
    return a, w, sa, sw


def to_u8(w: torch.Tensor) -> torch.Tensor:
    return (w.to(torch.int16) + 128).to(torch.uint8)


def guarded(shape, dtype, fill):
    """An output buffer with a guard band on both sides: returns (view, check) where check()
    asserts that nothing outside the view was written."""
    numel = 1
    for s in shape:
        numel *= s
    pad = 256
    storage = torch.full((numel + 2 * pad,), fill, dtype=dtype, device=DEV)
    view = storage[pad:pad + numel].view(*shape)

    def check():
        head, tail = storage[:pad].cpu(), storage[pad + numel:].cpu()
        reference = torch.full((pad,), fill, dtype=dtype)
        assert torch.equal(bits(head), bits(reference)) and torch.equal(bits(tail), bits(reference)), \
            "a kernel wrote outside its output buffer"

    return view, check

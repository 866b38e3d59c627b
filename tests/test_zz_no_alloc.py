"""ci8_q8_block_mm_static: the block-32 (Q8_0) W8A8 product for callers that cannot allocate.

Some hosts of this library have no way to give it scratch memory: a plugin inside a serving engine
whose pool already holds the whole GPU, or code that runs while a stream is being captured. For them
the library carries the scratch itself (a fixed array in device memory) behind one extra C entry
point. These tests call that entry point through the C ABI, exactly as such a host would, and require
the output to be bit-identical to ci8_q8_block_mm with caller-owned scratch: twice in a row with
different shapes and data, so that whatever the first call left in the shared array must not leak
into the second. Sizes beyond the array are refused before anything is launched.

The file sorts last on purpose: a run that stops at the first failure has then seen every other test.
"""
import ctypes

import pytest
import torch

from gpu_common import DEV, assert_bit_equal, device_status

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=g)
    sw = (torch.randn(n, k // 32, generator=g) * 0.01).half()
    x = (torch.randn(m, k, generator=g) * 0.1).bfloat16()
    return x.to(DEV), w.to(DEV), sw.to(DEV)


def _both(lib, x, w, sw, m, n, k):
    """(y from the entry point with built-in scratch, y from the one with caller-owned scratch)."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a = torch.empty(m, k, dtype=torch.int8, device=DEV)
    sa = torch.empty(m, k // 32, device=DEV)
    want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert lib.ci8_q8_block_mm(_ptr(x), _ptr(a), _ptr(sa), _ptr(w), _ptr(sw), _ptr(want), m, n, k, stream) == 0
    before = torch.cuda.memory_allocated()
    assert lib.ci8_q8_block_mm_static(_ptr(x), _ptr(w), _ptr(sw), _ptr(got), m, n, k, stream) == 0
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    return got, want


def test_built_in_scratch_gives_the_same_bits_twice_in_a_row(ops):
    lib = ops.libci8
    # first a tall case that fills a good part of the array, then a smaller one with other data: stale
    # codes and scales of the first call sit right behind (and between) what the second one writes
    for m, n, k in [(300, 130, 1056), (17, 200, 4096), (300, 130, 1056)]:
        x, w, sw = _case(m, n, k, seed=m + k)
        got, want = _both(lib, x, w, sw, m, n, k)
        assert torch.isfinite(got.float()).all()
        assert_bit_equal(got, want, f"y {m}x{n}x{k}")
    assert device_status(ops) == 0


def test_sizes_beyond_the_built_in_scratch_are_refused(ops):
    lib = ops.libci8
    limit = lib.ci8_q8_block_static_max_values()
    assert limit == 4 << 20
    t = torch.zeros(64, dtype=torch.int8, device=DEV)
    stream = ctypes.c_void_p(0)
    k = 4096
    too_many_rows = limit // k + 1
    assert lib.ci8_q8_block_mm_static(_ptr(t), _ptr(t), _ptr(t), _ptr(t), too_many_rows, 8, k, stream) == 1
    assert lib.ci8_q8_block_mm_static(_ptr(t), _ptr(t), _ptr(t), _ptr(t), 1, 8, 48, stream) == 1      # k % 32
    assert lib.ci8_q8_block_mm_static(ctypes.c_void_p(0), _ptr(t), _ptr(t), _ptr(t), 1, 8, 32, stream) == 1
    lib.ci8_error_string.restype = ctypes.c_char_p
    assert b"invalid" in lib.ci8_error_string(1).lower()


def test_the_largest_accepted_size_runs(ops):
    lib = ops.libci8
    k = 4096
    m = lib.ci8_q8_block_static_max_values() // k          # exactly at the limit
    x, w, sw = _case(m, 64, k, seed=5)
    got, want = _both(lib, x, w, sw, m, 64, k)
    assert_bit_equal(got, want, "y at the size limit")
    assert device_status(ops) == 0

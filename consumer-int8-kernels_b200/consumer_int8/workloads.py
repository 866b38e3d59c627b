"""Seeded synthetic inputs for the W8A8 linear path.

The reference publishes no dataset for this path; its microbenchmarks draw random
tensors (benchmarks/microbench.py:175-197). These generators build the tensors on the
CPU from a seeded ``torch.Generator`` so that a host checker and the GPU kernels see
identical bits, in the shapes and value distributions of the five benchmark configs:

  0  M=8, K=4096, N=4096                      (host plumbing case)
  1  M in {1,4,8,16}, K=5120, N=34816         (decode, 0.1 % outlier channels x50)
  2  M=4096, K=5120, N=34816 and M=4096, K=17408, N=5120   (prefill)
  3  M=2048, K=8x4096, N=7168, per-group magnitudes log-uniform in [0.1, 10]
  4  M=16384, K=5120, N=34816 split by output channel over 1/2/4/8 GPUs
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class LinearInputs:
    x: torch.Tensor          # BF16 [M,K] (config 3: [M,G,4096])
    w: torch.Tensor          # INT8 [N,K] signed codes
    w_scale: torch.Tensor    # BF16 [N]

    @property
    def w_u8(self) -> torch.Tensor:
        """The checkpoint storage form: signed code + 128 as UINT8."""
        return (self.w.to(torch.int16) + 128).to(torch.uint8)


def activations(m: int, k: int, generator: torch.Generator, outliers: bool = True) -> torch.Tensor:
    """~N(0,1) BF16 activations; ``round(0.001*K)`` seeded channels are scaled by 50."""
    x = torch.randn(m, k, generator=generator)
    if outliers:
        count = round(0.001 * k)
        if count:
            channels = torch.randperm(k, generator=generator)[:count]
            x[:, channels] *= 50.0
    return x.bfloat16()


def grouped_activations(m: int, groups: int, generator: torch.Generator) -> torch.Tensor:
    """BF16 [M,G,4096]; one magnitude per group, log-uniform in [0.1, 10]."""
    magnitude = 10.0 ** (2.0 * torch.rand(groups, generator=generator) - 1.0)
    x = torch.randn(m, groups, 4096, generator=generator) * magnitude[None, :, None]
    return x.bfloat16()


def weights(n: int, k: int, generator: torch.Generator) -> tuple[torch.Tensor, torch.Tensor]:
    """Signed INT8 codes uniform in [-127,127] and BF16 channel scales uniform in [1e-3, 2e-2]."""
    w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=generator)
    w_scale = (torch.rand(n, generator=generator) * (2e-2 - 1e-3) + 1e-3).bfloat16()
    return w, w_scale


def linear_inputs(m: int, n: int, k: int, seed: int = 0, outliers: bool = True) -> LinearInputs:
    generator = torch.Generator().manual_seed(seed)
    x = activations(m, k, generator, outliers)
    w, w_scale = weights(n, k, generator)
    return LinearInputs(x, w, w_scale)


def grouped_inputs(m: int, n: int, groups: int, seed: int = 0) -> LinearInputs:
    generator = torch.Generator().manual_seed(seed)
    x = grouped_activations(m, groups, generator)
    w, w_scale = weights(n, groups * 4096, generator)
    return LinearInputs(x, w, w_scale)


CONFIGS = {
    "cfg0": dict(m=8, k=4096, n=4096, outliers=False),
    "cfg1_decode": dict(m=(1, 4, 8, 16), k=5120, n=34816),
    "cfg2_gate_up": dict(m=4096, k=5120, n=34816),
    "cfg2_down": dict(m=4096, k=17408, n=5120),
    "cfg3_grouped": dict(m=2048, groups=8, n=7168),
    "cfg4_sharded": dict(m=16384, k=5120, n=34816),
}

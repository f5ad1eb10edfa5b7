"""Weight initialisers with the reference's draws (scirust-core/src/nn/init/mod.rs:22-140):
each fills a ``[rows, cols]`` fp32 tensor element by element from a ``PcgEngine``."""
from __future__ import annotations

import math

import numpy as np
import torch

from .rng import PcgEngine


class Initializer:
    def fill(self, shape, fan_in: int, fan_out: int, rng: PcgEngine) -> torch.Tensor:
        raise NotImplementedError


class KaimingNormal(Initializer):
    def fill(self, shape, fan_in, fan_out, rng):
        std = float(np.sqrt(np.float32(2.0) / np.float32(fan_in)))
        return rng.fill_normal(shape, 0.0, std)


class XavierUniform(Initializer):
    def fill(self, shape, fan_in, fan_out, rng):
        bound = float(np.sqrt(np.float32(6.0) / np.float32(fan_in + fan_out)))
        return rng.fill_uniform_signed(shape, bound)


class Zeros(Initializer):
    def fill(self, shape, fan_in, fan_out, rng):
        return torch.zeros(shape, dtype=torch.float32)


class SmallNormal(Initializer):
    def __init__(self, std: float):
        self.std = std

    def fill(self, shape, fan_in, fan_out, rng):
        return rng.fill_normal(shape, 0.0, self.std)


class TruncatedNormal(Initializer):
    """Inverse-CDF truncated normal on ``[mean - k*std, mean + k*std]`` (default k = 2), one
    uniform draw per element, CDF math in fp64 (nn/init/mod.rs:96-140)."""

    def __init__(self, mean: float = 0.0, std: float = 1.0, bound: float = 2.0):
        self.mean, self.std, self.bound = mean, std, bound

    def fill(self, shape, fan_in, fan_out, rng):
        k = abs(float(self.bound))
        if self.std <= 0 or k <= 0:
            return torch.full(shape, float(self.mean), dtype=torch.float32)
        a, b = self.mean - k * self.std, self.mean + k * self.std
        cdf = lambda x: 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))  # noqa: E731
        lo, hi = cdf(-k), cdf(k)
        span = 2.0 * (hi - lo)
        scale = self.std * math.sqrt(2.0)
        u = rng.fill_float(shape).double()
        # uniform in the truncated CDF interval, mapped through sqrt(2)*erfinv
        arg = (2.0 * lo - 1.0) + span * u
        arg = arg.clamp(-1.0 + 1e-15, 1.0 - 1e-15)
        x = self.mean + scale * torch.erfinv(arg)
        return x.clamp(a, b).float()

"""Low-precision codecs (scirust-core/src/lowprec.rs:36-377, stochastic_round.rs, amp.rs:44-194):
bf16 / f16 / fp8 (E4M3, E5M2) conversion with round-to-nearest-even or stochastic rounding driven by
the counter-based Philox stream, an exact bf16 GEMM (bf16 products are exact in fp32; fp32
accumulation in ascending k), and the dynamic loss scaler used by AMP training."""
from __future__ import annotations

import numpy as np
import torch

from ..nn.rng import Philox4x32


def f32_to_bf16_bits(x) -> np.ndarray:
    """RNE truncation of fp32 to the upper 16 bits (NaN kept quiet)."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    rounded = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return np.where(nan, (b >> 16) | 0x40, rounded).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_bf16(x) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def to_f16(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def to_fp8(x, fmt: str = "e4m3") -> torch.Tensor:
    dt = torch.float8_e4m3fn if fmt.lower() == "e4m3" else torch.float8_e5m2
    return torch.as_tensor(x, dtype=torch.float32).to(dt).float()


def stochastic_round_bf16(x, seed: int = 0, stream: int = 0, start: int = 0) -> np.ndarray:
    """Round up with probability equal to the discarded fraction; the uniform for element i is
    Philox(seed, stream, start + i), so the result is independent of chunking and thread count."""
    xf = np.asarray(x, dtype=np.float32)
    bits = xf.view(np.uint32).reshape(-1).astype(np.uint64)
    rng = Philox4x32(seed)
    r = np.array([rng.u32_at(stream, start + i) & 0xFFFF for i in range(bits.size)], dtype=np.uint64)
    out = ((bits + r) >> 16).astype(np.uint16)
    special = (bits & 0x7F800000) == 0x7F800000
    out = np.where(special, (bits >> 16).astype(np.uint16), out)
    return bf16_bits_to_f32(out).reshape(xf.shape)


def gemm_bf16_exact(a, b) -> np.ndarray:
    """Inputs rounded to bf16, products exact in fp32, sequential fp32 accumulation in ascending k."""
    a = to_bf16(a)
    b = to_bf16(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.zeros((m, n), dtype=np.float32)
    for l in range(k):
        c = (c + np.outer(a[:, l], b[l, :]).astype(np.float32)).astype(np.float32)
    return c


class DynamicLossScaler:
    """Scale the loss by ``scale``; on overflow halve it and skip the step, after ``growth_interval``
    clean steps double it (amp.rs:44-194; autodiff/mixed_precision.rs:7-90)."""

    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff: float = 0.5,
                 growth_interval: int = 2000, min_scale: float = 1.0):
        self.scale, self.growth_factor, self.backoff = init_scale, growth_factor, backoff
        self.growth_interval, self.min_scale, self._good = growth_interval, min_scale, 0

    def unscale_and_check(self, grads) -> bool:
        finite = True
        for g in grads:
            if g is None:
                continue
            g.div_(self.scale)
            if not bool(torch.isfinite(g).all()):
                finite = False
        return finite

    def update(self, found_overflow: bool) -> bool:
        """Returns True when the optimizer step should run."""
        if found_overflow:
            self.scale = max(self.min_scale, self.scale * self.backoff)
            self._good = 0
            return False
        self._good += 1
        if self._good >= self.growth_interval:
            self.scale *= self.growth_factor
            self._good = 0
        return True

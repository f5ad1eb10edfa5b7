"""Run-time value contracts on a module's input and output. NOT a proof: the wrapper inspects the values and returns
a scrubbed tensor in which everything outside ``[lo, hi]`` (infinities included) is clamped to the nearest bound and
NaN becomes a fixed in-range value (0 when the interval contains it, else the bound nearest to 0). Provable bounds
are in ``scirust_b200.certify`` / ``scirust_b200.verify`` (intervals, zonotopes, DeepPoly), ``nn.lipschitz`` and
``nn.smoothing``. The check is one fused elementwise pass on whatever device the tensor is on, and ``violations``
counts how often it fired. Reference counterpart: scirust-core/src/nn/certified.rs:18-140 (``Contract``,
``ValueBoundedContract<MIN, MAX>`` with integer bounds, ``CertifiedModule``).
"""
from __future__ import annotations

import torch


class ValueBoundedContract:
    def __init__(self, lo: float, hi: float):
        if lo > hi:
            raise ValueError("ValueBoundedContract: contract bounds must satisfy MIN <= MAX")
        self.lo, self.hi = float(lo), float(hi)
        self.nan_value = 0.0 if lo <= 0.0 <= hi else (self.lo if lo > 0.0 else self.hi)

    def validate(self, t: torch.Tensor):
        """The scrubbed tensor if ``t`` broke the contract, else None."""
        bad = torch.isnan(t) | (t < self.lo) | (t > self.hi)
        if not bool(bad.any()):
            return None
        return torch.nan_to_num(t, nan=self.nan_value, posinf=self.hi, neginf=self.lo).clamp(self.lo, self.hi)


class CertifiedModule(torch.nn.Module):
    def __init__(self, inner, contract: ValueBoundedContract):
        super().__init__()
        self.inner, self.contract = inner, contract
        self.violations = 0

    def _scrub(self, t):
        fixed = self.contract.validate(t)
        if fixed is None:
            return t
        self.violations += 1
        return fixed

    def forward(self, x, *a, **kw):
        return self._scrub(self.inner(self._scrub(x), *a, **kw))

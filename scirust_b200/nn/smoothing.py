"""Certified L2 robustness by randomised smoothing (Cohen, Rosenfeld & Kolter, 2019).

The smoothed classifier ``g(x) = argmax_c P(f(x + eps) = c)``, ``eps ~ N(0, sigma^2 I)``, is constant on the
ball ``||delta||_2 <= sigma * probit(p_A)`` when the top class has probability ``p_A > 1/2``. ``p_A`` is
estimated by Monte-Carlo and replaced by its one-sided Clopper-Pearson lower bound, so the radius holds with
probability at least ``1 - alpha`` over the sampling. ``certify_cohen`` uses separate selection and estimation
samples (the procedure of the paper); ``certify`` reuses one set.

The base classifier receives ALL noisy copies at once as an ``[n, d]`` tensor and returns ``n`` class indices:
on a GPU the Monte-Carlo loop is one batched forward instead of ``n`` launches. The Gaussian draws come from the
seeded PCG stream in sample-major order, so a seed reproduces the same votes as a one-sample-at-a-time loop.
Reference counterpart: scirust-core/src/nn/smoothing.rs:151-545.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..numerics.special import clopper_pearson_lower, inv_normal_cdf  # noqa: F401
from .rng import PcgEngine


@dataclass
class Certificate:
    cls: int
    radius: float
    p_a_lower: float
    abstained: bool


def _per_sample(f):
    """Adapt a one-vector classifier ``f(x[d]) -> int`` to the batched calling convention."""
    return lambda X: torch.tensor([int(f(row)) for row in X], dtype=torch.int64)


class SmoothedClassifier:
    def __init__(self, sigma: float):
        if not (sigma == sigma) or sigma in (float("inf"), float("-inf")) or sigma <= 0.0:
            raise ValueError("randomized smoothing sigma must be finite and > 0")
        self.sigma = float(sigma)

    @staticmethod
    def _check_alpha(alpha):
        if not (0.0 < alpha < 1.0):
            raise ValueError("randomized smoothing alpha must be finite and in (0, 1)")

    def vote_counts(self, f, x, n: int, num_classes: int, rng: PcgEngine, batched: bool = True) -> torch.Tensor:
        if n == 0:
            raise ValueError("randomized smoothing requires at least one Monte-Carlo sample")
        if num_classes == 0:
            raise ValueError("randomized smoothing requires at least one class")
        x = torch.as_tensor(x, dtype=torch.float32).reshape(-1)
        if not bool(torch.isfinite(x).all()):
            raise ValueError("randomized smoothing input must contain only finite values")
        noise = rng.fill_normal((n, x.numel()), 0.0, self.sigma)
        noisy = x.cpu()[None, :] + noise
        cls = (f if batched else _per_sample(f))(noisy.to(x.device))
        cls = torch.as_tensor(cls, dtype=torch.int64).reshape(-1).cpu()
        if cls.numel() != n:
            raise ValueError(f"base classifier returned {cls.numel()} classes for {n} samples")
        if int(cls.max()) >= num_classes or int(cls.min()) < 0:
            raise ValueError(f"base classifier returned class {int(cls.max())}, but num_classes is {num_classes}")
        return torch.bincount(cls, minlength=num_classes)

    def predict(self, f, x, n, num_classes, rng, batched=True) -> int:
        return int(torch.argmax(self.vote_counts(f, x, n, num_classes, rng, batched)))   # first maximum

    def _certificate(self, cls: int, k: int, n: int, alpha: float) -> Certificate:
        p_lo = clopper_pearson_lower(k, n, alpha)
        if p_lo <= 0.5:
            return Certificate(cls, 0.0, float(p_lo), True)
        return Certificate(cls, float(self.sigma * inv_normal_cdf(p_lo)), float(p_lo), False)

    def certify(self, f, x, n, num_classes, alpha, rng, batched=True) -> Certificate:
        self._check_alpha(alpha)
        if num_classes < 2:
            raise ValueError("randomized-smoothing certification requires at least two classes")
        counts = self.vote_counts(f, x, n, num_classes, rng, batched)
        cls = int(torch.argmax(counts))
        return self._certificate(cls, int(counts[cls]), n, alpha)

    def certify_cohen(self, f, x, n0, n, num_classes, alpha, rng, batched=True) -> Certificate:
        """Selection from ``n0`` samples, then the bound from ``n`` fresh ones."""
        self._check_alpha(alpha)
        if n0 == 0:
            raise ValueError("Cohen randomized smoothing requires at least one selection sample")
        if num_classes < 2:
            raise ValueError("Cohen randomized-smoothing certification requires at least two classes")
        cls = int(torch.argmax(self.vote_counts(f, x, n0, num_classes, rng, batched)))
        est = self.vote_counts(f, x, n, num_classes, rng, batched)
        return self._certificate(cls, int(est[cls]), n, alpha)

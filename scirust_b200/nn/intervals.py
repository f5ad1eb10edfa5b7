"""Parametric prediction intervals from calibration residuals: the large-sample Gaussian interval
``y_hat +- probit((1+c)/2) * sigma`` and the small-sample Student-t interval with ``nu = n`` degrees of
freedom (wider for few residuals, converging to the Gaussian one). ``sigma`` is the residuals' RMS (zero-mean
assumption). Reference counterpart: scirust-core/src/nn/intervals.rs:27-160; the distribution-free
alternative is ``scirust_b200.conformal``.
"""
from __future__ import annotations

import numpy as np

from ..numerics.special import inv_normal_cdf, normal_cdf, student_t_cdf, student_t_ppf  # noqa: F401


def _rms(residuals) -> float:
    r = np.asarray(residuals, dtype=np.float32).reshape(-1)
    if r.size == 0:
        return 0.0
    acc = np.float32(0.0)
    for v in r:
        acc += v * v
    return float(np.sqrt(acc / np.float32(r.size)))


class GaussianInterval:
    def __init__(self, sigma: float):
        self.sigma = float(sigma)

    @staticmethod
    def from_residuals(residuals) -> "GaussianInterval":
        return GaussianInterval(_rms(residuals))

    def half_width(self, confidence: float) -> float:
        return float(np.float32(inv_normal_cdf(0.5 * (1.0 + confidence)) * self.sigma))

    def interval(self, y_hat: float, confidence: float):
        h = self.half_width(confidence)
        return y_hat - h, y_hat + h


class StudentTInterval:
    def __init__(self, sigma: float, dof: float):
        self.sigma, self.dof = float(sigma), float(dof)

    @staticmethod
    def from_residuals(residuals) -> "StudentTInterval":
        n = int(np.asarray(residuals).size)
        return StudentTInterval(_rms(residuals), max(n, 1))

    def half_width(self, confidence: float) -> float:
        return float(np.float32(student_t_ppf(0.5 * (1.0 + confidence), self.dof) * self.sigma))

    def interval(self, y_hat: float, confidence: float):
        h = self.half_width(confidence)
        return y_hat - h, y_hat + h


def coverage(intervals, truths) -> float:
    """Fraction of (lo, hi) intervals that contain their truth."""
    hits = sum(1 for (lo, hi), y in zip(intervals, truths) if lo <= y <= hi)
    return hits / max(len(truths), 1)

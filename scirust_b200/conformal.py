"""Distribution-free uncertainty: split conformal prediction and risk control.

* ``conformal_quantile``: the ``ceil((n+1)(1-alpha))``-th smallest calibration score (``+inf`` when the set is
  too small for the level: the prediction is then "everything").
* ``ConformalRegressor`` (absolute residuals, constant half-width), ``ConformalClassifier`` (threshold rule on
  ``1 - p_true``), ``ConformalQuantileRegressor`` (CQR: signed distance outside a predicted quantile band, widths
  that vary with the input), ``AdaptivePredictionSets`` (APS, and RAPS with the ``lambda * max(0, rank - k_reg)``
  penalty), ``AdaptiveConformal`` (online ACI: ``alpha_t += gamma (alpha - err_t)``, coverage under shift).
* Risk control: ``hoeffding_ucb``, ``rcps_select`` (smallest lambda whose bound, and every bound to its right,
  is under alpha), ``hoeffding_pvalue`` and ``learn_then_test`` (Bonferroni over a grid, no monotonicity needed).

Everything is plain arithmetic on calibration scores; the score tensors may live on any device (sorting a few
thousand scores is not a GPU problem, computing the model probabilities that produce them is).
Reference counterpart: scirust-core/src/nn/conformal.rs:26-425; ``scirust_b200.certify.StatisticalGuard`` builds
its accept / abstain / reject verdict on ``ConformalClassifier``.
"""
from __future__ import annotations

import math

import numpy as np
import torch


def conformal_quantile(scores, alpha: float) -> float:
    if not 0.0 < alpha < 1.0:
        raise ValueError("alpha must be in (0,1)")
    s = torch.as_tensor(scores, dtype=torch.float32).reshape(-1)
    n = s.numel()
    if n == 0:
        return math.inf
    k = math.ceil(float(np.float32(n + 1) * (np.float32(1.0) - np.float32(alpha))))      # fp32, as calibrated sets are compared across runs
    if 1 <= k <= n:
        return float(torch.sort(s).values[k - 1])
    return math.inf


class ConformalRegressor:
    def __init__(self, q: float, alpha: float):
        self.q, self.alpha = q, alpha

    @staticmethod
    def calibrate(residuals, alpha: float) -> "ConformalRegressor":
        """``residuals`` are the calibration ``|y - y_hat|``."""
        return ConformalRegressor(conformal_quantile(residuals, alpha), alpha)

    def interval(self, y_hat):
        return y_hat - self.q, y_hat + self.q

    def half_width(self) -> float:
        return self.q

    def covers(self, y_hat: float, y_true: float) -> bool:
        return abs(y_true - y_hat) <= self.q


class ConformalClassifier:
    def __init__(self, q: float):
        self.q = q
        self.qhat = q

    @staticmethod
    def calibrate(cal_probs, cal_labels, alpha: float) -> "ConformalClassifier":
        probs = torch.as_tensor(cal_probs, dtype=torch.float32)
        labels = torch.as_tensor(cal_labels, dtype=torch.int64)
        if probs.shape[0] != labels.numel():
            raise ValueError("conformal: probs/labels length mismatch")
        scores = 1.0 - probs.gather(1, labels.reshape(-1, 1)).squeeze(1)
        return ConformalClassifier(conformal_quantile(scores, alpha))

    def predict_set(self, probs):
        p = torch.as_tensor(probs, dtype=torch.float32)
        return [int(i) for i in torch.nonzero(1.0 - p <= self.q).reshape(-1)]

    def predict_sets(self, probs) -> torch.Tensor:
        """Boolean membership matrix for a batch of probability rows."""
        return 1.0 - torch.as_tensor(probs, dtype=torch.float32) <= self.q

    def covers(self, probs, y_true: int) -> bool:
        return bool(1.0 - float(torch.as_tensor(probs, dtype=torch.float32)[y_true]) <= self.q)


class ConformalQuantileRegressor:
    def __init__(self, q: float, alpha: float):
        self.q, self.alpha = q, alpha

    @staticmethod
    def calibrate(q_lo, q_hi, y, alpha: float) -> "ConformalQuantileRegressor":
        lo, hi, yy = (torch.as_tensor(t, dtype=torch.float32).reshape(-1) for t in (q_lo, q_hi, y))
        if not lo.numel() == hi.numel() == yy.numel():
            raise ValueError("CQR: predictions/targets length mismatch")
        return ConformalQuantileRegressor(conformal_quantile(torch.maximum(lo - yy, yy - hi), alpha), alpha)

    def interval(self, q_lo_x, q_hi_x):
        return q_lo_x - self.q, q_hi_x + self.q

    def covers(self, q_lo_x, q_hi_x, y_true) -> bool:
        return q_lo_x - self.q <= y_true <= q_hi_x + self.q

    def correction(self) -> float:
        return self.q


def aps_scores(probs, k_reg: int = 0, lam: float = 0.0) -> torch.Tensor:
    """Cumulative-mass score of EVERY class of every row: classes ranked by descending probability (ties to the
    lower index), score = mass of the classes ranked at or above it + ``lam * max(0, rank - k_reg)``."""
    p = torch.as_tensor(probs, dtype=torch.float32)
    single = p.dim() == 1
    if single:
        p = p[None]
    order = torch.sort(p, dim=1, descending=True, stable=True).indices
    ranked = p.gather(1, order)
    cum = torch.cumsum(ranked, 1)
    rank = torch.arange(1, p.shape[1] + 1, dtype=torch.float32, device=p.device)
    cum = cum + lam * (rank - float(k_reg)).clamp_min(0)
    out = torch.empty_like(p).scatter_(1, order, cum)
    return out[0] if single else out


class AdaptivePredictionSets:
    def __init__(self, q: float, k_reg: int = 0, lam: float = 0.0):
        self.q, self.k_reg, self.lam = q, k_reg, lam

    @staticmethod
    def calibrate(cal_probs, cal_labels, alpha: float) -> "AdaptivePredictionSets":
        return AdaptivePredictionSets.calibrate_raps(cal_probs, cal_labels, alpha, 0, 0.0)

    @staticmethod
    def calibrate_raps(cal_probs, cal_labels, alpha: float, k_reg: int, lam: float) -> "AdaptivePredictionSets":
        labels = torch.as_tensor(cal_labels, dtype=torch.int64).reshape(-1, 1)
        s = aps_scores(cal_probs, k_reg, lam)
        if s.shape[0] != labels.shape[0]:
            raise ValueError("APS: probs/labels length mismatch")
        return AdaptivePredictionSets(conformal_quantile(s.gather(1, labels).squeeze(1), alpha), k_reg, lam)

    def predict_set(self, probs):
        s = aps_scores(probs, self.k_reg, self.lam)
        return [int(i) for i in torch.nonzero(s <= self.q).reshape(-1)]

    def covers(self, probs, y_true: int) -> bool:
        return bool(aps_scores(probs, self.k_reg, self.lam)[y_true] <= self.q)

    def threshold(self) -> float:
        return self.q


class AdaptiveConformal:
    def __init__(self, target_alpha: float, gamma: float):
        if not 0.0 < target_alpha < 1.0:
            raise ValueError("ACI: target_alpha must be in (0,1)")
        if gamma <= 0.0:
            raise ValueError("ACI: gamma must be positive")
        self.target_alpha, self.gamma, self.alpha_t = target_alpha, gamma, target_alpha

    def step(self, scores, score: float) -> bool:
        """Did the level-(1 - alpha_t) set built from ``scores`` cover ``score``? Then update alpha_t."""
        if self.alpha_t <= 0.0:
            q = math.inf
        elif self.alpha_t >= 1.0:
            q = -math.inf
        else:
            q = conformal_quantile(scores, self.alpha_t)
        covered = score <= q
        self.alpha_t = min(max(self.alpha_t + self.gamma * (self.target_alpha - (0.0 if covered else 1.0)), 0.0), 1.0)
        return covered

    def alpha(self) -> float:
        return self.alpha_t


def hoeffding_ucb(mean: float, n: int, delta: float) -> float:
    if not 0.0 < delta < 1.0:
        raise ValueError("delta must be in (0,1)")
    return math.inf if n == 0 else mean + math.sqrt(math.log(1.0 / delta) / (2.0 * n))


def rcps_select(risks, n: int, alpha: float, delta: float):
    """Index of the smallest lambda (risks listed for increasing lambda, non-increasing risk) whose upper bound
    and every bound to its right is at most ``alpha``; None if even the largest lambda fails."""
    hat = None
    for i in range(len(risks) - 1, -1, -1):
        if hoeffding_ucb(float(risks[i]), n, delta) <= alpha:
            hat = i
        else:
            break
    return hat


def hoeffding_pvalue(emp_risk: float, n: int, alpha: float) -> float:
    slack = max(alpha - emp_risk, 0.0)
    return math.exp(-2.0 * n * slack * slack)


def learn_then_test(emp_risks, n: int, alpha: float, delta: float):
    if not 0.0 < delta < 1.0:
        raise ValueError("delta must be in (0,1)")
    m = len(emp_risks)
    return [i for i in range(m) if hoeffding_pvalue(float(emp_risks[i]), n, alpha) <= delta / m]

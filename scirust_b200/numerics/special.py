"""Scalar special functions used by the statistical certificates (float64, fixed evaluation order).

``erf`` is the C library's; the regularised incomplete beta is the Lentz continued fraction with the usual
symmetry switch; ``beta_inv`` inverts it by bisection; ``inv_normal_cdf`` is Acklam's rational probit
(absolute error about 1e-9). Consumers: ``scirust_b200.nn.smoothing`` (Clopper-Pearson bound, certified
radius) and ``scirust_b200.nn.intervals`` (Student-t quantiles). Reference counterparts: the
``scirust_special`` helpers called from scirust-core/src/nn/smoothing.rs:151-222 and
scirust-core/src/nn/intervals.rs:27-79.
"""
from __future__ import annotations

import math


def normal_cdf(x: float) -> float:
    return 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))


_A = (-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02, 1.38357751867269e+02,
      -3.066479806614716e+01, 2.506628277459239e+00)
_B = (-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02, 6.680131188771972e+01,
      -1.328068155288572e+01)
_C = (-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00, -2.549732539343734e+00,
      4.374664141464968e+00, 2.938163982698783e+00)
_D = (7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00, 3.754408661907416e+00)


def _horner(coeffs, x):
    acc = 0.0
    for c in coeffs:
        acc = acc * x + c
    return acc


def inv_normal_cdf(p: float) -> float:
    """Probit: the x with normal_cdf(x) = p (Acklam's piecewise rational approximation)."""
    if p <= 0.0:
        return -math.inf
    if p >= 1.0:
        return math.inf
    p_low = 0.02425
    if p < p_low:
        q = math.sqrt(-2.0 * math.log(p))
        return _horner(_C, q) / (_horner(_D, q) * q + 1.0)
    if p <= 1.0 - p_low:
        q = p - 0.5
        r = q * q
        return _horner(_A, r) * q / (_horner(_B, r) * r + 1.0)
    q = math.sqrt(-2.0 * math.log(1.0 - p))
    return -_horner(_C, q) / (_horner(_D, q) * q + 1.0)


def _betacf(a: float, b: float, x: float) -> float:
    tiny = 1e-300
    qab, qap, qam = a + b, a + 1.0, a - 1.0
    c = 1.0
    d = 1.0 - qab * x / qap
    d = 1.0 / (d if abs(d) > tiny else tiny)
    h = d
    for m in range(1, 400):
        m2 = 2 * m
        aa = m * (b - m) * x / ((qam + m2) * (a + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        h *= d * c
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        delta = d * c
        h *= delta
        if abs(delta - 1.0) < 1e-15:
            break
    return h


def regularized_incomplete_beta(a: float, b: float, x: float) -> float:
    """I_x(a, b) for a, b > 0 and x in [0, 1]."""
    if x <= 0.0:
        return 0.0
    if x >= 1.0:
        return 1.0
    front = math.exp(math.lgamma(a + b) - math.lgamma(a) - math.lgamma(b) + a * math.log(x) + b * math.log1p(-x))
    if x < (a + 1.0) / (a + b + 2.0):
        return front * _betacf(a, b, x) / a
    return 1.0 - front * _betacf(b, a, 1.0 - x) / b


def beta_inv(p: float, a: float, b: float) -> float:
    """The x in [0, 1] with I_x(a, b) = p (bisection on the monotone CDF, 200 halvings)."""
    lo, hi = 0.0, 1.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if regularized_incomplete_beta(a, b, mid) < p:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def student_t_cdf(t: float, nu: float) -> float:
    if nu <= 0.0:
        return math.nan
    if t == 0.0:
        return 0.5
    ib = regularized_incomplete_beta(0.5 * nu, 0.5, nu / (nu + t * t))
    return 1.0 - 0.5 * ib if t > 0.0 else 0.5 * ib


def student_t_ppf(p: float, nu: float) -> float:
    p = min(max(p, 1e-12), 1.0 - 1e-12)
    if abs(p - 0.5) < 1e-15:
        return 0.0
    target = p if p > 0.5 else 1.0 - p
    lo, hi = 0.0, 1.0
    while student_t_cdf(hi, nu) < target and hi < 1e9:
        hi *= 2.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if student_t_cdf(mid, nu) < target:
            lo = mid
        else:
            hi = mid
    mag = 0.5 * (lo + hi)
    return mag if p > 0.5 else -mag


def clopper_pearson_lower(k: int, n: int, alpha: float) -> float:
    """One-sided lower confidence bound (level 1 - alpha) on a binomial proportion from k of n."""
    if not 0 <= k <= n:
        raise ValueError("clopper_pearson_lower: need 0 <= k <= n")
    if not 0.0 < alpha < 1.0:
        raise ValueError("clopper_pearson_lower: alpha must be in (0, 1)")
    if k == 0:
        return 0.0
    return beta_inv(alpha, float(k), float(n - k + 1))

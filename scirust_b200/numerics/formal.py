"""A-priori error proofs, in exact rational arithmetic, for libm-free polynomial kernels.

The kernels (``exp_kernel``, ``cos_kernel``, ``sin_kernel``) are plain float64 Horner evaluations of Taylor
polynomials on a reduced range: no library call, so the same bits on every IEEE-754 host. For each of them
``prove_*`` shows ONCE, for the whole continuous range, that the relative error stays below 2^-25, a sufficient
condition for a correctly rounded float32 result (half an ulp of the worst binade), using nothing but
``fractions.Fraction``: the proof's outcome cannot depend on the rounding of the machine that runs it.

* bounded-away-from-zero functions (exp on |r| <= ln2/2, cos on |r| <= pi/4): Lagrange remainder
  ``M R^(n+1) / (n+1)!`` plus Higham's Horner bound ``gamma_2n sum |c_i| R^i`` (``gamma_k = k u / (1 - k u)``,
  ``u = 2^-53``), divided by a lower bound of |f|;
* sin, which vanishes at the centre: the factor r is kept outside (``r (1 + z q(z))``, z = r^2), the error of the
  bracket is bounded the same way, and Jordan's inequality ``sin r / r >= 2 / pi`` turns it into a relative bound.

The constants ln 2 and pi enter through validated rational upper bounds (series with explicit tails). The argument
reduction that feeds the kernels is outside these proofs (it is tested against the host libm instead).
Method and thresholds of scirust-core/src/formal_proof.rs:1-520.
"""
from __future__ import annotations

from dataclasses import dataclass
from fractions import Fraction
from math import factorial

U = Fraction(1, 2 ** 53)
THRESHOLD = Fraction(1, 2 ** 25)
EXP_DEGREE, COS_DEGREE, SIN_DEGREE = 13, 14, 15


def gamma(k: int) -> Fraction:
    return k * U / (1 - k * U)


def ln2_upper() -> Fraction:
    """ln 2 = sum_{k>=1} 1 / (k 2^k): 60 terms, tail bounded by the geometric series 2^-60."""
    return sum(Fraction(1, k * 2 ** k) for k in range(1, 61)) + Fraction(1, 2 ** 60)


def pi_upper() -> Fraction:
    """Machin: pi = 16 atan(1/5) - 4 atan(1/239); alternating series, truncated so that each term errs upward."""
    def atan_upper(x: Fraction, terms: int) -> Fraction:       # ends on a positive term: an upper bound
        return sum(Fraction((-1) ** k, 2 * k + 1) * x ** (2 * k + 1) for k in range(terms | 1))

    def atan_lower(x: Fraction, terms: int) -> Fraction:       # ends on a negative term: a lower bound
        return sum(Fraction((-1) ** k, 2 * k + 1) * x ** (2 * k + 1) for k in range((terms | 1) + 1))
    return 16 * atan_upper(Fraction(1, 5), 25) - 4 * atan_lower(Fraction(1, 239), 9)


def _exp_upper(r: Fraction, terms: int = 30) -> Fraction:
    """e^r for 0 <= r < 1: partial sum plus the geometric tail r^n / n! / (1 - r)."""
    s = sum(r ** k / factorial(k) for k in range(terms))
    return s + r ** terms / factorial(terms) / (1 - r)


@dataclass(frozen=True)
class BoundProof:
    name: str
    range_bound: Fraction
    truncation_bound: Fraction
    rounding_bound: Fraction
    relative_bound: Fraction
    threshold: Fraction = THRESHOLD

    def holds(self) -> bool:
        return self.relative_bound < self.threshold


def prove_exp() -> BoundProof:
    R = ln2_upper() / 2
    n = EXP_DEGREE
    M = _exp_upper(R)                                   # sup of every derivative of e^r, and >= sum |c_i| R^i
    trunc = M * R ** (n + 1) / factorial(n + 1)
    rnd = gamma(2 * n) * M
    lower = 1 - R                                       # e^-R >= 1 - R
    return BoundProof(f"exp (Taylor-{n}, |r| <= ln2/2)", R, trunc, rnd, (trunc + rnd) / lower)


def prove_cos() -> BoundProof:
    R = pi_upper() / 4
    n = COS_DEGREE                                      # even polynomial up to r^14; next term r^16 / 16!
    trunc = R ** (n + 2) / factorial(n + 2)             # |derivatives| <= 1
    abs_sum = sum(R ** (2 * k) / factorial(2 * k) for k in range(n // 2 + 1))
    rnd = gamma(2 * n) * abs_sum
    lower = 1 - R * R / 2                               # cos r >= 1 - r^2 / 2
    return BoundProof(f"cos (Taylor-{n}, |r| <= pi/4)", R, trunc, rnd, (trunc + rnd) / lower)


def prove_sin() -> BoundProof:
    R = pi_upper() / 4
    n = SIN_DEGREE                                      # r (1 - z/3! + ... ) up to r^15; next term r^17 / 17!
    # bracket b(z) = sin r / r; its truncation and rounding errors, then the outer product r * b (one rounding)
    trunc = R ** (n + 1) / factorial(n + 2)             # |sin r / r - T| <= R^16 / 17!
    abs_sum = sum(R ** (2 * k) / factorial(2 * k + 1) for k in range((n + 1) // 2))
    rnd = gamma(2 * n) * abs_sum + U * abs_sum          # Horner in z, the square z = r r, the final product
    lower = 2 / pi_upper()                              # Jordan: sin r / r >= 2 / pi on |r| <= pi / 2
    return BoundProof(f"sin (r * Taylor-{n} bracket, |r| <= pi/4)", R, trunc, rnd, (trunc + rnd) / lower)


# ------------------------------------------------------------------------------------------- the kernels
_EXP_C = [1.0 / factorial(k) for k in range(EXP_DEGREE + 1)]
_COS_C = [(-1.0) ** k / factorial(2 * k) for k in range(COS_DEGREE // 2 + 1)]
_SIN_C = [(-1.0) ** k / factorial(2 * k + 1) for k in range((SIN_DEGREE + 1) // 2)]


def _horner(cs, x: float) -> float:
    acc = cs[-1]
    for c in reversed(cs[:-1]):
        acc = acc * x + c
    return acc


def exp_kernel(r: float) -> float:
    """e^r for |r| <= ln2 / 2."""
    return _horner(_EXP_C, r)


def cos_kernel(r: float) -> float:
    """cos r for |r| <= pi / 4."""
    return _horner(_COS_C, r * r)


def sin_kernel(r: float) -> float:
    """sin r for |r| <= pi / 4 (the factor r stays outside the polynomial)."""
    return r * _horner(_SIN_C, r * r)


def exp_portable(x: float) -> float:
    """e^x from the kernel: x = k ln2 + r with ln 2 split in two float64 parts, scaled by 2^k exactly."""
    import math
    if x != x:
        return x
    if x > 709.0:
        return math.inf
    if x < -745.0:
        return 0.0
    k = round(x / 0.6931471805599453)
    r = (x - k * 0.6931471803691238) - k * 1.9082149292705877e-10
    return math.ldexp(exp_kernel(r), k)

"""Certified transform pairs and certificate-driven summation (float64).

* ``CertifiedMonotone`` pairs (encode / decode) carry a machine-checkable round-trip certificate: with
  ``kappa_rt(x) = |phi(x) / (x phi'(x))|`` (the relative condition number of the decoder at ``phi(x)``),
  ``|x_hat - x| / |x| <= (kappa_rt(x) B_ENC + B_DEC) u`` with ``u = eps / 2``, and ``kappa_rt(x) u >= 1/2`` means no
  digit of ``x`` survives the round trip (``invalid_at``). ``kappa_rt_sup`` is a sound upper bound over an interval
  (end points plus a closed-form cap where the maximum is interior). Pairs: ``Log``, ``Log1p``, ``SignedLog`` (asinh),
  ``Power`` (unshifted Box-Cox; its certificate adds the ``|ln x| / 2`` ulps of the rounded exponent ``1 / lambda``),
  ``MuLaw`` (decoder through ``expm1``), ``Logit``, ``Anscombe``.
* ``select_sum`` picks the cheapest reduction (plain, fixed-tree pairwise, Neumaier) whose analytic bound
  ``K(method, n) C_sum`` meets a relative tolerance, ``C_sum = sum |x_i| / |sum x_i|`` measured with compensated /
  exact sums, and falls back to the exact Shewchuk expansion.

The budgets ``B_ENC`` / ``B_DEC`` (4 ulps each) are accuracy budgets for the host's libm, not reproducibility claims.
Interface and bounds of scirust-core/src/certified_numerics.rs:71-640.
"""
from __future__ import annotations

import math
import sys
from dataclasses import dataclass

B_ENC = 4.0
B_DEC = 4.0
UNIT = sys.float_info.epsilon / 2.0
_MAX, _MINPOS, _EPS = sys.float_info.max, sys.float_info.min, sys.float_info.epsilon


@dataclass(frozen=True)
class Interval:
    lo: float
    hi: float

    def __post_init__(self):
        if not self.lo <= self.hi:
            raise ValueError("interval needs lo <= hi")

    def contains(self, x: float) -> bool:
        return self.lo <= x <= self.hi


@dataclass(frozen=True)
class UlpBound:
    ulps: float


class CertifiedMonotone:
    def domain(self) -> Interval:
        raise NotImplementedError

    def encode(self, x: float):
        """``phi(x)``, or None outside the domain."""
        return self._phi(x) if self.domain().contains(x) else None

    def decode(self, y: float) -> float:
        raise NotImplementedError

    def kappa_rt(self, x: float) -> float:
        raise NotImplementedError

    def kappa_rt_sup(self, iv: Interval) -> float:
        return max(self.kappa_rt(iv.lo), self.kappa_rt(iv.hi), self._interior_cap)

    _interior_cap = 0.0

    def roundtrip_bound(self, iv: Interval) -> UlpBound:
        return UlpBound(self.kappa_rt_sup(iv) * B_ENC + B_DEC)

    def invalid_at(self, x: float) -> bool:
        return self.kappa_rt(x) * UNIT >= 0.5


class Log(CertifiedMonotone):
    def domain(self):
        return Interval(_MINPOS, _MAX)

    _phi = staticmethod(math.log)
    decode = staticmethod(math.exp)

    def kappa_rt(self, x):
        return abs(math.log(x))


class Log1p(CertifiedMonotone):
    _interior_cap = 1.0

    def domain(self):
        return Interval(-1.0 + _EPS, _MAX)

    _phi = staticmethod(math.log1p)
    decode = staticmethod(math.expm1)

    def kappa_rt(self, x):
        return 1.0 if x == 0.0 else abs(math.log1p(x) * (1.0 + x) / x)


class SignedLog(CertifiedMonotone):
    _interior_cap = 1.0

    def domain(self):
        return Interval(-_MAX, _MAX)

    _phi = staticmethod(math.asinh)
    decode = staticmethod(math.sinh)

    def kappa_rt(self, x):
        return 1.0 if x == 0.0 else abs(math.asinh(x) * math.hypot(1.0, x) / x)


class Power(CertifiedMonotone):
    def __init__(self, lam: float):
        if not (lam > 0.0 and math.isfinite(lam)):
            raise ValueError("Power requires lambda > 0")
        self.lam = lam

    def domain(self):
        return Interval(0.0, _MAX)

    def _phi(self, x):
        return x ** self.lam

    def decode(self, y):
        return y ** (1.0 / self.lam)

    def kappa_rt(self, x):
        return 1.0 / self.lam

    def kappa_rt_sup(self, iv):
        return 1.0 / self.lam

    def roundtrip_bound(self, iv):
        def at(x):
            return abs(math.log(x)) if x > 0.0 else 0.0
        return UlpBound(B_ENC / self.lam + B_DEC + 0.5 * max(at(iv.lo), at(iv.hi)))


class MuLaw(CertifiedMonotone):
    _interior_cap = 1.0

    def __init__(self, mu: float = 255.0):
        if not (mu > 0.0 and math.isfinite(mu)):
            raise ValueError("MuLaw requires mu > 0")
        self.mu = mu

    def domain(self):
        return Interval(-1.0, 1.0)

    def _phi(self, x):
        return math.copysign(math.log1p(self.mu * abs(x)) / math.log1p(self.mu), x)

    def decode(self, y):
        return math.copysign(math.expm1(abs(y) * math.log1p(self.mu)) / self.mu, y)

    def kappa_rt(self, x):
        t = self.mu * abs(x)
        return 1.0 if t == 0.0 else math.log1p(t) * (1.0 + t) / t


class Logit(CertifiedMonotone):
    _interior_cap = 0.2785          # max over t of t ln((1 - t) / t), the interior maximum on (1/2, 1)

    def domain(self):
        return Interval(_MINPOS, 1.0 - _EPS)

    def _phi(self, x):
        return math.log(x / (1.0 - x))

    def decode(self, y):
        return 1.0 / (1.0 + math.exp(-y))

    def kappa_rt(self, x):
        return abs(math.log(x / (1.0 - x)) * (1.0 - x))


class Anscombe(CertifiedMonotone):
    def domain(self):
        return Interval(0.0, _MAX)

    def _phi(self, x):
        return 2.0 * math.sqrt(x + 0.375)

    def decode(self, y):
        return (y * 0.5) ** 2 - 0.375

    def kappa_rt(self, x):
        return math.inf if x == 0.0 else 2.0 + 0.75 / x

    def kappa_rt_sup(self, iv):
        return self.kappa_rt(iv.lo)          # strictly decreasing


# ------------------------------------------------------------------------------------------- summation
def sum_neumaier(xs) -> float:
    s = c = 0.0
    for x in xs:
        t = s + x
        c += (s - t) + x if abs(s) >= abs(x) else (x - t) + s
        s = t
    return s + c


def sum_klein(xs) -> float:
    s = cs = ccs = 0.0
    for x in xs:
        t = s + x
        c = (s - t) + x if abs(s) >= abs(x) else (x - t) + s
        s = t
        t2 = cs + c
        cc = (cs - t2) + c if abs(cs) >= abs(c) else (c - t2) + cs
        cs = t2
        ccs += cc
    return s + cs + ccs


def sum_pairwise(xs) -> float:
    n = len(xs)
    if n <= 8:
        s = 0.0
        for x in xs:
            s += x
        return s
    return sum_pairwise(xs[: n // 2]) + sum_pairwise(xs[n // 2:])


def sum_expansion(xs) -> float:
    """Shewchuk's non-overlapping expansion: exact for any order, rounded once at the end (within one ulp)."""
    partials: list = []
    for x in xs:
        i = 0
        for y in partials:
            if abs(x) < abs(y):
                x, y = y, x
            hi = x + y
            lo = y - (hi - x)
            if lo != 0.0:
                partials[i] = lo
                i += 1
            x = hi
        del partials[i:]
        partials.append(x)
    s = 0.0
    for p in partials:
        s += p
    return s


def sum_condition(xs) -> float:
    denom = abs(sum_expansion(xs))
    return math.inf if denom == 0.0 else sum_neumaier([abs(x) for x in xs]) / denom


@dataclass(frozen=True)
class SumSelection:
    method: str               # "naive" | "pairwise" | "neumaier" | "expansion"
    value: float
    cert_rel_bound: float
    condition: float


def select_sum(xs, tau: float) -> SumSelection:
    xs = list(xs)
    n = float(max(len(xs), 2))
    cond = sum_condition(xs)
    for method, coeff in (("naive", (n - 1.0) * UNIT), ("pairwise", math.ceil(math.log2(n)) * UNIT * 1.05),
                          ("neumaier", 2.0 * UNIT + n * n * UNIT * UNIT)):
        bound = coeff * cond
        if bound <= tau:
            value = {"naive": lambda: math.fsum([]) + _naive(xs), "pairwise": lambda: sum_pairwise(xs),
                     "neumaier": lambda: sum_neumaier(xs)}[method]()
            return SumSelection(method, value, bound, cond)
    return SumSelection("expansion", sum_expansion(xs), UNIT, cond)


def _naive(xs) -> float:
    s = 0.0
    for x in xs:
        s += x
    return s

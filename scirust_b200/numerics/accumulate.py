"""fp32 accumulation strategies and their autotuner: naive left-to-right, pairwise (leaves of 8), Neumaier
(compensated), Klein (second-order compensated) and an unbiased stochastic-rounding sum keyed by a counter-based
generator (bitwise reproducible for a given seed, stream and input order). ``autotune_accumulator`` picks the most
accurate method on a DEVELOPMENT batch (relative error against the exact sum, which the exact accumulator provides)
and re-scores the winner on a HELD-OUT batch against the naive baseline; ``beats_baseline`` False means: fall back to
the naive sum. ``autotune_by`` is the generic dev / held-out harness behind it.
Reference counterparts: scirust-core/src/autotune_accumulate.rs:27-200, stochastic_round.rs:60-166,
transform_autotune.rs:159-222 (``GenericAutotune``, ``autotune_by``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from ..nn.rng import Philox4x32
from .reproducible import ExactAccumulator

f32 = np.float32


@dataclass(frozen=True)
class AccumMethod:
    kind: str                     # naive | pairwise | neumaier | klein | stochastic
    seed: int = 0
    stream: int = 0

    def cost(self) -> int:
        """Relative floating-point work per element."""
        return {"naive": 1, "pairwise": 1, "stochastic": 3, "neumaier": 7, "klein": 14}[self.kind]


NAIVE, PAIRWISE, NEUMAIER, KLEIN = (AccumMethod(k) for k in ("naive", "pairwise", "neumaier", "klein"))


def default_accumulators():
    return [NAIVE, PAIRWISE, NEUMAIER, KLEIN, AccumMethod("stochastic", 0x5CA1AB1E, 0)]


def _naive(xs):
    s = f32(0.0)
    for x in xs:
        s = f32(s + x)
    return s


def _pairwise(xs):
    if len(xs) <= 8:
        return _naive(xs)
    mid = len(xs) // 2
    return f32(_pairwise(xs[:mid]) + _pairwise(xs[mid:]))


def _two_sum_err(s, x, t):
    return f32(f32(s - t) + x) if abs(s) >= abs(x) else f32(f32(x - t) + s)


def _neumaier(xs):
    s = c = f32(0.0)
    for x in xs:
        t = f32(s + x)
        c = f32(c + _two_sum_err(s, x, t))
        s = t
    return f32(s + c)


def _klein(xs):
    s = cs = ccs = f32(0.0)
    for x in xs:
        t = f32(s + x)
        c = _two_sum_err(s, x, t)
        s = t
        t2 = f32(cs + c)
        cc = _two_sum_err(cs, c, t2)
        cs = t2
        ccs = f32(ccs + cc)
    return f32(f32(s + cs) + ccs)


def stochastic_round_to_f32(x: float, u: float) -> np.float32:
    """Round the float64 ``x`` to one of its two fp32 neighbours: up with probability (x - lo) / (hi - lo)."""
    if not math.isfinite(x):
        return f32(x)
    fmax = float(np.finfo(np.float32).max)
    if x >= fmax:
        return f32(fmax)
    if x <= -fmax:
        return f32(-fmax)
    r = f32(x)
    lo = r if float(r) <= x else np.nextafter(r, f32(-np.inf))
    if float(lo) == x:
        return lo
    hi = np.nextafter(lo, f32(np.inf))
    p_up = (x - float(lo)) / (float(hi) - float(lo))
    return hi if float(u) < p_up else lo


def stochastic_sum_f32(xs, seed: int, stream: int = 0) -> np.float32:
    rng = Philox4x32(seed)
    acc = f32(0.0)
    for i, x in enumerate(xs):
        acc = stochastic_round_to_f32(float(acc) + float(x), rng.f32_at(stream, i))
    return acc


def accumulate(method: AccumMethod, xs) -> np.float32:
    xs = np.asarray(xs, dtype=np.float32).reshape(-1)
    with np.errstate(over="ignore", invalid="ignore"):
        if method.kind == "stochastic":
            return stochastic_sum_f32(xs, method.seed, method.stream)
        return {"naive": _naive, "pairwise": _pairwise, "neumaier": _neumaier, "klein": _klein}[method.kind](xs)


def exact_sum(xs) -> float:
    acc = ExactAccumulator()
    for x in np.asarray(xs, dtype=np.float32).reshape(-1):
        acc.add(float(x))
    return acc.round_f64()


def accum_score(method: AccumMethod, xs):
    """``-|relative error|`` against the exact sum (0 is exact); None when the exact sum is 0."""
    exact = exact_sum(xs)
    if exact == 0.0:
        return None
    return -abs((float(accumulate(method, xs)) - exact) / exact)


@dataclass
class GenericAutotune:
    chosen: object
    chosen_eval_score: float
    baseline_eval_score: float
    beats_baseline: bool
    dev_scores: list


def autotune_by(dev, held_out, candidates, score, baseline) -> GenericAutotune:
    """``score(candidate, fit_set, score_set) -> float | None`` (higher is better); ``baseline(fit_set, score_set)``.
    Selection on ``dev`` (first best wins ties), validation of the winner on ``held_out``."""
    dev_scores, best = [], None
    for c in candidates:
        s = score(c, dev, dev)
        if s is not None and (best is None or s > best[1]):
            best = (c, s)
        dev_scores.append((c, s))
    base = baseline(dev, held_out)
    if best is None:
        return GenericAutotune(None, -math.inf, base, False, dev_scores)
    ev = score(best[0], dev, held_out)
    ev = -math.inf if ev is None else ev
    return GenericAutotune(best[0], ev, base, ev > base, dev_scores)


def autotune_accumulator(dev, held_out, candidates=None) -> GenericAutotune:
    def base(_fit, scr):
        s = accum_score(NAIVE, scr)
        return -math.inf if s is None else s
    return autotune_by(dev, held_out, candidates or default_accumulators(), lambda m, _fit, scr: accum_score(m, scr), base)

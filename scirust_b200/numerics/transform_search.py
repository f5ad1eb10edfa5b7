"""Selecting a numerical REPRESENTATION for a data set.

* ``select_transform`` (the certificate gate): among a declared dictionary of certified monotone transform pairs, accept
  a candidate iff every sample lies in its domain, the support stays clear of the invalid region (``kappa_rt * u >=
  1/2``: no digit survives the round trip) and the certified round-trip bound ``kappa_rt_sup * B_ENC + B_DEC`` fits the
  tolerance in ulps. The cheapest accepted candidate wins (ties: the tighter certificate); every rejection carries its
  reason. Nothing is measured: the answer is a certificate.
* ``autotune_quantizer`` (the empirical stage): encode, quantise with an L-level uniform quantiser whose range is FITTED
  on the development set, decode; the score is the SQNR in dB. The development winner is re-scored on held-out data
  against direct (no transform) quantisation; ``beats_baseline`` False means: do not transform.
* ``joint_search`` / ``sequential_baseline``: the pipeline "encode, quantise (64 levels), decode, narrow to fp32,
  accumulate" scored by the held-out relative error of the accumulated total against the exact sum of the originals.
  The joint search tries every (representation, accumulation) pair; the sequential baseline picks the representation
  by certificate first, then the accumulation. ``PlanCache`` stores winners keyed by a coarse DISTRIBUTION summary
  (sign, decades of dynamic range, log-scale skew bucket) so that a similar data set reuses the plan.

Reference counterparts: scirust-core/src/transform_search.rs:43-290, transform_autotune.rs:40-310,
representation_graph.rs:96-800 (the prototype's dictionary, pipeline objective, both searches and the plan cache).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from . import accumulate as A
from .certified import (B_DEC, B_ENC, UNIT, Anscombe, CertifiedMonotone, Interval, Log, Log1p, Logit, MuLaw, Power,
                        SignedLog)


@dataclass(frozen=True)
class Representation:
    kind: str                       # log | log1p | signed-log | power | mu-law | logit | anscombe | identity
    param: float = 0.0

    def transform(self) -> CertifiedMonotone | None:
        return {"log": Log, "log1p": Log1p, "signed-log": SignedLog, "logit": Logit, "anscombe": Anscombe,
                "power": lambda: Power(self.param), "mu-law": lambda: MuLaw(self.param), "identity": lambda: None}[self.kind]()

    @property
    def name(self) -> str:
        return self.kind if self.kind not in ("power", "mu-law") else f"{self.kind}({self.param:g})"

    def cost(self) -> int:
        return {"identity": 0, "anscombe": 2, "log": 3, "log1p": 3, "power": 3, "logit": 4, "signed-log": 4, "mu-law": 5}[self.kind]

    def encode(self, x: float):
        t = self.transform()
        return x if t is None else t.encode(x)

    def decode(self, y: float) -> float:
        t = self.transform()
        return y if t is None else t.decode(y)


LOG, LOG1P, SIGNED_LOG, LOGIT, ANSCOMBE, IDENTITY = (Representation(k) for k in
                                                     ("log", "log1p", "signed-log", "logit", "anscombe", "identity"))


def default_positive_dictionary():
    return [LOG, LOG1P, Representation("power", 0.5), SIGNED_LOG, ANSCOMBE]


def power_lambda_grid(lambdas):
    return [Representation("power", float(l)) for l in lambdas]


def default_positive_quantizer_dictionary():
    return [LOG, LOG1P, ANSCOMBE] + power_lambda_grid([0.1, 0.2, 0.3, 0.5, 0.7, 1.0])


@dataclass(frozen=True)
class RejectReason:
    kind: str                       # outside-domain | invalid-region | tolerance-exceeded
    value: float


@dataclass(frozen=True)
class CandidateVerdict:
    repr: Representation
    bound_ulps: float | None
    rejected: RejectReason | None

    @property
    def accepted(self) -> bool:
        return self.rejected is None


@dataclass
class SelectionReport:
    chosen: Representation | None
    chosen_bound_ulps: float | None
    support: Interval
    verdicts: list


def _gate(rep: Representation, samples, support: Interval):
    t = rep.transform()
    dom = t.domain()
    for s in samples:
        if not dom.contains(s):
            return None, RejectReason("outside-domain", float(s))
    ksup = t.kappa_rt_sup(support)
    if ksup * UNIT >= 0.5:
        return None, RejectReason("invalid-region", ksup)
    return ksup, None


def select_transform(samples, tau_ulps: float, dictionary) -> SelectionReport:
    xs = [float(v) for v in samples]
    if not xs:
        return SelectionReport(None, None, Interval(0.0, 0.0), [])
    support = Interval(min(xs), max(xs))
    verdicts, chosen = [], None
    for rep in dictionary:
        ksup, why = _gate(rep, xs, support)
        if why is None:
            bound = ksup * B_ENC + B_DEC
            if bound > tau_ulps:
                why = RejectReason("tolerance-exceeded", bound)
        verdicts.append(CandidateVerdict(rep, None if why else bound, why))
        if why is None and (chosen is None or rep.cost() < chosen[0].cost()
                            or (rep.cost() == chosen[0].cost() and bound < chosen[1])):
            chosen = (rep, bound)
    return SelectionReport(chosen[0] if chosen else None, chosen[1] if chosen else None, support, verdicts)


# ------------------------------------------------------------------ empirical quantiser autotune
class UniformQuantizer:
    """L cells over the fitted range; reconstruction at the cell centre."""

    def __init__(self, lo: float, step: float, levels: int):
        self.lo, self.step, self.levels = lo, step, levels

    @staticmethod
    def fit(enc, levels: int) -> "UniformQuantizer":
        e = np.asarray(enc, dtype=np.float64)
        span = max(float(e.max() - e.min()), np.finfo(np.float64).tiny)
        return UniformQuantizer(float(e.min()), span / levels, levels)

    def round_trip(self, e):
        idx = np.clip(np.floor((np.asarray(e, dtype=np.float64) - self.lo) / self.step), 0.0, self.levels - 1)
        return self.lo + (idx + 0.5) * self.step


def sqnr_db(reference, estimate) -> float:
    r, e = np.asarray(reference, dtype=np.float64), np.asarray(estimate, dtype=np.float64)
    err = float(((r - e) ** 2).sum())
    return math.inf if err == 0.0 else 10.0 * math.log10(float((r * r).sum()) / err)


def _encode_all(rep, xs):
    out = []
    for x in xs:
        e = rep.encode(float(x))
        if e is None:
            return None
        out.append(e)
    return np.asarray(out)


def quantize_reconstruct(rep: Representation, fit, data, levels: int):
    """Reconstruction of ``data`` through ``rep`` and a quantiser fitted on ``fit``; None outside the domain."""
    ef, ed = _encode_all(rep, fit), _encode_all(rep, data)
    if ef is None or ed is None:
        return None
    q = UniformQuantizer.fit(ef, levels)
    return np.asarray([rep.decode(float(v)) for v in q.round_trip(ed)])


@dataclass
class AutotuneReport:
    chosen: Representation | None
    chosen_eval_sqnr_db: float
    baseline_eval_sqnr_db: float
    beats_baseline: bool
    verdicts: list                   # (representation, dev score | RejectReason)


def autotune_quantizer(dev, held_out, dictionary, levels: int) -> AutotuneReport:
    dev, held_out = [float(v) for v in dev], [float(v) for v in held_out]
    both = dev + held_out
    support = Interval(min(both), max(both))
    gates = {rep: _gate(rep, both, support)[1] for rep in dictionary}

    def score(rep, fit, scr):
        if gates[rep] is not None:
            return None
        rec = quantize_reconstruct(rep, fit, scr, levels)
        return None if rec is None else sqnr_db(scr, rec)

    out = A.autotune_by(dev, held_out, list(dictionary), score,
                        lambda fit, scr: sqnr_db(scr, UniformQuantizer.fit(fit, levels).round_trip(scr)))
    verdicts = [(rep, gates[rep] if gates[rep] is not None else s) for rep, s in out.dev_scores]
    return AutotuneReport(out.chosen, out.chosen_eval_score, out.baseline_eval_score, out.beats_baseline, verdicts)


# ------------------------------------------------------------------ joint (representation, accumulation) plans
@dataclass(frozen=True)
class Plan:
    representation: Representation
    accumulation: A.AccumMethod

    def cost(self) -> int:
        return self.representation.cost() + self.accumulation.cost()


def default_representation_dictionary():
    return [IDENTITY, LOG, LOG1P, ANSCOMBE] + power_lambda_grid([0.25, 0.5])


def pipeline_relative_error(plan: Plan, fit, score_on, levels: int = 64):
    """|accumulated reconstruction - exact sum of the originals| / |exact sum|; None if infeasible."""
    rec = quantize_reconstruct(plan.representation, fit, score_on, levels)
    if rec is None or not np.isfinite(rec).all():
        return None
    exact = A.exact_sum(np.asarray(score_on, dtype=np.float32))
    if exact == 0.0:
        return None
    return abs((float(A.accumulate(plan.accumulation, rec.astype(np.float32))) - exact) / exact)


@dataclass
class PlanSearchReport:
    chosen: Plan | None
    held_out_error: float
    evaluated: int
    dev_errors: list = field(default_factory=list)


def joint_search(dev, held_out, representations=None, accumulators=None, levels: int = 64) -> PlanSearchReport:
    reps = representations or default_representation_dictionary()
    accs = accumulators or A.default_accumulators()
    best, errs = None, []
    for r in reps:
        for a in accs:
            p = Plan(r, a)
            e = pipeline_relative_error(p, dev, dev, levels)
            errs.append((p, e))
            if e is not None and (best is None or (e, p.cost()) < (best[1], best[0].cost())):
                best = (p, e)
    if best is None:
        return PlanSearchReport(None, math.inf, len(errs), errs)
    ho = pipeline_relative_error(best[0], dev, held_out, levels)
    return PlanSearchReport(best[0], math.inf if ho is None else ho, len(errs), errs)


def sequential_baseline(dev, held_out, tau_ulps: float = 64.0, representations=None, accumulators=None,
                        levels: int = 64) -> PlanSearchReport:
    """Representation by certificate (identity when nothing is accepted), then the best accumulation for it."""
    reps = [r for r in (representations or default_representation_dictionary()) if r.kind != "identity"]
    sel = select_transform(dev, tau_ulps, reps)
    rep = sel.chosen or IDENTITY
    best, errs = None, []
    for a in accumulators or A.default_accumulators():
        p = Plan(rep, a)
        e = pipeline_relative_error(p, dev, dev, levels)
        errs.append((p, e))
        if e is not None and (best is None or e < best[1]):
            best = (p, e)
    if best is None:
        return PlanSearchReport(None, math.inf, len(errs), errs)
    ho = pipeline_relative_error(best[0], dev, held_out, levels)
    return PlanSearchReport(best[0], math.inf if ho is None else ho, len(errs), errs)


@dataclass(frozen=True)
class DistributionSummary:
    sign: str                        # positive | negative | mixed
    decades: int                     # floor(log10(max|x| / min|x| over non-zeros))
    skew_bucket: int                 # sign and rough size of the skewness of log|x|


def summarize(xs) -> DistributionSummary:
    x = np.asarray(xs, dtype=np.float64)
    sign = "positive" if (x > 0).all() else "negative" if (x < 0).all() else "mixed"
    mag = np.abs(x[x != 0])
    if mag.size == 0:
        return DistributionSummary(sign, 0, 0)
    decades = int(math.floor(math.log10(float(mag.max() / mag.min())))) if mag.max() > mag.min() else 0
    l = np.log(mag)
    sd = float(l.std())
    skew = 0.0 if sd == 0 else float(((l - l.mean()) ** 3).mean() / sd ** 3)
    return DistributionSummary(sign, decades, int(np.clip(round(skew), -3, 3)))


class PlanCache:
    """Plans keyed by (task, hardware, distribution summary): a data set that looks like an earlier one reuses its plan."""

    def __init__(self):
        self._plans: dict = {}
        self.hits = self.misses = 0

    def get(self, task: str, hardware: str, summary: DistributionSummary):
        p = self._plans.get((task, hardware, summary))
        if p is None:
            self.misses += 1
        else:
            self.hits += 1
        return p

    def insert(self, task: str, hardware: str, summary: DistributionSummary, plan: Plan) -> None:
        self._plans[(task, hardware, summary)] = plan

    def plan_for(self, task: str, hardware: str, dev, held_out, **search) -> Plan | None:
        s = summarize(dev)
        p = self.get(task, hardware, s)
        if p is None:
            p = joint_search(dev, held_out, **search).chosen
            if p is not None:
                self.insert(task, hardware, s, p)
        return p


def current_hardware_key() -> str:
    import torch
    if torch.cuda.is_available():
        cc = torch.cuda.get_device_capability()
        return f"cuda-sm{cc[0]}{cc[1]}"
    return "cpu"

"""Held-out engineering-metric gate: decides whether a specialised (fine-tuned) model is kept. Training loss plays no
part: the candidate and its baseline are measured on EXACTLY the same frozen held-out task ids, and the update is
retained only if every absolute threshold and every improvement-over-baseline threshold is met. The gate fails closed:
a missing measurement, a duplicated or drifting task set, a probability outside [0, 1] or a side that spent more than
the evaluation budget raises instead of producing a decision.

Metrics per side: valid-patch-set rate, Brier score of the predicted compile-pass probability, first-pass gate success
rate, accepted candidates per unit of evaluation budget. The report carries the SHA-256 of the criterion's canonical
JSON so a stored decision names the exact thresholds it was taken under.
Reference counterpart: scirust-sciagent/src/engineering_specialization.rs:13-609.
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import asdict, dataclass, field

CRITERION_VERSION = 1
REPORT_VERSION = 1


class SpecializationGateError(ValueError):
    pass


def _prob(name, v):
    if not (isinstance(v, (int, float)) and math.isfinite(v) and 0.0 <= v <= 1.0):
        raise SpecializationGateError(f"{name} must be a probability in [0, 1], got {v!r}")


def _nonneg(name, v):
    if not (isinstance(v, (int, float)) and math.isfinite(v) and v >= 0.0):
        raise SpecializationGateError(f"{name} must be finite and non-negative, got {v!r}")


@dataclass(frozen=True)
class Criterion:
    max_evaluation_budget: int
    min_valid_patch_set_rate: float
    max_compile_brier_score: float
    min_first_pass_gate_success_rate: float
    min_accepted_candidate_yield_per_budget: float
    min_valid_patch_set_rate_delta: float = 0.0
    min_compile_brier_improvement: float = 0.0
    min_first_pass_gate_success_rate_delta: float = 0.0
    min_accepted_candidate_yield_per_budget_delta: float = 0.0
    version: int = CRITERION_VERSION

    def validate(self) -> None:
        if self.version != CRITERION_VERSION:
            raise SpecializationGateError(f"unsupported criterion version {self.version}")
        if not isinstance(self.max_evaluation_budget, int) or self.max_evaluation_budget <= 0:
            raise SpecializationGateError("max_evaluation_budget must be a positive integer")
        for n in ("min_valid_patch_set_rate", "max_compile_brier_score", "min_first_pass_gate_success_rate"):
            _prob(n, getattr(self, n))
        for n in ("min_accepted_candidate_yield_per_budget", "min_valid_patch_set_rate_delta", "min_compile_brier_improvement",
                  "min_first_pass_gate_success_rate_delta", "min_accepted_candidate_yield_per_budget_delta"):
            _nonneg(n, getattr(self, n))

    def sha256(self) -> str:
        self.validate()
        return hashlib.sha256(json.dumps(asdict(self), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


@dataclass(frozen=True)
class Observation:
    task_spec_id: str
    patch_set_valid: bool | None = None
    compile_pass_probability: float | None = None
    compile_passed: bool | None = None
    first_pass_gate_success: bool | None = None
    accepted_candidate: bool | None = None
    evaluation_cost: int | None = None


@dataclass(frozen=True)
class Metrics:
    tasks: int
    valid_patch_set_rate: float
    compile_brier_score: float
    first_pass_gate_success_rate: float
    accepted_candidates: int
    evaluation_budget: int
    accepted_candidate_yield_per_budget: float


@dataclass
class Report:
    criterion_sha256: str
    held_out_task_ids: list
    baseline: Metrics
    candidate: Metrics
    decision: str                                                             # "retain" | "reject"
    failed_criteria: list = field(default_factory=list)
    report_version: int = REPORT_VERSION

    def to_json(self) -> str:
        return json.dumps(asdict(self), sort_keys=True, indent=2)


def _canonical(side: str, observations) -> dict:
    out = {}
    for o in observations:
        if not o.task_spec_id or not o.task_spec_id.strip():
            raise SpecializationGateError(f"{side}: empty task id")
        if o.task_spec_id in out:
            raise SpecializationGateError(f"{side}: task {o.task_spec_id!r} is measured twice")
        for name in ("patch_set_valid", "compile_pass_probability", "compile_passed", "first_pass_gate_success",
                     "accepted_candidate", "evaluation_cost"):
            if getattr(o, name) is None:
                raise SpecializationGateError(f"{side}: task {o.task_spec_id!r} lacks {name}")
        _prob(f"{side}: compile_pass_probability of {o.task_spec_id!r}", o.compile_pass_probability)
        if not isinstance(o.evaluation_cost, int) or o.evaluation_cost < 0:
            raise SpecializationGateError(f"{side}: evaluation_cost of {o.task_spec_id!r} must be a non-negative integer")
        out[o.task_spec_id] = o
    if not out:
        raise SpecializationGateError(f"{side}: no held-out observation")
    return dict(sorted(out.items()))


def measure(by_task: dict) -> Metrics:
    obs = list(by_task.values())
    n = len(obs)
    budget = sum(o.evaluation_cost for o in obs)
    if budget <= 0:
        raise SpecializationGateError("the evaluation budget spent is zero: yield per budget is undefined")
    accepted = sum(bool(o.accepted_candidate) for o in obs)
    return Metrics(n, sum(bool(o.patch_set_valid) for o in obs) / n,
                   sum((o.compile_pass_probability - float(bool(o.compile_passed))) ** 2 for o in obs) / n,
                   sum(bool(o.first_pass_gate_success) for o in obs) / n, accepted, budget, accepted / budget)


def evaluate(criterion: Criterion, baseline, candidate) -> Report:
    criterion.validate()
    b, c = _canonical("baseline", baseline), _canonical("candidate", candidate)
    if list(b) != list(c):
        raise SpecializationGateError(f"held-out task sets differ: baseline {list(b)}, candidate {list(c)}")
    mb, mc = measure(b), measure(c)
    for side, m in (("baseline", mb), ("candidate", mc)):
        if m.evaluation_budget > criterion.max_evaluation_budget:
            raise SpecializationGateError(f"{side} spent {m.evaluation_budget} of at most {criterion.max_evaluation_budget}")
    failed = []

    def at_least(name, value, bound):
        if not value >= bound - 1e-15:
            failed.append(f"{name}: {value:.6g} < {bound:.6g}")

    at_least("valid_patch_set_rate.absolute", mc.valid_patch_set_rate, criterion.min_valid_patch_set_rate)
    at_least("valid_patch_set_rate.delta", mc.valid_patch_set_rate - mb.valid_patch_set_rate, criterion.min_valid_patch_set_rate_delta)
    if not mc.compile_brier_score <= criterion.max_compile_brier_score + 1e-15:
        failed.append(f"compile_brier_score.absolute: {mc.compile_brier_score:.6g} > {criterion.max_compile_brier_score:.6g}")
    at_least("compile_brier_score.improvement", mb.compile_brier_score - mc.compile_brier_score, criterion.min_compile_brier_improvement)
    at_least("first_pass_gate_success_rate.absolute", mc.first_pass_gate_success_rate, criterion.min_first_pass_gate_success_rate)
    at_least("first_pass_gate_success_rate.delta", mc.first_pass_gate_success_rate - mb.first_pass_gate_success_rate,
             criterion.min_first_pass_gate_success_rate_delta)
    at_least("accepted_candidate_yield_per_budget.absolute", mc.accepted_candidate_yield_per_budget,
             criterion.min_accepted_candidate_yield_per_budget)
    at_least("accepted_candidate_yield_per_budget.delta", mc.accepted_candidate_yield_per_budget - mb.accepted_candidate_yield_per_budget,
             criterion.min_accepted_candidate_yield_per_budget_delta)
    return Report(criterion.sha256(), list(b), mb, mc, "retain" if not failed else "reject", failed)

"""Held-out engineering-metric gate (CPU)."""
import dataclasses
import json

import pytest

from scirust_b200.train import specialization_gate as G


def _obs(task, valid, prob, passed, gate, accepted, cost=10):
    return G.Observation(task, valid, prob, passed, gate, accepted, cost)


CRIT = G.Criterion(max_evaluation_budget=100, min_valid_patch_set_rate=0.6, max_compile_brier_score=0.2,
                   min_first_pass_gate_success_rate=0.5, min_accepted_candidate_yield_per_budget=0.02,
                   min_valid_patch_set_rate_delta=0.1, min_compile_brier_improvement=0.01,
                   min_first_pass_gate_success_rate_delta=0.1, min_accepted_candidate_yield_per_budget_delta=0.01)
BASE = [_obs("t1", True, 0.6, True, True, True), _obs("t2", False, 0.5, False, False, False),
        _obs("t3", True, 0.4, True, False, False), _obs("t4", False, 0.6, False, False, False)]
GOOD = [_obs("t4", True, 0.2, False, True, True), _obs("t1", True, 0.9, True, True, True),
        _obs("t2", True, 0.7, True, True, False), _obs("t3", False, 0.3, False, False, True)]


def test_a_better_candidate_is_retained_with_exact_metrics():
    r = G.evaluate(CRIT, BASE, GOOD)
    assert r.decision == "retain" and r.failed_criteria == [] and r.held_out_task_ids == ["t1", "t2", "t3", "t4"]
    assert r.baseline.valid_patch_set_rate == 0.5 and r.candidate.valid_patch_set_rate == 0.75
    assert r.baseline.compile_brier_score == pytest.approx((0.16 + 0.25 + 0.36 + 0.36) / 4)
    assert r.candidate.compile_brier_score == pytest.approx((0.01 + 0.09 + 0.09 + 0.04) / 4)
    assert r.candidate.accepted_candidates == 3 and r.candidate.accepted_candidate_yield_per_budget == pytest.approx(3 / 40)
    assert r.criterion_sha256 == CRIT.sha256() and len(r.criterion_sha256) == 64
    assert json.loads(r.to_json())["decision"] == "retain"
    assert dataclasses.replace(CRIT, min_valid_patch_set_rate=0.61).sha256() != CRIT.sha256()


def test_unmet_criteria_reject_and_are_named():
    same = G.evaluate(CRIT, BASE, BASE)
    assert same.decision == "reject"
    assert {f.split(":")[0] for f in same.failed_criteria} >= {"valid_patch_set_rate.absolute", "valid_patch_set_rate.delta",
                                                                 "compile_brier_score.absolute", "compile_brier_score.improvement",
                                                                 "first_pass_gate_success_rate.delta"}
    strict = dataclasses.replace(CRIT, min_first_pass_gate_success_rate=0.9)
    r = G.evaluate(strict, BASE, GOOD)
    assert r.decision == "reject" and [f.split(":")[0] for f in r.failed_criteria] == ["first_pass_gate_success_rate.absolute"]


def test_the_gate_fails_closed():
    with pytest.raises(G.SpecializationGateError, match="task sets differ"):
        G.evaluate(CRIT, BASE, GOOD[:3] + [_obs("t5", True, 0.5, True, True, True)])
    with pytest.raises(G.SpecializationGateError, match="lacks compile_passed"):
        G.evaluate(CRIT, BASE, GOOD[:3] + [G.Observation("t3", False, 0.3, None, False, True, 10)])
    with pytest.raises(G.SpecializationGateError, match="measured twice"):
        G.evaluate(CRIT, BASE + [BASE[0]], GOOD)
    with pytest.raises(G.SpecializationGateError, match="spent 400"):
        G.evaluate(CRIT, BASE, [dataclasses.replace(o, evaluation_cost=100) for o in GOOD])
    with pytest.raises(G.SpecializationGateError, match="probability"):
        G.evaluate(CRIT, BASE, [dataclasses.replace(GOOD[0], compile_pass_probability=1.2)] + GOOD[1:])
    with pytest.raises(G.SpecializationGateError, match="no held-out"):
        G.evaluate(CRIT, [], [])
    with pytest.raises(G.SpecializationGateError, match="budget spent is zero"):
        G.evaluate(CRIT, [dataclasses.replace(o, evaluation_cost=0) for o in BASE], GOOD)
    for bad in (dataclasses.replace(CRIT, version=2), dataclasses.replace(CRIT, max_evaluation_budget=0),
                dataclasses.replace(CRIT, min_valid_patch_set_rate=1.5), dataclasses.replace(CRIT, min_compile_brier_improvement=float("nan"))):
        with pytest.raises(G.SpecializationGateError):
            G.evaluate(bad, BASE, GOOD)

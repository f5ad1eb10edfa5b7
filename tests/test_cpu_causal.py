"""Causal graphs, structural models, conditional-independence tests, structure discovery and effect estimates (CPU)."""
import pytest
import torch

from scirust_b200 import causal as C


def _confounded():
    g = C.CausalGraph(edges=[("z", "x"), ("z", "y"), ("x", "m"), ("m", "y"), ("x", "c"), ("y", "c")])
    scm = C.LinearScm(g, {("z", "x"): 0.8, ("z", "y"): 1.5, ("x", "m"): 0.9, ("m", "y"): 0.7, ("x", "c"): 0.5, ("y", "c"): 0.5})
    return g, scm


def test_graph_queries_d_separation_and_backdoor_sets():
    g, _ = _confounded()
    assert g.parents("y") == {"z", "m"} and g.ancestors("c") == {"x", "y", "z", "m"} and g.descendants("x") == {"m", "y", "c"}
    order = g.topological_order()
    assert all(order.index(a) < order.index(b) for a, b in g.edges())
    with pytest.raises(C.CausalError):
        g.add_edge("c", "z")
    assert not g.d_separated(["x"], ["y"]) and not g.d_separated(["x"], ["y"], ["z"])              # the mediated path stays open
    assert g.d_separated(["x"], ["y"], ["z", "m"]) and not g.d_separated(["x"], ["y"], ["z", "m", "c"])    # conditioning on a collider opens it
    chain = C.CausalGraph(edges=[("a", "b"), ("b", "c")])
    assert not chain.d_separated(["a"], ["c"]) and chain.d_separated(["a"], ["c"], ["b"])
    coll = C.CausalGraph(edges=[("a", "b"), ("c", "b"), ("b", "d")])
    assert coll.d_separated(["a"], ["c"]) and not coll.d_separated(["a"], ["c"], ["d"])            # a descendant of the collider
    assert g.satisfies_backdoor("x", "y", ["z"]) and not g.satisfies_backdoor("x", "y", []) and not g.satisfies_backdoor("x", "y", ["z", "m"])
    assert g.minimal_adjustment_set("x", "y") == ["z"] and chain.minimal_adjustment_set("a", "c") == []


def test_structural_model_interventions_effects_and_counterfactuals():
    g, scm = _confounded()
    assert scm.total_effect("x", "y") == pytest.approx(0.9 * 0.7) and scm.total_effect("y", "x") == 0.0
    data, _ = scm.sample(40000, seed=1)
    ix = scm.index
    naive = C.regression_adjustment(data, ix["x"], ix["y"])
    adjusted = C.regression_adjustment(data, ix["x"], ix["y"], [ix["z"]])
    assert abs(adjusted - 0.63) < 0.02 and abs(naive - 0.63) > 0.3                                 # confounding bias without z
    assert abs(C.regression_adjustment(data, ix["x"], ix["y"], [ix["z"], ix["c"]]) - 0.63) > 0.1    # collider bias
    do1, _ = scm.sample(40000, seed=2, do={"x": 1.0})
    do0, _ = scm.sample(40000, seed=2, do={"x": 0.0})
    assert abs(float((do1[:, ix["y"]] - do0[:, ix["y"]]).mean()) - 0.63) < 1e-9                    # same noise: exact difference
    assert float(do1[:, ix["z"]].sub(do0[:, ix["z"]]).abs().max()) == 0.0                          # upstream untouched
    unit = {n: float(data[0, ix[n]]) for n in scm.order}
    same = scm.counterfactual(unit, {})
    assert all(abs(same[n] - unit[n]) < 1e-12 for n in unit)                                       # consistency
    cf = scm.counterfactual(unit, {"x": unit["x"] + 1.0})
    assert cf["y"] - unit["y"] == pytest.approx(0.63) and cf["z"] == pytest.approx(unit["z"])
    with pytest.raises(C.CausalError):
        C.LinearScm(g, {("y", "x"): 1.0})


def test_partial_correlation_and_pc_recover_the_equivalence_class():
    g = C.CausalGraph(edges=[("a", "c"), ("b", "c"), ("c", "d")])
    scm = C.LinearScm(g, {("a", "c"): 1.0, ("b", "c"): -1.0, ("c", "d"): 0.8})
    data, _ = scm.sample(5000, seed=3)
    ix = scm.index
    assert abs(C.partial_correlation(data, ix["a"], ix["b"])) < 0.05
    assert abs(C.partial_correlation(data, ix["a"], ix["b"], [ix["c"]])) > 0.3                     # explaining away
    assert abs(C.partial_correlation(data, ix["a"], ix["d"], [ix["c"]])) < 0.05
    indep, p = C.fisher_z_test(data, ix["a"], ix["d"], [ix["c"]])
    assert indep and p > 0.05 and not C.fisher_z_test(data, ix["a"], ix["c"])[0]
    directed, undirected, sep = C.pc_algorithm(data, scm.order)
    assert directed == [("a", "c"), ("b", "c"), ("c", "d")] and undirected == set()                # collider + Meek rule 1
    assert sep[frozenset(("a", "d"))] == {"c"}
    chain = C.LinearScm(C.CausalGraph(edges=[("u", "v"), ("v", "w")]), {("u", "v"): 1.0, ("v", "w"): 1.0})
    cd, cu, _ = C.pc_algorithm(chain.sample(5000, seed=4)[0], chain.order)
    assert cd == [] and cu == {frozenset(("u", "v")), frozenset(("v", "w"))}                       # a chain has no orientable edge


def test_notears_learns_a_weighted_dag_and_the_acyclicity_function_detects_cycles():
    dag = torch.tensor([[0.0, 1.0, 0.0], [0.0, 0.0, 2.0], [0.0, 0.0, 0.0]], dtype=torch.float64)
    cyc = dag.clone()
    cyc[2, 0] = 0.5
    assert abs(float(C.acyclicity(dag))) < 1e-12 and float(C.acyclicity(cyc)) > 0.1
    g = C.CausalGraph(edges=[("a", "b"), ("a", "c"), ("b", "d"), ("c", "d")])
    scm = C.LinearScm(g, {("a", "b"): 1.5, ("a", "c"): -1.2, ("b", "d"): 1.0, ("c", "d"): 1.3})
    data, _ = scm.sample(2000, seed=5)
    w = C.notears_linear(data, lam=0.02, max_outer=8, inner_steps=200)
    assert float(C.acyclicity(w)) < 1e-6
    truth = scm.b
    assert torch.equal(w != 0, truth != 0) and float((w - truth).abs().max()) < 0.15


def test_inverse_probability_weighting_removes_confounding_of_a_binary_treatment():
    g = torch.Generator().manual_seed(6)
    n = 40000
    z = torch.randn(n, generator=g, dtype=torch.float64)
    t = (torch.rand(n, generator=g, dtype=torch.float64) < torch.sigmoid(1.5 * z)).double()
    y = 2.0 * t + 3.0 * z + torch.randn(n, generator=g, dtype=torch.float64)
    data = torch.stack([z, t, y], 1)
    naive = float(y[t == 1].mean() - y[t == 0].mean())
    assert abs(naive - 2.0) > 1.5 and abs(C.ipw_effect(data, 1, 2, [0]) - 2.0) < 0.15
    assert abs(C.regression_adjustment(data, 1, 2, [0]) - 2.0) < 0.05

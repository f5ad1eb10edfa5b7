"""Monitoring, packaging and model-search utilities (CPU)."""
import math

import torch

from scirust_b200 import automl as A
from scirust_b200 import mlops as M


def test_psi_drift_detector():
    rng = A.XorShift64(0xD1F70001)
    ref = [rng.uniform(0, 10) for _ in range(1000)]
    det = M.DataDriftDetector(ref, 10, 200, 0.25)
    for _ in range(199):
        det.add_sample(rng.uniform(0, 10))
    assert det.check() is None and det.window_fill() == 199
    det.add_sample(rng.uniform(0, 10))
    rep = det.check()
    assert rep.drift_type == M.NO_DRIFT and rep.data_drift_score < 0.25 and det.window_fill() == 0
    for _ in range(200):
        det.add_sample(rng.uniform(8, 10))            # mass moved to the top bins
    rep = det.check()
    assert rep.drift_type == M.DATA_DRIFT and rep.data_drift_score > 0.25 and rep.sample_count == 400


def test_model_drift_and_shadow():
    md = M.ModelDriftDetector(10, baseline_error=0.1, threshold_factor=2.0)
    for _ in range(10):
        md.add_observation(1.0, 1.05)
    assert md.check().drift_type == M.NO_DRIFT
    for _ in range(10):
        md.add_observation(1.0, 2.0)
    rep = md.check()
    assert rep.drift_type == M.MODEL_DRIFT and math.isclose(rep.model_drift_score, 10.0)
    assert M.combine_reports(None, rep) == M.MODEL_DRIFT

    sh = M.ShadowDeployment(50, "mae", 0.05)
    for _ in range(50):
        sh.add_observation(11.0, 10.1, 10.0)
    res = sh.evaluate()
    assert res.improvement and res.recommendation == M.PROMOTE and math.isclose(res.production_metric, 1.0)
    sh = M.ShadowDeployment(4, "f1", 0.05)
    for p, s, a in [(1, 0, 1), (1, 0, 1), (0, 1, 0), (0, 0, 0)]:
        sh.add_observation(p, s, a)
    assert sh.evaluate().recommendation == M.KEEP


def test_ota_package_signature():
    key = M.SigningKey.derive("fleet-key", "correct horse")
    upd = M.OtaUpdate.create(b"weights" * 100, "1.2.0", "edge-7", key)
    assert upd.verify(key) and upd.apply(key).success
    other = M.SigningKey.derive("fleet-key", "wrong horse")
    assert not upd.verify(other)
    upd.model_bytes = upd.model_bytes[:-1] + b"!"
    res = upd.apply(key)
    assert not res.success and not res.signature_valid


def test_cross_validation_and_automl_pick_a_fitting_model():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(120, 3, generator=g, dtype=torch.float64)
    y = 2.0 * x[:, 0] - x[:, 1] + 0.5 + 0.01 * torch.randn(120, generator=g, dtype=torch.float64)
    splits = A.k_fold_splits(120, 4, A.XorShift64(3))
    assert sorted(i for _, va in splits for i in va) == list(range(120))
    cv = A.cross_validate(lambda: A.Ridge(1e-6), x, y, splits, "r2")
    assert cv.mean > 0.99
    ts = A.time_series_splits(100, 4)
    assert all(max(tr) < min(va) for tr, va in ts) and len(ts) == 4
    rep = A.AutoML(kinds=("ridge", "knn"), trials_per_kind=4, k=3, seed=1).fit(x, y)
    assert rep.best_kind == "ridge" and rep.best_score > -0.01
    rep2 = A.AutoML(kinds=("ridge", "knn"), trials_per_kind=4, k=3, seed=1).fit(x, y)
    assert rep.leaderboard == rep2.leaderboard          # seeded: the same trials in the same order


def test_bayesian_optimisation_finds_the_peak():
    def f(v):
        return -((v[0] - 0.3) ** 2 + (v[1] + 0.2) ** 2)
    x, y, hist = A.bayesian_optimize(f, [(-1, 1), (-1, 1)], max_iter=25, initial_samples=5, seed=4)
    assert y > -0.01 and len(hist) == 25
    assert A.bayesian_optimize(f, [(-1, 1), (-1, 1)], max_iter=25, initial_samples=5, seed=4)[0] == x
    gp = A.GaussianProcess(torch.tensor([[0.0], [1.0]]), torch.tensor([0.0, 1.0]))
    mu, var = gp.predict(torch.tensor([[0.0], [0.5]]))
    assert abs(float(mu[0])) < 1e-3 and float(var[0]) < 1e-4 and float(var[1]) > float(var[0])


def test_t_test_ensemble_and_spaces():
    r = A.paired_t_test([1.0, 2.0, 3.0, 4.0, 5.0], [0.9, 1.7, 2.9, 3.6, 4.8])
    assert r["df"] == 4 and r["t"] > 3 and r["p"] < 0.05
    from scipy.special import betainc
    for (pa, pb, px) in [(2.0, 0.5, 0.4), (0.5, 2.0, 0.9), (5.0, 0.5, 0.99)]:
        assert abs(A._betainc(pa, pb, px) - float(betainc(pa, pb, px))) < 1e-9
    same = A.paired_t_test([1.0, 2.0], [1.0, 2.0])
    assert same["p"] == 1.0
    rng = A.XorShift64(5)
    for d in (A.Uniform(0, 2), A.LogUniform(1e-4, 1.0), A.IntRange(3, 9), A.Choice(["a", "b", "c"])):
        v = d.sample(rng)
        assert d.from_unit(d.to_unit(v)) == v or abs(d.from_unit(d.to_unit(v)) - v) < 1e-9

    class Const:
        def __init__(self, c):
            self.c = c

        def predict(self, x):
            return torch.full((len(x),), self.c, dtype=torch.float64)
    x = torch.zeros(3, 1)
    assert A.ModelEnsemble([Const(1.0), Const(3.0)]).predict(x).tolist() == [2.0] * 3
    assert A.ModelEnsemble([Const(1.0), Const(3.0)], "weighted", [3, 1]).predict(x).tolist() == [1.5] * 3
    assert A.ModelEnsemble([Const(1.0), Const(1.0), Const(0.0)], "vote").predict(x).tolist() == [1.0] * 3


def test_nas_evolution_improves_and_builds():
    cfg = A.NasConfig(in_features=16, out_features=4, min_hidden=8, max_hidden=256, max_models=200, seed=7)
    s = A.NasSearch(cfg)
    arch = s.random_architecture(42)
    assert cfg.min_layers <= len(arch.layers) <= cfg.max_layers and arch.params_m > 0
    assert "Linear(" in str(arch)
    s.evolve(0, 16)
    first = s.population[0].fitness
    pop = s.evolve(8, 16)
    assert pop[0].fitness >= first and all(pop[i].fitness >= pop[i + 1].fitness for i in range(len(pop) - 1))
    assert [str(a) for a in A.NasSearch(cfg).evolve(8, 16)] == [str(a) for a in pop]
    net = A.build_module(pop[0], 16, 4)
    assert tuple(net(torch.randn(5, 16)).shape) == (5, 4)
    n_params = sum(p.numel() for p in net.parameters())
    assert abs(n_params / 1e6 - pop[0].params_m) < 1e-9
    trained = A.NasSearch(A.NasConfig(in_features=16, out_features=4, min_hidden=8, max_hidden=32, max_models=12),
                          score=lambda a: 1.0 / (1.0 + len(a.layers)))
    best = trained.evolve(2, 4)[0]
    assert best.accuracy is not None

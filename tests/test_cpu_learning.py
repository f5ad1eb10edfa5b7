"""Classical learning algorithms: regression family, Gaussian processes, unsupervised learning, forecasting, policy
gradients (CPU)."""
import math

import pytest
import torch

from scirust_b200.learning import (GaussianProcess, IsotonicRegression, KernelRidgeRegression, Matern32, Matern52, Rbf,
                                   fit_high_breakdown, fit_multi_output_robust, fit_quantile_regression,
                                   fit_robust_regression, influence_report)
from scirust_b200.learning import forecast as F
from scirust_b200.learning import rl as R
from scirust_b200.learning import unsupervised as U

D = torch.float64


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _contaminated(seed=0, n=200, bad=60):
    g = _gen(seed)
    x = torch.randn(n, 3, dtype=D, generator=g)
    beta = torch.tensor([1.5, -2.0, 0.5], dtype=D)
    y = x @ beta + 0.7 + 0.1 * torch.randn(n, dtype=D, generator=g)
    yc = y.clone()
    yc[:bad] += 20 + 5 * torch.randn(bad, dtype=D, generator=g)
    return x, y, yc, beta


def test_robust_and_high_breakdown_regression_survive_thirty_percent_outliers():
    x, y, yc, beta = _contaminated()
    ls = torch.linalg.lstsq(torch.cat([torch.ones(200, 1, dtype=D), x], 1), yc[:, None]).solution[:, 0]
    assert float((ls[1:] - beta).abs().max()) > 0.5                                         # least squares is wrecked
    for loss in ("tukey", "cauchy"):
        rep = fit_robust_regression(x, yc, loss)
        assert rep.converged and float((rep.model.coefficients - beta).abs().max()) < 0.05 and abs(float(rep.model.intercept) - 0.7) < 0.05
    hub = fit_robust_regression(x, yc, "huber")
    assert float((hub.model.coefficients - beta).abs().max()) < 0.1                         # monotone loss: bounded, not redescending
    lts = fit_high_breakdown(x, yc, seed=1)
    assert float((lts.model.coefficients - beta).abs().max()) < 0.05 and abs(float(lts.model.intercept) - 0.7) < 0.05
    assert set(range(60)) <= set(lts.outliers) and len(lts.outliers) < 75 and abs(lts.scale - 0.1) < 0.03
    clean = fit_robust_regression(x, y, "huber")
    assert len(clean.outliers) < 10 and abs(clean.scale - 0.1) < 0.03
    with pytest.raises(ValueError):
        fit_robust_regression(x[:3], y[:3])


def test_kernel_ridge_isotonic_quantile_multi_output_and_influence():
    g = _gen(2)
    x = torch.linspace(-3, 3, 80, dtype=D)
    y = torch.sin(x) + 0.05 * torch.randn(80, dtype=D, generator=g)
    kr = KernelRidgeRegression("rbf", gamma=0.5, ridge=1e-2).fit(x, y)
    assert float((kr.predict(x) - torch.sin(x))[5:-5].abs().max()) < 0.06 and kr.support_len() == 80
    lin = KernelRidgeRegression("linear", ridge=1e-8).fit(x, 2 * x)
    assert abs(float(lin.predict(torch.tensor([10.0], dtype=D))) - 20.0) < 1e-4
    with pytest.raises(ValueError):
        KernelRidgeRegression(ridge=0.0)
    iso = IsotonicRegression().fit([1, 2, 3, 4, 5], [1, 3, 2, 4, 3.5])
    assert iso.knots()[1].tolist() == [1.0, 2.5, 2.5, 3.75, 3.75]
    assert iso.predict([2.5, 0.0, 6.0]).tolist() == [2.5, 1.0, 3.75]                        # flat outside the data
    dec = IsotonicRegression(increasing=False).fit([1, 2, 3, 4], [4, 2, 3, 1])
    fitted = dec.predict([1.0, 2.0, 3.0, 4.0])
    assert bool((fitted[1:] <= fitted[:-1]).all()) and abs(float(fitted.sum()) - 10.0) < 1e-12    # the mean is preserved
    xs, yy, _, _ = _contaminated(3)
    for tau in (0.1, 0.5, 0.9):
        q = fit_quantile_regression(xs, yy, tau)
        assert abs(float((yy <= q.model.predict(xs)).double().mean()) - tau) < 0.03
    y2 = torch.stack([yy, 2 * yy + 1], 1)
    y2[:20] += 30
    mo = fit_multi_output_robust(xs, y2)
    assert float((mo.coefficients[:, 0] - torch.tensor([1.5, -2.0, 0.5], dtype=D)).abs().max()) < 0.05
    assert float((mo.intercept - torch.tensor([0.7, 2.4], dtype=D)).abs().max()) < 0.1 and float(mo.weights[:20].max()) < 0.1
    xi = torch.cat([torch.linspace(0, 1, 30, dtype=D), torch.tensor([5.0], dtype=D)])
    yi = torch.cat([2 * torch.linspace(0, 1, 30, dtype=D) + 0.01 * torch.randn(30, dtype=D, generator=g), torch.tensor([0.0], dtype=D)])
    inf = influence_report(xi, yi)
    assert 30 in inf.high_leverage and 30 in inf.influential and abs(float(inf.leverage.sum()) - 2.0) < 1e-9    # trace(H) = p
    assert int(inf.cooks_distance.argmax()) == 30 and inf.count("leverage") >= 1


def test_gaussian_process_interpolates_and_reports_honest_uncertainty():
    g = _gen(4)
    x = torch.linspace(-3, 3, 40, dtype=D)
    y = torch.sin(x) + 0.05 * torch.randn(40, dtype=D, generator=g)
    for kernel in (Rbf(1.0, 1.0), Matern32(1.5, 1.0), Matern52(1.5, 1.0)):
        gp = GaussianProcess(kernel, 0.05 ** 2).fit(x, y)
        mean, var = gp.predict_many(torch.tensor([0.5, 1.7, 30.0], dtype=D))
        assert abs(float(mean[0]) - math.sin(0.5)) < 0.08 and abs(float(mean[1]) - math.sin(1.7)) < 0.08
        assert float(var[0]) < 0.01 and abs(float(var[2]) - 1.0) < 1e-6                     # far away: the prior variance
        assert abs(float(mean[2]) - float(y.mean())) < 1e-6
    single = GaussianProcess(Rbf(), 1e-2).fit(x, y)
    m, v = single.predict([0.5])
    assert abs(m - math.sin(0.5)) < 0.08 and v >= 0
    poor = GaussianProcess(Rbf(0.01, 1.0), 1e-2).fit(x, y).log_marginal_likelihood()
    best = GaussianProcess.fit_best(x, y)
    assert best.log_marginal_likelihood() > poor + 10 and 0.3 < best.kernel.length_scale < 6.0
    with pytest.raises(ValueError):
        GaussianProcess(Rbf(), -1.0)


def _blobs(seed=5):
    g = _gen(seed)
    centers = torch.tensor([[0.0, 0.0], [3.0, 3.0], [0.0, 3.0]], dtype=D)
    x = torch.cat([torch.randn(100, 2, dtype=D, generator=g) * 0.3 + c for c in centers])
    return x, torch.tensor([[8.0, 8.0], [-5.0, 6.0]], dtype=D)


def test_clustering_density_models_and_anomaly_detectors():
    x, out = _blobs()
    xo = torch.cat([x, out])
    km = U.KMeans(3).fit(x)
    assert sorted(torch.bincount(km.predict(x)).tolist()) == [100, 100, 100] and km.inertia < 70
    p2 = U.Pca(2).fit(x)
    assert float((p2.inverse_transform(p2.transform(x)) - x).abs().max()) < 1e-12 and abs(float(p2.explained_ratio.sum()) - 1) < 1e-12
    labels = U.Dbscan(0.5, 5).fit(xo)
    assert labels[-2:].tolist() == [-1, -1] and int(labels.max()) + 1 == 3
    assert len({int(labels[i]) for i in range(0, 100) if int(labels[i]) >= 0}) == 1
    lof = U.LocalOutlierFactor(10).fit_predict(xo)
    assert float(lof[-2:].min()) > 3.0 and float(lof[:300].median()) < 1.2
    gm = U.GaussianMixture(3).fit(x)
    assert gm.converged and max(abs(w - 1 / 3) for w in gm.weights.tolist()) < 0.02
    assert gm.bic(x) < U.GaussianMixture(1).fit(x).bic(x) and gm.bic(x) < U.GaussianMixture(6).fit(x).bic(x)
    assert float(gm.predict_proba(x).sum(1).sub(1).abs().max()) < 1e-12
    assert len(set(gm.predict(x[:100]).tolist())) == 1
    forest = U.IsolationForest(50, 128).fit(xo)
    s = forest.anomaly_scores(xo)
    assert float(s[-2:].min()) > float(s[:300].max()) and forest.detect_anomalies(xo, 0.7) == [300, 301]
    ae = U.AutoencoderDetector(2, 8, 1)
    ae.train(x, 200)
    assert float(ae.anomaly_scores(out).min()) > 5 * float(ae.anomaly_scores(x).max())
    with pytest.raises(ValueError):
        U.KMeans(0).fit(x)


def test_forecasting_models_recover_their_generating_processes():
    g = _gen(6)
    n = torch.arange(120, dtype=D)
    y = 10 + 0.5 * n + 5 * torch.sin(2 * math.pi * n / 12) + 0.3 * torch.randn(120, dtype=D, generator=g)
    hw = F.ExponentialSmoothing(trend=True, season=12).fit(y[:108])
    fc = hw.forecast(12)
    assert F.rmse(y[108:], fc) < 0.6 and F.mase(y[108:], fc, y[:108], 12) < 0.2 and F.smape(y[108:], fc) < 1.0
    holt = F.ExponentialSmoothing(trend=True).fit(3 + 2 * n[:40])
    assert float((holt.forecast(3) - torch.tensor([83.0, 85.0, 87.0], dtype=D)).abs().max()) < 1e-6
    ses = F.ExponentialSmoothing(alpha=0.5).fit([1.0, 2.0, 3.0])
    assert ses.forecast(2).tolist() == [2.25, 2.25]
    e = torch.randn(800, dtype=D, generator=g)
    ar_y = [0.0, 0.0]
    for t in range(2, 800):
        ar_y.append(0.6 * ar_y[-1] - 0.3 * ar_y[-2] + float(e[t]))
    ar = F.AutoRegression(2).fit(ar_y)
    assert float((ar.coefficients - torch.tensor([0.6, -0.3], dtype=D)).abs().max()) < 0.08 and abs(ar.sigma2 - 1) < 0.15
    assert F.AutoRegression(2).fit(ar_y).aic() < F.AutoRegression(1).fit(ar_y).aic()
    ma = [float(e[t] + 0.5 * e[t - 1]) for t in range(1, 800)]
    assert abs(float(F.Arima(0, 0, 1).fit(ma).ma[0]) - 0.5) < 0.1
    walk = torch.cumsum(torch.tensor(ar_y, dtype=D) + 0.2, 0)
    ai = F.Arima(2, 1, 0).fit(walk)
    assert float((ai.ar - torch.tensor([0.6, -0.3], dtype=D)).abs().max()) < 0.08
    assert float((ai.forecast(3) - walk[-1]).abs().max()) < 5.0                             # forecasts continue from the last level
    assert torch.equal(F.undifference(F.difference(walk, 2)[-3:], walk[:-3], 2), walk[-3:]) or \
        float((F.undifference(F.difference(walk, 2)[-3:], walk[:-3], 2) - walk[-3:]).abs().max()) < 1e-9
    assert F.mae([1, 2, 3], [1, 2, 5]) == pytest.approx(2 / 3) and F.mape([2, 4], [1, 5]) == pytest.approx(37.5)
    with pytest.raises(ValueError):
        F.Arima(0, 1, 0)


def test_policy_gradient_agents_learn_their_tasks():
    for algo in ("reinforce", "a2c", "ppo"):
        agent = R.PolicyGradientAgent(R.Corridor(), algo, seed=0)
        history = agent.train(40, 32)
        assert agent.evaluate() > 0.9 and history[-1] > history[0] + 0.5, algo
    agent = R.PolicyGradientAgent(R.CartPole(horizon=200), "a2c", seed=1)
    history = agent.train(45, 16)
    assert sum(history[-5:]) / 5 > 4 * history[0] and agent.evaluate() > 120
    rew, mask = torch.ones(3, 1), torch.ones(3, 1)
    assert R.discounted_returns(rew, mask, 0.5)[:, 0].tolist() == [1.75, 1.5, 1.0]
    adv, ret = R.gae(rew, torch.zeros(3, 1), mask, 0.5, 1.0)                                 # lambda = 1: Monte-Carlo returns
    assert ret[:, 0].tolist() == [1.75, 1.5, 1.0]
    with pytest.raises(ValueError):
        R.PolicyGradientAgent(R.Corridor(), "dqn")

"""Statistical and formal certificates: special functions, conformal family, randomised smoothing, Lipschitz
certificates, abstract domains (zonotope, DeepPoly), branch and bound against the exact 2-input verifiers,
certified training, run-time contracts, watermark, seeded sampling, prediction intervals, deep ensembles."""
import math

import pytest
import torch

from scirust_b200 import conformal as CF
from scirust_b200 import verify as V
from scirust_b200.certify import IbpLinear, IbpMlp, Interval, StatisticalGuard, certified_robust
from scirust_b200.nn import intervals, lipschitz, sampling, smoothing, watermark
from scirust_b200.nn.contracts import CertifiedModule, ValueBoundedContract
from scirust_b200.nn.crown_ibp import CrownIbpMlp
from scirust_b200.nn.ensemble import DeepEnsemble
from scirust_b200.nn.rng import PcgEngine
from scirust_b200.numerics import special as S


def test_special_functions_against_known_values():
    assert abs(S.inv_normal_cdf(0.975) - 1.959964) < 1e-5
    assert abs(S.normal_cdf(S.inv_normal_cdf(0.3)) - 0.3) < 1e-8
    assert S.inv_normal_cdf(0.0) == -math.inf and S.inv_normal_cdf(1.0) == math.inf
    # I_x(a, b) closed forms: I_x(1, 1) = x; I_x(2, 1) = x^2; symmetry I_x(a,b) = 1 - I_{1-x}(b,a)
    assert abs(S.regularized_incomplete_beta(1, 1, 0.37) - 0.37) < 1e-12
    assert abs(S.regularized_incomplete_beta(2, 1, 0.6) - 0.36) < 1e-12
    a = S.regularized_incomplete_beta(2.5, 4.0, 0.3)
    assert abs(a - (1 - S.regularized_incomplete_beta(4.0, 2.5, 0.7))) < 1e-12
    assert abs(S.beta_inv(a, 2.5, 4.0) - 0.3) < 1e-9
    # Student t: nu = 1 is Cauchy, cdf(1) = 3/4; t_{0.975, 5} = 2.5706
    assert abs(S.student_t_cdf(1.0, 1.0) - 0.75) < 1e-10
    assert abs(S.student_t_ppf(0.975, 5) - 2.570582) < 1e-5
    assert S.student_t_ppf(0.025, 5) == -S.student_t_ppf(0.975, 5)
    # Clopper-Pearson: k = n gives alpha^(1/n)
    assert abs(S.clopper_pearson_lower(50, 50, 0.01) - 0.01 ** (1 / 50)) < 1e-9
    assert S.clopper_pearson_lower(0, 10, 0.05) == 0.0


def test_conformal_quantile_and_coverage():
    assert CF.conformal_quantile([0.1 * i for i in range(1, 10)], 0.2) == pytest.approx(0.8)
    assert CF.conformal_quantile([0.5, 0.7], 0.1) == math.inf          # too few points for the level
    assert CF.conformal_quantile([], 0.1) == math.inf
    torch.manual_seed(0)
    probs = torch.softmax(torch.randn(1200, 6) * 2, 1)
    y = torch.multinomial(probs, 1).squeeze(1)
    cal, test = slice(0, 600), range(600, 1200)
    for clf in (CF.ConformalClassifier.calibrate(probs[cal], y[cal], 0.1),
                CF.AdaptivePredictionSets.calibrate(probs[cal], y[cal], 0.1),
                CF.AdaptivePredictionSets.calibrate_raps(probs[cal], y[cal], 0.1, 2, 0.05)):
        cov = sum(clf.covers(probs[i], int(y[i])) for i in test) / 600
        assert 0.85 <= cov <= 0.96
        assert all(int(y[i]) in clf.predict_set(probs[i]) for i in test if clf.covers(probs[i], int(y[i])))
    # APS score: cumulative mass in descending order
    assert torch.allclose(CF.aps_scores(torch.tensor([0.2, 0.5, 0.3])), torch.tensor([1.0, 0.5, 0.8]))
    # the guard's verdicts come from the same threshold rule
    g = StatisticalGuard.calibrate(probs[cal], y[cal], 0.1)
    verdicts = {g.decide(probs[i])[0] for i in test}
    assert verdicts <= {"accept", "abstain", "reject"} and "accept" in verdicts


def test_conformal_regression_cqr_and_aci():
    torch.manual_seed(1)
    x = torch.rand(2000) * 4
    noise = torch.randn(2000) * (0.2 + 0.5 * x)                 # heteroscedastic
    y = torch.sin(x) + noise
    y_hat = torch.sin(x)
    reg = CF.ConformalRegressor.calibrate((y - y_hat)[:1000].abs(), 0.1)
    cov = sum(reg.covers(float(y_hat[i]), float(y[i])) for i in range(1000, 2000)) / 1000
    assert 0.86 <= cov <= 0.94
    lo, hi = y_hat - 1.0 * (0.2 + 0.5 * x), y_hat + 1.0 * (0.2 + 0.5 * x)       # a too-narrow base band
    cqr = CF.ConformalQuantileRegressor.calibrate(lo[:1000], hi[:1000], y[:1000], 0.1)
    cov2 = sum(cqr.covers(float(lo[i]), float(hi[i]), float(y[i])) for i in range(1000, 2000)) / 1000
    assert 0.86 <= cov2 <= 0.94 and cqr.correction() > 0
    # adaptive widths: CQR intervals at small x are narrower than the constant-width ones
    assert (torch.tensor([cqr.interval(float(l), float(h))[1] - cqr.interval(float(l), float(h))[0]
                          for l, h in zip(lo[:50], hi[:50])]).std() > 0.1)
    # ACI holds its level through a shift in the score scale
    aci = CF.AdaptiveConformal(0.1, 0.02)
    torch.manual_seed(2)
    scores = torch.cat([torch.rand(600), torch.rand(900) * 3]).tolist()
    window, misses = [], 0
    for t, s in enumerate(scores):
        if len(window) >= 50:
            covered = aci.step(window[-200:], s)
            misses += (not covered) and t >= 700
        window.append(s)
    assert misses / 800 < 0.16
    with pytest.raises(ValueError):
        CF.AdaptiveConformal(1.5, 0.1)


def test_risk_control():
    assert CF.hoeffding_ucb(0.1, 0, 0.05) == math.inf
    assert CF.hoeffding_ucb(0.1, 1000, 0.05) == pytest.approx(0.1 + math.sqrt(math.log(20) / 2000))
    risks = [0.40, 0.22, 0.12, 0.05, 0.01]
    i = CF.rcps_select(risks, 2000, 0.15, 0.05)
    assert i == 2 and CF.rcps_select(risks, 2000, 0.001, 0.05) is None
    # a non-monotone bump to the right stops the scan there
    assert CF.rcps_select([0.01, 0.5, 0.01], 2000, 0.15, 0.05) == 2
    assert CF.hoeffding_pvalue(0.3, 100, 0.2) == 1.0
    sel = CF.learn_then_test([0.30, 0.02, 0.25, 0.01], 500, 0.2, 0.05)
    assert sel == [1, 3]


def test_randomised_smoothing_certificate():
    f = lambda X: (X[:, 0] > 0).long()                               # half-space classifier
    sm = smoothing.SmoothedClassifier(0.5)
    x = torch.tensor([1.0, 0.0, 0.0])
    cert = sm.certify_cohen(f, x, 100, 2000, 2, 0.001, PcgEngine(7))
    assert cert.cls == 1 and not cert.abstained
    # exact radius of the smoothed half-space is the distance to the boundary (1.0); the certificate is below it
    assert 0.5 < cert.radius <= 1.0 + 1e-6
    # same seed, same certificate; per-sample and batched base classifiers see the same noise
    again = sm.certify_cohen(lambda v: int(v[0] > 0), x, 100, 2000, 2, 0.001, PcgEngine(7), batched=False)
    assert again == cert
    # on the boundary the vote is split and the classifier abstains
    c0 = sm.certify(f, torch.zeros(3), 1000, 2, 0.001, PcgEngine(1))
    assert c0.abstained and c0.radius == 0.0
    assert sm.predict(f, x, 200, 2, PcgEngine(3)) == 1
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(ValueError):
            smoothing.SmoothedClassifier(bad)
    with pytest.raises(ValueError):
        sm.certify(f, x, 10, 2, 1.5, PcgEngine(0))
    with pytest.raises(ValueError):
        sm.certify(lambda X: torch.full((X.shape[0],), 5), x, 10, 2, 0.01, PcgEngine(0))


def test_lipschitz_bounds_and_gloro():
    torch.manual_seed(0)
    W = torch.randn(5, 9)
    exact = float(torch.linalg.svdvals(W)[0])
    est = lipschitz.spectral_norm(W, iters=200)
    ub = lipschitz.spectral_norm_upper_bound(W)
    assert abs(est - exact) < 1e-3 and ub >= exact
    assert lipschitz.spectral_norm(W.reshape(-1).tolist(), 5, 9, 200) == pytest.approx(est)
    assert abs(lipschitz.spectral_norm(lipschitz.spectral_normalize(W, iters=200), iters=200) - 1.0) < 1e-3
    # the float32 narrowing never lands below the true norm (all-ones matrix times 2^23 + 1)
    big = torch.full((7, 7), float(2 ** 23 + 1))
    assert lipschitz.spectral_norm_upper_bound(big) >= 7 * (2 ** 23 + 1)
    g = lipschitz.GloroClassifier(W, 5, 9)
    x = torch.randn(9)
    cls, radius = g.certify(x)
    assert g.lipschitz() >= g.lipschitz_estimate() - 1e-4 and radius >= 0
    # no perturbation inside the ball changes the class
    for _ in range(200):
        d = torch.randn(9)
        d = d / d.norm() * radius * 0.999
        assert int(g.logits(x + d).argmax()) == cls
    cb, rb = g.certify(torch.stack([x, x * 2]))
    assert int(cb[0]) == cls and float(rb[1]) == pytest.approx(2 * radius, rel=1e-4)
    with pytest.raises(ValueError):
        lipschitz.GloroClassifier(W, 1, 45)
    with pytest.raises(ValueError):
        g.logits(torch.randn(4))


def _net(dims, seed):
    torch.manual_seed(seed)
    return [IbpLinear(torch.randn(a, b) * 0.7, torch.randn(b) * 0.3) for a, b in zip(dims[:-1], dims[1:])]


def test_zonotope_and_deeppoly_are_sound_and_tighter_than_ibp():
    for seed in range(5):
        layers = _net([4, 8, 8, 3], seed)
        mlp = IbpMlp(layers)
        x = torch.randn(4)
        box = Interval.around(x, 0.1)
        ibp, zono, dp = mlp.certify(box), mlp.certify_zonotope(box), mlp.certify_deeppoly(box)
        pts = x + (torch.rand(5000, 4) * 2 - 1) * 0.1
        out = mlp.forward(pts)
        for b in (ibp, zono, dp):
            assert bool((out >= b.lo - 1e-4).all()) and bool((out <= b.hi + 1e-4).all())
        assert float(zono.width().sum()) <= float(ibp.width().sum()) + 1e-4
        assert float(dp.width().sum()) <= float(ibp.width().sum()) + 1e-4
    # a point box certifies to the point
    p = Interval.around(x, 0.0)
    assert torch.allclose(mlp.certify_deeppoly(p).lo, mlp.forward(x), atol=1e-5)
    # relu(x) + relu(-x) = |x|: DeepPoly keeps the relation, intervals lose it
    l1 = IbpLinear(torch.tensor([[1.0, -1.0]]), torch.zeros(2))
    l2 = IbpLinear(torch.tensor([[1.0], [1.0]]), torch.zeros(1))
    box = Interval(torch.tensor([-1.0]), torch.tensor([1.0]))
    assert float(V.deeppoly_certify([l1, l2], box).hi) <= float(IbpMlp([l1, l2]).certify(box).hi)
    # batched boxes equal one-at-a-time
    lo = torch.randn(6, 4)
    hi = lo + torch.rand(6, 4) * 0.3
    bl, bh = V.deeppoly_bounds(layers, lo, hi)
    for i in range(6):
        one = V.deeppoly_certify(layers, Interval(lo[i], hi[i]))
        assert torch.allclose(one.lo, torch.minimum(bl[i], bh[i]), atol=1e-5) and torch.allclose(one.hi, bh[i], atol=1e-5)


def test_branch_and_bound_agrees_with_exact_verifiers():
    outcomes = set()
    for seed in range(30):
        torch.manual_seed(seed)
        l1 = IbpLinear(torch.randn(2, 5), torch.randn(5) * 0.5)
        l2 = IbpLinear(torch.randn(5, 3), torch.randn(3) * 0.5)
        net = IbpMlp([l1, l2])
        x = torch.randn(2)
        t = int(net.forward(x).argmax())
        box = Interval.around(x, 0.15)
        milp = V.milp_verify_robustness(l1, l2, box, t)
        plex = V.reluplex_verify(l1, l2, box, t)
        bab = V.verify_robustness([l1, l2], box, t, 1e-5, 20000)
        assert milp.status == plex.status
        assert bab.status in (milp.status, "unknown")
        assert plex.boxes <= 1 << 5 and V.reluplex_unstable_count(l1, box) <= 5
        outcomes.add(milp.status)
        if bab.status == "unsafe":
            ce = bab.counterexample
            assert bool(((ce >= box.lo) & (ce <= box.hi)).all()) and int(net.forward(ce).argmax()) != t
        if milp.status == "unsafe":
            m, w = V.milp_min_margin(l1, l2, box, t)
            z = net.forward(w)
            others = torch.cat([z[:t], z[t + 1:]])
            assert m <= 0 and float(z[t] - others.max()) == pytest.approx(m, abs=1e-3)
        if milp.status == "robust":
            assert not certified_robust(net.certify(box), t) or bab.status == "robust"
    assert outcomes == {"robust", "unsafe"}
    # the box budget is honoured
    r = V.verify_robustness(_net([3, 16, 16, 4], 3), Interval.around(torch.zeros(3), 2.0), 0, 1e-9, 50)
    assert r.status in ("unknown", "unsafe") and r.boxes <= 50 + 256


def test_certified_training_grows_the_certified_radius():
    torch.manual_seed(0)
    X = torch.cat([torch.randn(150, 2) * 0.45 + torch.tensor([1.0, 0.0]), torch.randn(150, 2) * 0.45 - torch.tensor([1.0, 0.0])])
    y = torch.cat([torch.zeros(150), torch.ones(150)]).long()

    def fit(eps):
        m = CrownIbpMlp([2, 24, 24, 2], PcgEngine(3))
        opt = torch.optim.Adam(m.parameters(), 1e-2)
        for s in range(400):
            opt.zero_grad()
            loss = m.robust_loss(X, eps * min(1.0, s / 150), y) if eps > 0 else torch.nn.functional.cross_entropy(m(X), y)
            loss.backward()
            opt.step()
        return m

    plain, robust = fit(0.0), fit(0.2)
    assert robust.certified_accuracy(X, y, 0.2) > plain.certified_accuracy(X, y, 0.2) + 0.1
    # the training bound and the stand-alone verifier agree on the box
    lo, hi = robust.certified_box(X[0], 0.2)
    ref = robust.to_ibp_mlp().certify(Interval.around(X[0], 0.2))
    assert torch.allclose(lo, ref.lo, atol=1e-5) and torch.allclose(hi, ref.hi, atol=1e-5)
    for bad in (-0.1, float("nan")):
        with pytest.raises(ValueError):
            robust.robust_loss(X, bad, y)
    with pytest.raises(ValueError):
        robust.robust_loss(X, 0.1, y[:5])
    with pytest.raises(ValueError):
        robust.robust_loss(X, 0.1, torch.full((300,), 7))


def test_value_contract_scrubs_and_counts():
    c = ValueBoundedContract(-1, 1)
    t = torch.tensor([0.5, 3.0, float("nan"), float("-inf"), -0.2])
    assert c.validate(torch.tensor([0.1, -1.0, 1.0])) is None
    assert c.validate(t).tolist() == [0.5, 1.0, 0.0, -1.0, pytest.approx(-0.2)]
    assert ValueBoundedContract(2, 5).validate(torch.tensor([float("nan")])).item() == 2.0
    assert ValueBoundedContract(-5, -2).validate(torch.tensor([float("nan")])).item() == -2.0
    with pytest.raises(ValueError):
        ValueBoundedContract(1, 0)
    m = CertifiedModule(torch.nn.Linear(2, 2), c)
    with torch.no_grad():
        m.inner.weight.fill_(10.0)
    out = m(torch.tensor([[1.0, 1.0], [float("nan"), 0.0]]))
    assert float(out.detach().abs().max()) <= 1.0 and m.violations == 2


def test_watermark_is_detectable_without_the_model():
    seed, gamma, vocab = 1, 0.3, 200
    frac = sum(watermark.green_mask(seed, p, vocab, gamma).sum() for p in range(vocab)) / vocab ** 2
    assert abs(frac - gamma) < 0.02
    logits = torch.zeros(64)
    watermark.apply_green_bias(logits, 3, 11, 0.25, 2.0)
    for tok in range(64):
        assert logits[tok].item() == (2.0 if watermark.is_green(3, 11, tok, 0.25) else 0.0)
    rng = PcgEngine(5)
    plain, marked = [0], [0]
    for _ in range(300):
        plain.append(int(rng.float() * vocab))
        row = rng.fill_normal((vocab,))
        watermark.apply_green_bias(row, seed, marked[-1], gamma, 4.0)
        marked.append(int(row.argmax()))
    assert abs(watermark.detect_z(seed, plain, gamma)) < 3.0
    assert watermark.detect_z(seed, marked, gamma) > 8.0
    assert watermark.detect_z(seed + 1, marked, gamma) < 3.0                 # wrong key: nothing to see
    assert watermark.detect_p_value(seed, marked, gamma) < 1e-10
    assert watermark.detect_z(seed, [4], gamma) == 0.0


def test_seeded_sampling():
    logits = [0.1, 2.0, -1.0, 1.9]
    assert sampling.sample_token(logits, sampling.SamplingConfig.greedy(), PcgEngine(0)) == 1
    assert sampling.sample_token(logits, sampling.SamplingConfig(temperature=5.0, top_k=1), PcgEngine(0)) == 1
    assert sampling.sample_token([], sampling.SamplingConfig(), PcgEngine(0)) == 0
    a = [sampling.sample_token(logits, sampling.SamplingConfig(temperature=1.0), PcgEngine(s)) for s in range(50)]
    b = [sampling.sample_token(logits, sampling.SamplingConfig(temperature=1.0), PcgEngine(s)) for s in range(50)]
    assert a == b and len(set(a)) > 1
    rng = PcgEngine(9)
    topk = {sampling.sample_token(logits, sampling.SamplingConfig(temperature=1.0, top_k=2), rng) for _ in range(200)}
    assert topk == {1, 3}
    rng = PcgEngine(9)
    nucleus = {sampling.sample_token(logits, sampling.SamplingConfig(temperature=0.3, top_p=0.5), rng) for _ in range(100)}
    assert nucleus == {1}
    # frequencies follow the softmax
    rng = PcgEngine(11)
    n = 4000
    counts = torch.zeros(4)
    for _ in range(n):
        counts[sampling.sample_token(logits, sampling.SamplingConfig(), rng)] += 1
    assert torch.allclose(counts / n, torch.softmax(torch.tensor(logits), 0), atol=0.03)


def test_prediction_intervals():
    torch.manual_seed(0)
    res = (torch.randn(40) * 2.0).tolist()
    g, t = intervals.GaussianInterval.from_residuals(res), intervals.StudentTInterval.from_residuals(res)
    assert g.sigma == pytest.approx(t.sigma) and t.dof == 40
    assert t.half_width(0.95) > g.half_width(0.95) > 0
    assert g.half_width(0.95) == pytest.approx(1.959964 * g.sigma, rel=1e-4)
    lo, hi = g.interval(3.0, 0.9)
    assert lo < 3.0 < hi and (hi - 3.0) == pytest.approx(3.0 - lo)
    big = intervals.StudentTInterval.from_residuals((torch.randn(5000)).tolist())
    assert big.half_width(0.95) == pytest.approx(1.96 * big.sigma, rel=2e-3)
    assert intervals.GaussianInterval.from_residuals([]).sigma == 0.0


def test_deep_ensemble_uncertainty_grows_off_the_data():
    xs = torch.linspace(-1, 1, 40)
    ys = torch.sin(3 * xs)
    ens = DeepEnsemble.train(xs, ys, 5, 16, 400, 0.02, 100)
    assert len(ens) == 5
    mean, std = ens.predict(xs)
    assert float(((mean - ys) ** 2).mean()) < 0.02
    _, far = ens.predict(torch.tensor([4.0, -4.0]))
    assert float(far.mean()) > 3 * float(std.mean())
    m0, s0 = ens.predict(0.25)
    assert isinstance(m0, float) and s0 >= 0
    # members are independent of how many are trained together, and the run is reproducible
    solo = DeepEnsemble.train(xs, ys, 1, 16, 400, 0.02, 102)
    assert torch.allclose(solo.member_predictions(xs)[0], ens.member_predictions(xs)[2], atol=1e-4)
    again = DeepEnsemble.train(xs, ys, 5, 16, 400, 0.02, 100)
    assert torch.equal(again.w1, ens.w1)
    with pytest.raises(ValueError):
        DeepEnsemble.train(xs, ys[:5], 2, 4, 1, 0.1, 0)

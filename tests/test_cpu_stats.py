"""Statistics against scipy where it has the same routine, and against known closed forms otherwise (CPU)."""
import math

import numpy as np
import pytest
import torch

from scirust_b200 import stats as S

sp = pytest.importorskip("scipy.stats")


def test_descriptive_and_robust_summaries():
    x = [2.0, 4.0, 4.0, 4.0, 5.0, 5.0, 7.0, 9.0]
    assert S.mean(x) == 5.0 and S.variance(x) == pytest.approx(32 / 7) and S.std_error(x) == pytest.approx(math.sqrt(32 / 7 / 8))
    assert S.median(x) == 4.5 and S.quantile(x, 0.25) == pytest.approx(np.quantile(x, 0.25)) and S.interquartile_range(x) == pytest.approx(1.5)
    y = x + [1000.0]
    assert S.trimmed_mean(y, 0.12) == pytest.approx(np.mean(sorted(y)[1:-1])) and S.winsorized_mean(y, 0.12) == pytest.approx(np.mean([4.0] + sorted(y)[1:-1] + [9.0]))
    assert S.median_absolute_deviation(y, consistent=False) == 1.0 and S.weighted_median([1, 2, 3], [1, 1, 5]) == 3.0
    heavy = torch.cat([torch.randn(999, generator=torch.Generator().manual_seed(0), dtype=torch.float64), torch.tensor([1e6], dtype=torch.float64)])
    assert abs(S.median_of_means(heavy, 20)) < 0.3 < abs(S.mean(heavy))
    with pytest.raises(ValueError):
        S.trimmed_mean(x, 0.5)
    with pytest.raises(ValueError):
        S.mean([])


def test_distribution_functions_match_scipy():
    for a, x in ((0.5, 0.1), (2.0, 1.5), (10.0, 3.0), (10.0, 25.0), (100.0, 90.0)):
        assert S.regularized_gamma_p(a, x) == pytest.approx(float(sp.gamma.cdf(x, a)), abs=1e-12)
    assert S.chi2_cdf(3.84, 1) == pytest.approx(float(sp.chi2.cdf(3.84, 1)), abs=1e-12)
    assert S.f_cdf(2.5, 3, 20) == pytest.approx(float(sp.f.cdf(2.5, 3, 20)), abs=1e-10)
    assert S.binomial_cdf(3, 10, 0.4) == pytest.approx(float(sp.binom.cdf(3, 10, 0.4)), abs=1e-12)
    assert S.poisson_cdf(4, 2.5) == pytest.approx(float(sp.poisson.cdf(4, 2.5)), abs=1e-12)
    for v in (0.3, 0.8, 1.36, 2.0):
        assert S.kolmogorov_sf(v) == pytest.approx(float(sp.kstwobign.sf(v)), abs=1e-9)
    assert S.binomial_cdf(-1, 5, 0.5) == 0.0 and S.binomial_cdf(5, 5, 0.5) == 1.0 and S.poisson_cdf(-1, 1.0) == 0.0


def test_hypothesis_tests_match_scipy():
    g = np.random.default_rng(1)
    x, y, z = g.normal(0.3, 1.0, 40), g.normal(0.0, 2.0, 55), g.normal(0.5, 1.0, 30)
    r = S.t_test_one_sample(x, 0.0)
    ref = sp.ttest_1samp(x, 0.0)
    assert r.statistic == pytest.approx(ref.statistic) and r.p_value == pytest.approx(ref.pvalue, abs=1e-10) and r.dof == 39
    for eq in (False, True):
        r, ref = S.t_test_two_sample(x, y, equal_var=eq), sp.ttest_ind(x, y, equal_var=eq)
        assert r.statistic == pytest.approx(ref.statistic) and r.p_value == pytest.approx(ref.pvalue, abs=1e-10)
    r, ref = S.one_way_anova([x, y, z]), sp.f_oneway(x, y, z)
    assert r.statistic == pytest.approx(ref.statistic) and r.p_value == pytest.approx(ref.pvalue, abs=1e-10)
    obs, exp = [18, 22, 25, 35], [25, 25, 25, 25]
    r, ref = S.chi_square_gof(obs, exp), sp.chisquare(obs, exp)
    assert r.statistic == pytest.approx(ref.statistic) and r.p_value == pytest.approx(ref.pvalue, abs=1e-12) and r.rejects(0.1) and not r.rejects(0.05)
    table = [[20, 30, 10], [25, 15, 20]]
    r = S.chi_square_independence(table)
    ref = sp.chi2_contingency(table, correction=False)
    assert r.statistic == pytest.approx(ref[0]) and r.p_value == pytest.approx(ref[1], abs=1e-12) and r.dof == 2
    r, ref = S.ks_test_one_sample(x, lambda v: float(sp.norm(0.3, 1.0).cdf(v))), sp.kstest(x, sp.norm(0.3, 1.0).cdf)
    assert r.statistic == pytest.approx(ref.statistic) and abs(r.p_value - ref.pvalue) < 0.03
    assert S.ks_test_one_sample(y, lambda v: float(sp.norm(5.0, 1.0).cdf(v))).p_value < 1e-6
    a, b = np.round(x, 1), np.round(z, 1)                                       # rounding makes ties
    r, ref = S.mann_whitney_u(a, b), sp.mannwhitneyu(a, b, alternative="two-sided", method="asymptotic")
    assert r.statistic == pytest.approx(ref.statistic) and r.p_value == pytest.approx(ref.pvalue, abs=1e-10)


def test_survival_curves_log_rank_and_cox_regression():
    times = [6, 6, 6, 6, 7, 9, 10, 10, 11, 13, 16, 17, 19, 20, 22, 23, 25, 32, 32, 34, 35]       # 6-MP arm of the Freireich trial
    events = [1, 1, 1, 0, 1, 0, 1, 0, 0, 1, 1, 0, 0, 0, 1, 1, 0, 0, 0, 0, 0]
    km = S.kaplan_meier(times, events)
    assert [p[0] for p in km] == [6.0, 7.0, 10.0, 13.0, 16.0, 22.0, 23.0]
    assert km[0][1:4] == (21, 3, pytest.approx(18 / 21)) and km[-1][3] == pytest.approx(0.4482, abs=1e-4) and km[0][4] == pytest.approx(0.0764, abs=1e-4)
    na = S.nelson_aalen(times, events)
    assert na[0][1] == pytest.approx(3 / 21) and na[1][1] == pytest.approx(3 / 21 + 1 / 17)
    placebo = [1, 1, 2, 2, 3, 4, 4, 5, 5, 8, 8, 8, 8, 11, 11, 12, 12, 15, 17, 22, 23]
    lr = S.log_rank(times, events, placebo, [1] * 21)
    assert lr.statistic == pytest.approx(16.79, abs=0.01) and lr.p_value < 1e-4
    g = torch.Generator().manual_seed(2)
    n = 3000
    x = torch.randn(n, 2, generator=g, dtype=torch.float64)
    beta = torch.tensor([0.8, -0.5], dtype=torch.float64)
    t = -torch.log(torch.rand(n, generator=g, dtype=torch.float64)) / torch.exp(x @ beta)
    c = -torch.log(torch.rand(n, generator=g, dtype=torch.float64)) / 0.3
    fit = S.cox_proportional_hazards(torch.minimum(t, c), (t <= c).double(), x)
    assert fit.converged and float((fit.coefficients - beta).abs().max()) < 0.08
    assert float(fit.standard_errors.max()) < 0.05 and float(fit.p_values.max()) < 1e-6
    assert torch.allclose(fit.hazard_ratios(), torch.exp(fit.coefficients))
    null = S.cox_proportional_hazards(torch.minimum(t, c), (t <= c).double(), torch.randn(n, generator=g, dtype=torch.float64))
    assert abs(float(null.z[0])) < 3.5 and null.log_likelihood < fit.log_likelihood
    arm = torch.cat([torch.zeros(21, dtype=torch.float64), torch.ones(21, dtype=torch.float64)])
    tied = S.cox_proportional_hazards(times + placebo, events + [1] * 21, arm)              # heavy ties: Breslow
    assert float(tied.coefficients[0]) == pytest.approx(1.509, abs=0.01)

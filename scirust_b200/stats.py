"""Statistics: descriptive and robust summaries, distribution functions, hypothesis tests and survival analysis.

Distribution tails come from the regularised incomplete beta and gamma functions (continued fraction / series, to
about 1e-13), so p-values do not depend on a tabulated approximation. The Cox proportional-hazards fit is Newton's
method on the Breslow partial likelihood with the risk-set sums taken as reversed cumulative sums over the time-sorted
sample (one pass, vectorised), and reports coefficients, standard errors from the observed information, z statistics
and the log partial likelihood.
Reference counterpart: scirust-stats/src/{describe,robust,dist,htest,survival,cox}.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .numerics.special import normal_cdf, regularized_incomplete_beta, student_t_cdf

D = torch.float64


def _v(x):
    x = torch.as_tensor(x, dtype=D).reshape(-1)
    if x.numel() == 0:
        raise ValueError("empty sample")
    return x


# ------------------------------------------------------------------ descriptive and robust
def mean(x):
    return float(_v(x).mean())


def variance(x):
    x = _v(x)
    return float(x.var(unbiased=True)) if x.numel() > 1 else 0.0


def std_dev(x):
    return math.sqrt(variance(x))


def std_error(x):
    return std_dev(x) / math.sqrt(_v(x).numel())


def quantile(x, q: float):
    """Linear interpolation between order statistics (type 7)."""
    return float(torch.quantile(_v(x), q))


def median(x):
    return quantile(x, 0.5)


def median_absolute_deviation(x, consistent: bool = True):
    x = _v(x)
    m = (x - x.median()).abs()
    return float(torch.quantile(m, 0.5)) * (1.4826 if consistent else 1.0)


def interquartile_range(x):
    return quantile(x, 0.75) - quantile(x, 0.25)


def trimmed_mean(x, proportion: float):
    x = _v(x).sort().values
    k = int(math.floor(proportion * x.numel()))
    if 2 * k >= x.numel():
        raise ValueError("trimming removes every observation")
    return float(x[k:x.numel() - k].mean())


def winsorized_mean(x, proportion: float):
    x = _v(x).sort().values
    k = int(math.floor(proportion * x.numel()))
    if 2 * k >= x.numel():
        raise ValueError("winsorising replaces every observation")
    return float(x.clamp(x[k], x[x.numel() - 1 - k]).mean())


def weighted_median(x, w):
    x, w = _v(x), _v(w)
    if bool((w < 0).any()) or float(w.sum()) <= 0:
        raise ValueError("weights must be non-negative with a positive sum")
    order = torch.argsort(x)
    c = torch.cumsum(w[order], 0)
    return float(x[order][int(torch.searchsorted(c, 0.5 * c[-1]))])


def median_of_means(x, blocks: int, seed: int = 0):
    x = _v(x)
    if not 1 <= blocks <= x.numel():
        raise ValueError("1 <= blocks <= n")
    perm = torch.randperm(x.numel(), generator=torch.Generator().manual_seed(seed))
    return float(torch.stack([c.mean() for c in torch.tensor_split(x[perm], blocks)]).median())


# ------------------------------------------------------------------ distribution functions
def regularized_gamma_p(a: float, x: float) -> float:
    """P(a, x) = gamma(a, x) / Gamma(a): series for x < a + 1, Lentz continued fraction for the complement otherwise."""
    if x <= 0:
        return 0.0
    lg = math.lgamma(a)
    if x < a + 1:
        term = total = 1.0 / a
        n = a
        for _ in range(10000):
            n += 1
            term *= x / n
            total += term
            if abs(term) < abs(total) * 1e-16:
                break
        return min(1.0, total * math.exp(-x + a * math.log(x) - lg))
    tiny = 1e-300
    b = x + 1 - a
    c, d = 1 / tiny, 1 / b
    h = d
    for i in range(1, 10000):
        an = -i * (i - a)
        b += 2
        d = an * d + b
        d = tiny if abs(d) < tiny else d
        c = b + an / c
        c = tiny if abs(c) < tiny else c
        d = 1 / d
        delta = d * c
        h *= delta
        if abs(delta - 1) < 1e-16:
            break
    return max(0.0, 1.0 - math.exp(-x + a * math.log(x) - lg) * h)


def chi2_cdf(x: float, k: float) -> float:
    return regularized_gamma_p(k / 2, x / 2)


def f_cdf(x: float, d1: float, d2: float) -> float:
    return 0.0 if x <= 0 else regularized_incomplete_beta(d1 / 2, d2 / 2, d1 * x / (d1 * x + d2))


def binomial_cdf(k: int, n: int, p: float) -> float:
    if k < 0:
        return 0.0
    if k >= n:
        return 1.0
    return 1.0 - regularized_incomplete_beta(k + 1, n - k, p)


def poisson_cdf(k: int, lam: float) -> float:
    return 0.0 if k < 0 else 1.0 - regularized_gamma_p(k + 1, lam)


def kolmogorov_sf(x: float) -> float:
    """P(K > x) for the limiting Kolmogorov distribution."""
    if x <= 0:
        return 1.0
    if x < 1.18:                                                               # the theta-function form converges fast here
        t = math.exp(-math.pi ** 2 / (8 * x * x))
        return 1.0 - math.sqrt(2 * math.pi) / x * (t + t ** 9 + t ** 25 + t ** 49)
    return max(0.0, min(1.0, 2 * sum((-1) ** (j - 1) * math.exp(-2 * j * j * x * x) for j in range(1, 101))))


# ------------------------------------------------------------------ hypothesis tests
@dataclass
class TestResult:
    statistic: float
    p_value: float
    dof: float | None = None

    def rejects(self, alpha: float = 0.05) -> bool:
        return self.p_value < alpha


def _two_sided_t(t, nu):
    return 2.0 * (1.0 - student_t_cdf(abs(t), nu))


def t_test_one_sample(x, mu0: float = 0.0) -> TestResult:
    x = _v(x)
    t = (float(x.mean()) - mu0) / std_error(x)
    return TestResult(t, _two_sided_t(t, x.numel() - 1), x.numel() - 1)


def t_test_two_sample(x, y, equal_var: bool = False) -> TestResult:
    x, y = _v(x), _v(y)
    nx, ny, vx, vy = x.numel(), y.numel(), variance(x), variance(y)
    if equal_var:
        nu = nx + ny - 2
        se = math.sqrt(((nx - 1) * vx + (ny - 1) * vy) / nu * (1 / nx + 1 / ny))
    else:                                                                     # Welch-Satterthwaite
        se = math.sqrt(vx / nx + vy / ny)
        nu = (vx / nx + vy / ny) ** 2 / ((vx / nx) ** 2 / (nx - 1) + (vy / ny) ** 2 / (ny - 1))
    t = (float(x.mean()) - float(y.mean())) / se
    return TestResult(t, _two_sided_t(t, nu), nu)


def one_way_anova(groups) -> TestResult:
    gs = [_v(g) for g in groups]
    n, k = sum(g.numel() for g in gs), len(gs)
    if k < 2 or n <= k:
        raise ValueError("need at least two groups and more observations than groups")
    grand = torch.cat(gs).mean()
    ssb = sum(g.numel() * float((g.mean() - grand) ** 2) for g in gs)
    ssw = sum(float(((g - g.mean()) ** 2).sum()) for g in gs)
    f = (ssb / (k - 1)) / (ssw / (n - k))
    return TestResult(f, 1.0 - f_cdf(f, k - 1, n - k), k - 1)


def chi_square_gof(observed, expected, ddof: int = 0) -> TestResult:
    o, e = _v(observed), _v(expected)
    if o.shape != e.shape or bool((e <= 0).any()):
        raise ValueError("expected counts must be positive and match the observed ones")
    stat = float(((o - e) ** 2 / e).sum())
    k = o.numel() - 1 - ddof
    return TestResult(stat, 1.0 - chi2_cdf(stat, k), k)


def chi_square_independence(table) -> TestResult:
    t = torch.as_tensor(table, dtype=D)
    e = t.sum(1, keepdim=True) * t.sum(0, keepdim=True) / t.sum()
    stat = float(((t - e) ** 2 / e).sum())
    k = (t.shape[0] - 1) * (t.shape[1] - 1)
    return TestResult(stat, 1.0 - chi2_cdf(stat, k), k)


def ks_test_one_sample(x, cdf) -> TestResult:
    """``cdf`` maps a float to F(x); the p-value uses the limiting distribution with Stephens' finite-n correction."""
    x = _v(x).sort().values
    n = x.numel()
    f = torch.tensor([cdf(float(v)) for v in x], dtype=D)
    i = torch.arange(1, n + 1, dtype=D)
    d = float(torch.maximum(i / n - f, f - (i - 1) / n).max())
    return TestResult(d, kolmogorov_sf(d * (math.sqrt(n) + 0.12 + 0.11 / math.sqrt(n))))


def mann_whitney_u(x, y) -> TestResult:
    """Normal approximation with tie correction and continuity correction."""
    x, y = _v(x), _v(y)
    allv = torch.cat([x, y])
    order = torch.argsort(allv)
    ranks = torch.empty_like(allv)
    sv = allv[order]
    i, tie_term = 0, 0.0
    while i < sv.numel():
        j = i
        while j + 1 < sv.numel() and sv[j + 1] == sv[i]:
            j += 1
        ranks[order[i:j + 1]] = 0.5 * (i + j) + 1
        t = j - i + 1
        tie_term += t ** 3 - t
        i = j + 1
    nx, ny = x.numel(), y.numel()
    u = float(ranks[:nx].sum()) - nx * (nx + 1) / 2
    n = nx + ny
    sd = math.sqrt(nx * ny / 12 * ((n + 1) - tie_term / (n * (n - 1))))
    z = (u - nx * ny / 2 - math.copysign(0.5, u - nx * ny / 2)) / sd if sd > 0 else 0.0
    return TestResult(u, 2.0 * (1.0 - float(normal_cdf(abs(z)))))


# ------------------------------------------------------------------ survival analysis
def kaplan_meier(times, events):
    """-> [(time, at risk, events, survival, Greenwood standard error)] at the distinct event times."""
    t, e = _v(times), _v(events)
    out, s, gw = [], 1.0, 0.0
    for u in sorted({float(v) for v, d in zip(t, e) if d > 0}):
        at_risk = int((t >= u).sum())
        d = int(((t == u) & (e > 0)).sum())
        s *= 1 - d / at_risk
        gw += d / (at_risk * (at_risk - d)) if at_risk > d else 0.0
        out.append((u, at_risk, d, s, s * math.sqrt(gw)))
    return out


def nelson_aalen(times, events):
    t, e = _v(times), _v(events)
    out, h = [], 0.0
    for u in sorted({float(v) for v, d in zip(t, e) if d > 0}):
        at_risk = int((t >= u).sum())
        d = int(((t == u) & (e > 0)).sum())
        h += d / at_risk
        out.append((u, h))
    return out


def log_rank(times_a, events_a, times_b, events_b) -> TestResult:
    ta, ea, tb, eb = _v(times_a), _v(events_a), _v(times_b), _v(events_b)
    o_minus_e, var = 0.0, 0.0
    for u in sorted({float(v) for v, d in zip(torch.cat([ta, tb]), torch.cat([ea, eb])) if d > 0}):
        na, nb = int((ta >= u).sum()), int((tb >= u).sum())
        da, db = int(((ta == u) & (ea > 0)).sum()), int(((tb == u) & (eb > 0)).sum())
        n, d = na + nb, da + db
        o_minus_e += da - d * na / n
        if n > 1:
            var += d * (na / n) * (nb / n) * (n - d) / (n - 1)
    stat = o_minus_e ** 2 / var if var > 0 else 0.0
    return TestResult(stat, 1.0 - chi2_cdf(stat, 1), 1)


@dataclass
class CoxFit:
    coefficients: torch.Tensor
    standard_errors: torch.Tensor
    z: torch.Tensor
    p_values: torch.Tensor
    log_likelihood: float
    iterations: int
    converged: bool

    def hazard_ratios(self):
        return torch.exp(self.coefficients)


def cox_proportional_hazards(times, events, covariates, max_iter: int = 50, tol: float = 1e-10, ridge: float = 0.0) -> CoxFit:
    t, e = _v(times), _v(events)
    x = torch.as_tensor(covariates, dtype=D)
    x = x[:, None] if x.dim() == 1 else x
    if x.shape[0] != t.numel() or float(e.sum()) == 0:
        raise ValueError("one covariate row per observation and at least one event")
    order = torch.argsort(t, descending=True, stable=True)                    # risk set of i = everything sorted before or tied
    t, e, x = t[order], e[order], x[order]
    # Breslow ties: all observations with the same time share the risk set that includes the whole tie group
    last_of_tie = torch.tensor([i for i in range(t.numel()) if i + 1 == t.numel() or t[i + 1] != t[i]])
    group = torch.searchsorted(last_of_tie, torch.arange(t.numel()))
    idx = last_of_tie[group]
    beta = torch.zeros(x.shape[1], dtype=D)
    ll, it, converged = -math.inf, 0, False
    for it in range(1, max_iter + 1):
        eta = x @ beta
        w = torch.exp(eta - eta.max())
        s0 = torch.cumsum(w, 0)[idx]
        s1 = torch.cumsum(w[:, None] * x, 0)[idx]
        s2 = torch.cumsum(w[:, None, None] * x[:, :, None] * x[:, None, :], 0)[idx]
        mu = s1 / s0[:, None]
        grad = (e[:, None] * (x - mu)).sum(0) - ridge * beta
        info = (e[:, None, None] * (s2 / s0[:, None, None] - mu[:, :, None] * mu[:, None, :])).sum(0) + ridge * torch.eye(x.shape[1], dtype=D)
        new_ll = float((e * (eta - eta.max() - torch.log(s0))).sum())
        step = torch.linalg.solve(info, grad)
        beta = beta + step
        if abs(new_ll - ll) <= tol * (1 + abs(new_ll)) and float(step.abs().max()) < 1e-8:
            ll, converged = new_ll, True
            break
        ll = new_ll
    se = torch.sqrt(torch.diagonal(torch.linalg.inv(info)))
    z = beta / se
    p = torch.tensor([2.0 * (1.0 - float(normal_cdf(abs(float(v))))) for v in z], dtype=D)
    return CoxFit(beta, se, z, p, ll, it, converged)

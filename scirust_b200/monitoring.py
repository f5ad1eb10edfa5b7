"""Monitoring of processes and data streams: control charts, multivariate T^2, robust covariance, seasonal structure,
change points and remaining-useful-life extrapolation. The companion of ``mlops`` (population drift) for signals in time.

* ``ControlChart`` (Shewhart individuals / X-bar limits, Western Electric run rules), ``CusumChart`` (two one-sided
  tabular CUSUMs with reference value k and decision interval h, in sigma units), ``EwmaChart`` (exact time-varying
  limits), ``HotellingT2`` (Phase-II statistic with its F-based limit).
* ``mcd_covariance``: minimum covariance determinant: many random (d + 1)-subsets, concentration steps on ALL candidates
  at once (batched Mahalanobis distances and covariances), consistency-corrected; ``robust_mahalanobis`` flags outliers
  a classical covariance would mask.
* ``detect_period`` (autocorrelation peak confirmed by the periodogram), ``stl_decompose`` (iterated moving-average trend +
  per-phase seasonal medians, robust to isolated spikes), ``harmonic_fit`` (least-squares Fourier terms).
* ``cusum_change_points`` (binary segmentation on the CUSUM of residuals with a permutation-free significance bound) and
  ``page_hinkley`` (online mean-shift detector).
* ``health_index`` / ``estimate_rul``: monotone degradation trend and its crossing time of a failure threshold, with a
  residual-based interval.
Reference counterpart: scirust-spc/src/{shewhart,cusum,ewma,hotelling}.rs, scirust-multivariate/src/robust_geometry.rs,
scirust-seasonal/src/lib.rs, scirust-pdm/src/{change_detection,health,rul}.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .stats import chi2_cdf, f_cdf

D = torch.float64


def _v(x):
    return torch.as_tensor(x, dtype=D).reshape(-1)


# ------------------------------------------------------------------ univariate charts
@dataclass
class ControlChart:
    center: float
    sigma: float
    width: float = 3.0

    @staticmethod
    def from_individuals(x, width: float = 3.0) -> "ControlChart":
        """Sigma from the average moving range (divided by d2(2) = 1.128): insensitive to a slow drift in the phase-I data."""
        x = _v(x)
        return ControlChart(float(x.mean()), float((x[1:] - x[:-1]).abs().mean()) / 1.128, width)

    @staticmethod
    def from_subgroups(groups, width: float = 3.0) -> "ControlChart":
        g = torch.as_tensor(groups, dtype=D)
        n = g.shape[1]
        c4 = math.sqrt(2.0 / (n - 1)) * math.gamma(n / 2) / math.gamma((n - 1) / 2)
        return ControlChart(float(g.mean()), float(g.std(1).mean()) / c4 / math.sqrt(n), width)

    @property
    def ucl(self):
        return self.center + self.width * self.sigma

    @property
    def lcl(self):
        return self.center - self.width * self.sigma

    def out_of_control(self, x) -> list:
        x = _v(x)
        return torch.nonzero((x > self.ucl) | (x < self.lcl))[:, 0].tolist()

    def western_electric(self, x) -> dict:
        """Rule -> indices where it fires: 1 point beyond 3 sigma; 2 of 3 beyond 2 sigma (same side); 4 of 5 beyond 1
        sigma (same side); 8 in a row on one side."""
        z = ((_v(x) - self.center) / self.sigma).tolist()
        out = {1: [], 2: [], 3: [], 4: []}
        for i in range(len(z)):
            if abs(z[i]) > 3:
                out[1].append(i)
            for rule, span, need, lim in ((2, 3, 2, 2.0), (3, 5, 4, 1.0), (4, 8, 8, 0.0)):
                if i + 1 >= span:
                    w = z[i + 1 - span:i + 1]
                    for sgn in (1, -1):
                        if sum(sgn * v > lim for v in w) >= need and sgn * z[i] > lim:
                            out[rule].append(i)
                            break
        return out


class CusumChart:
    def __init__(self, target: float, sigma: float, k: float = 0.5, h: float = 5.0):
        self.target, self.sigma, self.k, self.h = target, sigma, k, h
        self.reset()

    def reset(self):
        self.hi = self.lo = 0.0

    def update(self, x: float):
        z = (x - self.target) / self.sigma
        self.hi = max(0.0, self.hi + z - self.k)
        self.lo = max(0.0, self.lo - z - self.k)
        return self.hi > self.h, self.lo > self.h

    def run(self, xs) -> list:
        """-> [(index, 'up' | 'down')]; the statistic restarts after each signal."""
        out = []
        for i, x in enumerate(_v(xs).tolist()):
            up, down = self.update(x)
            if up or down:
                out.append((i, "up" if up else "down"))
                self.reset()
        return out


class EwmaChart:
    def __init__(self, target: float, sigma: float, lam: float = 0.2, width: float = 3.0):
        self.target, self.sigma, self.lam, self.width = target, sigma, lam, width

    def run(self, xs):
        """-> (ewma values, half-widths of the limits, indices out of control)."""
        x = _v(xs)
        z, vals = self.target, []
        for v in x.tolist():
            z = self.lam * v + (1 - self.lam) * z
            vals.append(z)
        t = torch.arange(1, x.numel() + 1, dtype=D)
        half = self.width * self.sigma * torch.sqrt(self.lam / (2 - self.lam) * (1 - (1 - self.lam) ** (2 * t)))
        vals = torch.tensor(vals, dtype=D)
        return vals, half, torch.nonzero((vals - self.target).abs() > half)[:, 0].tolist()


class HotellingT2:
    def __init__(self, reference):
        x = torch.as_tensor(reference, dtype=D)
        self.n, self.p = x.shape
        if self.n <= self.p:
            raise ValueError("need more reference observations than variables")
        self.mean = x.mean(0)
        self.prec = torch.linalg.inv(torch.cov(x.t()).reshape(self.p, self.p))

    def statistic(self, x):
        d = torch.as_tensor(x, dtype=D).reshape(-1, self.p) - self.mean
        return ((d @ self.prec) * d).sum(1)

    def limit(self, alpha: float = 0.0027) -> float:
        """Phase-II limit p (n + 1)(n - 1) / (n (n - p)) F_{1 - alpha}(p, n - p), the quantile found by bisection."""
        lo, hi = 0.0, 1e4
        for _ in range(200):
            mid = 0.5 * (lo + hi)
            lo, hi = (mid, hi) if f_cdf(mid, self.p, self.n - self.p) < 1 - alpha else (lo, mid)
        return self.p * (self.n + 1) * (self.n - 1) / (self.n * (self.n - self.p)) * hi

    def out_of_control(self, x, alpha: float = 0.0027) -> list:
        return torch.nonzero(self.statistic(x) > self.limit(alpha))[:, 0].tolist()


# ------------------------------------------------------------------ robust covariance
def _chi2_ppf(p, k):
    lo, hi = 0.0, 1e4
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        lo, hi = (mid, hi) if chi2_cdf(mid, k) < p else (lo, mid)
    return hi


def mcd_covariance(x, coverage: float = 0.75, subsets: int = 300, c_steps: int = 8, seed: int = 0):
    """-> (location [d], covariance [d, d], inlier mask): covariance of the h = coverage * n points whose covariance has
    the smallest determinant (approximately: random starts + concentration), scaled to be consistent at the normal."""
    x = torch.as_tensor(x, dtype=D)
    n, d = x.shape
    h = max(int(math.ceil(coverage * n)), (n + d + 1) // 2)
    if n <= d + 1:
        raise ValueError("need more observations than dimensions + 1")
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(n, generator=g)[:d + 1] for _ in range(subsets)])
    eye = 1e-9 * torch.eye(d, dtype=D)

    def moments(sel):                                                         # sel [S, m] -> mean [S, d], cov [S, d, d]
        pts = x[sel]
        mu = pts.mean(1)
        c = pts - mu[:, None]
        return mu, c.transpose(1, 2) @ c / (sel.shape[1] - 1) + eye
    mu, cov = moments(idx)
    for _ in range(c_steps):
        diff = x[None] - mu[:, None]
        md = (torch.linalg.solve(cov, diff.transpose(1, 2)).transpose(1, 2) * diff).sum(2)      # [S, n]
        mu, cov = moments(md.topk(h, dim=1, largest=False).indices)
    best = int(torch.linalg.slogdet(cov)[1].argmin())
    mu, cov = mu[best], cov[best]
    diff = x - mu
    md = (torch.linalg.solve(cov, diff.t()).t() * diff).sum(1)
    cov = cov * (float(md.median()) / _chi2_ppf(0.5, d))                       # consistency: median distance = chi2 median
    md = (torch.linalg.solve(cov, diff.t()).t() * diff).sum(1)
    inl = md <= _chi2_ppf(0.975, d)
    if int(inl.sum()) > d + 1:                                                 # re-weighted estimate on the inliers
        mu = x[inl].mean(0)
        cov = torch.cov(x[inl].t()).reshape(d, d)
        diff = x - mu
        md = (torch.linalg.solve(cov, diff.t()).t() * diff).sum(1)
        inl = md <= _chi2_ppf(0.975, d)
    return mu, cov, inl


def robust_mahalanobis(x, **kw):
    x = torch.as_tensor(x, dtype=D)
    mu, cov, _ = mcd_covariance(x, **kw)
    diff = x - mu
    return torch.sqrt((torch.linalg.solve(cov, diff.t()).t() * diff).sum(1))


# ------------------------------------------------------------------ seasonal structure
def detect_period(x, min_period: int = 2, max_period: int | None = None):
    """-> (period, autocorrelation at that lag): the first local maximum of the autocorrelation of the detrended
    series above 0.3, checked against the periodogram's dominant frequency."""
    x = _v(x)
    n = x.numel()
    t = torch.arange(n, dtype=D)
    a = torch.stack([torch.ones(n, dtype=D), t], 1)
    r = x - a @ torch.linalg.lstsq(a, x[:, None]).solution[:, 0]
    r = r - r.mean()
    spec = torch.fft.rfft(r, n=2 * n)
    ac = torch.fft.irfft(spec * spec.conj(), n=2 * n)[:n]
    ac = ac / ac[0].clamp_min(1e-300)
    max_period = max_period or n // 2
    best = None
    for lag in range(max(min_period, 2), max_period):
        if ac[lag] > 0.3 and ac[lag] >= ac[lag - 1] and ac[lag] >= ac[lag + 1]:
            best = lag
            break
    if best is None:
        return None, 0.0
    power = torch.fft.rfft(r).abs() ** 2
    k = int(power[1:].argmax()) + 1
    freq_period = n / k
    if abs(freq_period - best) > 0.25 * best and abs(freq_period - best / 2) > 0.25 * best:
        # the periodogram disagrees: prefer its period when a harmonic relation does not explain the gap
        cand = int(round(freq_period))
        if min_period <= cand < max_period and ac[cand] > 0.3:
            best = cand
    return best, float(ac[best])


def _moving_average(x, k):
    """Centred moving average of length k (2 x k for even k), edges filled by shrinking the window."""
    n = x.numel()
    c = torch.cat([torch.zeros(1, dtype=D), torch.cumsum(x, 0)])
    half = k // 2
    lo = (torch.arange(n) - half).clamp(0, n)
    hi = (torch.arange(n) + half + 1).clamp(0, n)
    out = (c[hi] - c[lo]) / (hi - lo).to(D)
    if k % 2 == 0:                                                            # even window: average two adjacent windows
        lo2, hi2 = (lo + 1).clamp(0, n), (hi - 1).clamp(0, n)
        full = (hi - lo) == k + 1
        alt = ((c[hi] - c[lo]) - 0.5 * x[lo.clamp(max=n - 1)] - 0.5 * x[(hi - 1).clamp(0, n - 1)]) / k
        out = torch.where(full, alt, out)
    return out


def stl_decompose(x, period: int, iterations: int = 2):
    """-> (trend, seasonal, residual) with trend + seasonal + residual = x. The seasonal component is the per-phase
    MEDIAN of the detrended series (robust to spikes), centred to sum to zero over a period."""
    x = _v(x)
    n = x.numel()
    if period < 2 or n < 2 * period:
        raise ValueError("need at least two full periods")
    seasonal = torch.zeros(n, dtype=D)
    trend = _moving_average(x, period)
    for _ in range(iterations):
        det = x - trend
        phase = torch.arange(n) % period
        med = torch.stack([det[phase == p].median() for p in range(period)])
        med = med - med.mean()
        seasonal = med[phase]
        trend = _moving_average(x - seasonal, period)
    return trend, seasonal, x - trend - seasonal


def harmonic_fit(x, period: float, harmonics: int = 3):
    """Least-squares mean + linear trend + Fourier terms -> (fitted values, amplitudes per harmonic)."""
    x = _v(x)
    t = torch.arange(x.numel(), dtype=D)
    cols = [torch.ones_like(t), t]
    for k in range(1, harmonics + 1):
        w = 2 * math.pi * k * t / period
        cols += [torch.cos(w), torch.sin(w)]
    a = torch.stack(cols, 1)
    beta = torch.linalg.lstsq(a, x[:, None]).solution[:, 0]
    return a @ beta, [float(torch.hypot(beta[2 * k], beta[2 * k + 1])) for k in range(1, harmonics + 1)]


# ------------------------------------------------------------------ change points
def cusum_change_points(x, min_size: int = 10, threshold: float = 1.36, max_points: int = 10) -> list:
    """Mean-shift change points by binary segmentation: inside a segment the statistic max |S_k| / (sigma sqrt(n)) of the
    centred cumulative sum is compared with the Kolmogorov bound (1.36 ~ 5 %); the split is at the arg max."""
    x = _v(x)
    sigma = float(1.4826 * ((x[1:] - x[:-1]) - (x[1:] - x[:-1]).median()).abs().median() / math.sqrt(2)) or 1e-12
    out = []

    def split(lo, hi):
        n = hi - lo
        if n < 2 * min_size or len(out) >= max_points:
            return
        seg = x[lo:hi]
        s = torch.cumsum(seg - seg.mean(), 0)[min_size - 1:n - min_size]
        if s.numel() == 0:
            return
        k = int(s.abs().argmax())
        if float(s.abs()[k]) / (sigma * math.sqrt(n)) > threshold:
            cp = lo + min_size + k
            out.append(cp)
            split(lo, cp)
            split(cp, hi)
    split(0, x.numel())
    return sorted(out)


def page_hinkley(xs, delta: float = 0.05, lam: float = 5.0):
    """Online upward mean-shift detector -> index of the first alarm or None."""
    mean, m, mn = 0.0, 0.0, 0.0
    for i, v in enumerate(_v(xs).tolist(), 1):
        mean += (v - mean) / i
        m += v - mean - delta
        mn = min(mn, m)
        if m - mn > lam:
            return i - 1
    return None


# ------------------------------------------------------------------ degradation and remaining useful life
def health_index(features, healthy: int) -> torch.Tensor:
    """Distance of every sample from the healthy baseline (first ``healthy`` rows) in baseline standard deviations,
    averaged over features, then made monotone (a running maximum: damage does not heal)."""
    f = torch.as_tensor(features, dtype=D)
    f = f[:, None] if f.dim() == 1 else f
    base = f[:healthy]
    z = ((f - base.mean(0)) / base.std(0).clamp_min(1e-12)).abs().mean(1)
    return torch.cummax(z, 0).values


def estimate_rul(health, threshold: float, window: int = 30, model: str = "linear"):
    """Fit the last ``window`` points (``linear`` or ``exponential`` in time), extrapolate to ``threshold`` ->
    (remaining steps, lower, upper) from the fit's residual spread; (inf, inf, inf) when the trend does not rise."""
    h = _v(health)
    w = min(window, h.numel())
    y = h[-w:]
    if model == "exponential":
        y = torch.log(y.clamp_min(1e-12))
        threshold = math.log(threshold)
    t = torch.arange(w, dtype=D)
    a = torch.stack([torch.ones(w, dtype=D), t], 1)
    beta = torch.linalg.lstsq(a, y[:, None]).solution[:, 0]
    b0, b1 = float(beta[0]), float(beta[1])
    if b1 <= 1e-12:
        return math.inf, math.inf, math.inf
    resid = float((y - a @ beta).std()) if w > 2 else 0.0
    cross = lambda level: max(0.0, (level - b0) / b1 - (w - 1))
    return cross(threshold), cross(threshold - 2 * resid), cross(threshold + 2 * resid)

"""Regression beyond least squares.

* ``KernelRidgeRegression``: ``alpha = (K + lambda I)^-1 y`` by Cholesky, kernels rbf / polynomial / linear.
* ``fit_robust_regression``: M-estimation by iteratively re-weighted least squares with Huber, Tukey bisquare or Cauchy
  weights and the MAD residual scale (re-estimated every iteration), intercept included.
* ``fit_high_breakdown``: least trimmed squares: many random elemental subsets are solved as ONE batched system, each
  candidate is refined by concentration steps (refit on the h smallest residuals) and the best trimmed objective wins;
  tolerates just under 50 % contamination. Outliers are flagged by scaled residual.
* ``IsotonicRegression``: pool-adjacent-violators with weights, interpolating prediction, increasing or decreasing.
* ``fit_quantile_regression``: pinball loss by IRLS on a smoothed absolute value.
* ``fit_multi_output_robust``: one weight per ROW from the norm of its residual vector (an outlying observation is
  down-weighted in every output together).
* ``influence_report``: leverage, internally / externally studentised residuals, Cook's distance, DFFITS, with the usual
  cut-offs, computed from one QR factorisation.
Reference counterpart: scirust-learning/src/{kernel_ridge,robust_regression,high_breakdown,isotonic,quantile_regression,
multi_output,influence}.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

D = torch.float64


def _xy(x, y=None):
    x = torch.as_tensor(x, dtype=D)
    x = x[:, None] if x.dim() == 1 else x
    if y is None:
        return x
    y = torch.as_tensor(y, dtype=D, device=x.device)
    if y.shape[0] != x.shape[0]:
        raise ValueError("x and y differ in the number of observations")
    return x, y


def _design(x):
    return torch.cat([torch.ones(x.shape[0], 1, dtype=D, device=x.device), x], 1)


def _wls(a, y, w):
    sw = w.sqrt()
    return torch.linalg.lstsq(a * sw[:, None], (y * (sw if y.dim() == 1 else sw[:, None]))).solution


@dataclass
class LinearModel:
    intercept: torch.Tensor
    coefficients: torch.Tensor

    def predict(self, x):
        return _xy(x).to(self.coefficients.device) @ self.coefficients + self.intercept


# ------------------------------------------------------------------ kernel ridge
class KernelRidgeRegression:
    def __init__(self, kernel: str = "rbf", gamma: float = 1.0, degree: int = 3, coef0: float = 1.0, ridge: float = 1e-3):
        if ridge <= 0:
            raise ValueError("the ridge must be positive")
        self.kernel, self.gamma, self.degree, self.coef0, self.ridge = kernel, gamma, degree, coef0, ridge
        self.x = self.alpha = None

    def _k(self, a, b):
        if self.kernel == "linear":
            return a @ b.t()
        if self.kernel == "poly":
            return (self.gamma * (a @ b.t()) + self.coef0) ** self.degree
        if self.kernel == "rbf":
            return torch.exp(-self.gamma * torch.cdist(a, b) ** 2)
        raise ValueError(f"unknown kernel {self.kernel!r}")

    def fit(self, x, y):
        x, y = _xy(x, y)
        k = self._k(x, x) + self.ridge * torch.eye(x.shape[0], dtype=D, device=x.device)
        l, info = torch.linalg.cholesky_ex(k)
        if int(info):
            raise ValueError("the regularised kernel matrix is not positive-definite")
        self.x, self.alpha = x, torch.cholesky_solve(y.reshape(x.shape[0], -1), l).reshape(y.shape)
        return self

    def predict(self, x):
        if self.x is None:
            raise ValueError("fit first")
        return self._k(_xy(x).to(self.x.device), self.x) @ self.alpha

    def support_len(self) -> int:
        return 0 if self.x is None else self.x.shape[0]


# ------------------------------------------------------------------ M-estimation
def mad_scale(r):
    """Median absolute deviation scaled to be consistent for the normal distribution."""
    return 1.4826 * (r - r.median()).abs().median()


def _weights(u, loss: str, c: float):
    a = u.abs()
    if loss == "huber":
        return torch.where(a <= c, torch.ones_like(a), c / a.clamp_min(1e-300))
    if loss == "tukey":
        return torch.where(a <= c, (1 - (u / c) ** 2) ** 2, torch.zeros_like(a))
    if loss == "cauchy":
        return 1.0 / (1.0 + (u / c) ** 2)
    raise ValueError(f"unknown loss {loss!r}")


TUNING = {"huber": 1.345, "tukey": 4.685, "cauchy": 2.385}                      # 95 % efficiency at the normal model


@dataclass
class RobustReport:
    model: LinearModel
    scale: float
    weights: torch.Tensor
    iterations: int
    converged: bool
    outliers: list = field(default_factory=list)


def fit_robust_regression(x, y, loss: str = "huber", tuning: float | None = None, max_iter: int = 100, tol: float = 1e-10,
                          start: torch.Tensor | None = None) -> RobustReport:
    x, y = _xy(x, y)
    a = _design(x)
    if a.shape[0] <= a.shape[1]:
        raise ValueError("need more observations than parameters")
    c = tuning or TUNING[loss]
    beta = torch.linalg.lstsq(a, y[:, None]).solution[:, 0] if start is None else start.clone()
    w = torch.ones_like(y)
    it, converged, s = 0, False, torch.tensor(1.0, dtype=D)
    for it in range(1, max_iter + 1):
        r = y - a @ beta
        s = mad_scale(r).clamp_min(1e-12)
        w = _weights(r / s, loss, c)
        if float(w.sum()) < a.shape[1]:
            break
        new = _wls(a, y, w)
        delta = float((new - beta).abs().max())
        beta = new
        if delta <= tol * (1 + float(beta.abs().max())):
            converged = True
            break
    r = y - a @ beta
    flagged = torch.nonzero((r / s).abs() > 2.5)[:, 0].tolist()
    return RobustReport(LinearModel(beta[0], beta[1:]), float(s), w, it, converged, flagged)


# ------------------------------------------------------------------ least trimmed squares
@dataclass
class HighBreakdownReport:
    model: LinearModel
    scale: float
    objective: float
    inliers: torch.Tensor
    outliers: list

    def predict(self, x):
        return self.model.predict(x)


def fit_high_breakdown(x, y, coverage: float = 0.5, subsets: int = 500, c_steps: int = 10, seed: int = 0,
                       refine: bool = True) -> HighBreakdownReport:
    x, y = _xy(x, y)
    a = _design(x)
    n, p = a.shape
    h = max(int(math.ceil(coverage * n)), (n + p + 1) // 2)
    if n <= p or h > n:
        raise ValueError("not enough observations")
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(n, generator=g)[:p] for _ in range(subsets)]).to(a.device)      # [S, p]
    sub_a, sub_y = a[idx], y[idx]
    beta = torch.linalg.lstsq(sub_a, sub_y[..., None]).solution[..., 0]                                 # [S, p]
    for _ in range(c_steps):
        r2 = (y[None, :] - beta @ a.t()) ** 2                                                           # [S, n]
        keep = r2.topk(h, dim=1, largest=False).indices                                                 # [S, h]
        beta = torch.linalg.lstsq(a[keep], y[keep][..., None]).solution[..., 0]
    r2 = (y[None, :] - beta @ a.t()) ** 2
    obj = r2.topk(h, dim=1, largest=False).values.sum(1)
    obj = torch.where(torch.isfinite(obj), obj, torch.full_like(obj, math.inf))
    best = int(obj.argmin())
    b = beta[best]
    r = y - a @ b
    # consistency factor of the trimmed variance at the normal model
    q = _norm_ppf((1 + h / n) / 2)
    cons = 1.0 / math.sqrt(max(1e-12, 1 - 2 * n / h * q * _norm_pdf(q))) if h < n else 1.0
    s = cons * math.sqrt(float(obj[best]) / h)
    inl = (r / max(s, 1e-12)).abs() <= 2.5
    if refine and int(inl.sum()) > p:                                          # re-weighted step: plain LS on the inliers
        b = torch.linalg.lstsq(a[inl], y[inl][:, None]).solution[:, 0]
        r = y - a @ b
        s = math.sqrt(float((r[inl] ** 2).sum()) / max(1, int(inl.sum()) - p))
        inl = (r / max(s, 1e-12)).abs() <= 2.5
    return HighBreakdownReport(LinearModel(b[0], b[1:]), s, float(obj[best]), inl, torch.nonzero(~inl)[:, 0].tolist())


def _norm_pdf(z):
    return math.exp(-0.5 * z * z) / math.sqrt(2 * math.pi)


def _norm_ppf(p):
    from ..numerics.special import inv_normal_cdf
    return float(inv_normal_cdf(p))


# ------------------------------------------------------------------ isotonic
class IsotonicRegression:
    def __init__(self, increasing: bool = True):
        self.increasing = increasing
        self.knots_x = self.knots_y = None

    def fit(self, x, y, weights=None):
        x = torch.as_tensor(x, dtype=D).reshape(-1)
        y = torch.as_tensor(y, dtype=D).reshape(-1)
        if x.numel() != y.numel() or x.numel() == 0:
            raise ValueError("x and y need the same non-zero length")
        w = torch.ones_like(y) if weights is None else torch.as_tensor(weights, dtype=D).reshape(-1)
        if bool((w <= 0).any()) or not bool(torch.isfinite(x).all() and torch.isfinite(y).all()):
            raise ValueError("weights must be positive and data finite")
        order = torch.argsort(x, stable=True)
        xs, ys, ws = x[order].tolist(), (y[order] if self.increasing else -y[order]).tolist(), w[order].tolist()
        blocks = []                                                           # [sum w*y, sum w, x_lo, x_hi]
        for xi, yi, wi in zip(xs, ys, ws):
            if blocks and blocks[-1][3] == xi:                                # ties in x pool before the order constraint
                blocks[-1][0] += wi * yi
                blocks[-1][1] += wi
            else:
                blocks.append([wi * yi, wi, xi, xi])
            while len(blocks) > 1 and blocks[-2][0] / blocks[-2][1] > blocks[-1][0] / blocks[-1][1]:
                b = blocks.pop()
                blocks[-1][0] += b[0]
                blocks[-1][1] += b[1]
                blocks[-1][3] = b[3]
        kx, ky = [], []
        for s, wt, lo, hi in blocks:
            v = s / wt if self.increasing else -s / wt
            kx.append(lo)
            ky.append(v)
            if hi != lo:
                kx.append(hi)
                ky.append(v)
        self.knots_x, self.knots_y = torch.tensor(kx, dtype=D), torch.tensor(ky, dtype=D)
        return self

    def knots(self):
        return self.knots_x, self.knots_y

    def predict(self, x):
        if self.knots_x is None:
            raise ValueError("fit first")
        q = torch.as_tensor(x, dtype=D)
        kx, ky = self.knots_x, self.knots_y
        if kx.numel() == 1:
            return ky[0].expand_as(q).clone()
        i = torch.searchsorted(kx, q.reshape(-1).contiguous()).clamp(1, kx.numel() - 1)
        x0, x1, y0, y1 = kx[i - 1], kx[i], ky[i - 1], ky[i]
        t = ((q.reshape(-1) - x0) / (x1 - x0).clamp_min(1e-300)).clamp(0, 1)
        return (y0 + t * (y1 - y0)).reshape(q.shape)


# ------------------------------------------------------------------ quantile regression
@dataclass
class QuantileReport:
    model: LinearModel
    tau: float
    pinball_loss: float
    iterations: int
    converged: bool


def pinball(r, tau):
    return torch.where(r >= 0, tau * r, (tau - 1) * r).mean()


def fit_quantile_regression(x, y, tau: float = 0.5, max_iter: int = 200, tol: float = 1e-9, eps: float = 1e-6) -> QuantileReport:
    if not 0 < tau < 1:
        raise ValueError("0 < tau < 1")
    x, y = _xy(x, y)
    a = _design(x)
    beta = torch.linalg.lstsq(a, y[:, None]).solution[:, 0]
    it, converged = 0, False
    for it in range(1, max_iter + 1):
        r = y - a @ beta
        w = torch.where(r >= 0, tau, 1 - tau) / r.abs().clamp_min(eps)
        new = _wls(a, y, w)
        delta = float((new - beta).abs().max())
        beta = new
        if delta <= tol * (1 + float(beta.abs().max())):
            converged = True
            break
    return QuantileReport(LinearModel(beta[0], beta[1:]), tau, float(pinball(y - a @ beta, tau)), it, converged)


# ------------------------------------------------------------------ multi-output robust
@dataclass
class MultiOutputReport:
    intercept: torch.Tensor
    coefficients: torch.Tensor
    scale: float
    weights: torch.Tensor
    iterations: int
    converged: bool

    def predict(self, x):
        return _xy(x) @ self.coefficients + self.intercept


def fit_multi_output_robust(x, y, loss: str = "huber", tuning: float | None = None, max_iter: int = 100,
                            tol: float = 1e-10) -> MultiOutputReport:
    x, y = _xy(x, y)
    if y.dim() != 2:
        raise ValueError("y must be [observations, outputs]")
    a = _design(x)
    m = y.shape[1]
    c = (tuning or TUNING[loss]) * math.sqrt(m)                               # row norms of m unit normals grow like sqrt(m)
    beta = torch.linalg.lstsq(a, y).solution
    w = torch.ones(a.shape[0], dtype=D)
    it, converged, s = 0, False, torch.tensor(1.0, dtype=D)
    for it in range(1, max_iter + 1):
        r = y - a @ beta
        s = mad_scale(r.reshape(-1)).clamp_min(1e-12)
        w = _weights(r.norm(dim=1) / s, loss, c)
        new = _wls(a, y, w)
        delta = float((new - beta).abs().max())
        beta = new
        if delta <= tol * (1 + float(beta.abs().max())):
            converged = True
            break
    return MultiOutputReport(beta[0], beta[1:], float(s), w, it, converged)


# ------------------------------------------------------------------ influence diagnostics
@dataclass
class InfluenceReport:
    leverage: torch.Tensor
    residuals: torch.Tensor
    studentized_internal: torch.Tensor
    studentized_external: torch.Tensor
    cooks_distance: torch.Tensor
    dffits: torch.Tensor
    high_leverage: list
    outliers: list
    influential: list

    def count(self, kind: str) -> int:
        return len({"leverage": self.high_leverage, "outlier": self.outliers, "influential": self.influential}[kind])


def influence_report(x, y) -> InfluenceReport:
    x, y = _xy(x, y)
    a = _design(x)
    n, p = a.shape
    if n <= p + 1:
        raise ValueError("need at least p + 2 observations")
    q, _ = torch.linalg.qr(a)
    h = (q * q).sum(1).clamp(max=1 - 1e-12)
    r = y - q @ (q.t() @ y)
    s2 = float((r * r).sum()) / (n - p)
    t_int = r / torch.sqrt(s2 * (1 - h))
    s2_i = ((n - p) * s2 - r * r / (1 - h)) / (n - p - 1)
    t_ext = r / torch.sqrt(s2_i.clamp_min(1e-300) * (1 - h))
    cook = t_int ** 2 * h / ((1 - h) * p)
    dffits = t_ext * torch.sqrt(h / (1 - h))
    return InfluenceReport(h, r, t_int, t_ext, cook, dffits,
                           torch.nonzero(h > 2 * p / n)[:, 0].tolist(), torch.nonzero(t_ext.abs() > 3)[:, 0].tolist(),
                           torch.nonzero((cook > 4 / n) | (dffits.abs() > 2 * math.sqrt(p / n)))[:, 0].tolist())

"""Univariate forecasting: exponential smoothing (simple, Holt's linear trend, additive Holt-Winters), autoregression
by least squares, ARIMA(p, d, q) by the Hannan-Rissanen two-stage regression (a long AR supplies innovations, then
``y_t`` is regressed on its own lags and on lagged innovations), differencing helpers and the usual error metrics.
Smoothing parameters left as ``None`` are chosen on a grid by one-step-ahead squared error.
Reference counterpart: scirust-forecast/src/{smoothing,autoreg,arima,metrics,utils}.rs."""
from __future__ import annotations

import itertools
import math

import torch

D = torch.float64


def _series(y):
    y = torch.as_tensor(y, dtype=D).reshape(-1)
    if not bool(torch.isfinite(y).all()):
        raise ValueError("the series must be finite")
    return y


# ------------------------------------------------------------------ metrics
def mae(a, f):
    return float((_series(a) - _series(f)).abs().mean())


def rmse(a, f):
    return float(((_series(a) - _series(f)) ** 2).mean().sqrt())


def mape(a, f):
    a, f = _series(a), _series(f)
    return float(((a - f) / a).abs().mean() * 100)


def smape(a, f):
    a, f = _series(a), _series(f)
    return float((2 * (a - f).abs() / (a.abs() + f.abs()).clamp_min(1e-300)).mean() * 100)


def mase(a, f, train, season: int = 1):
    tr = _series(train)
    scale = float((tr[season:] - tr[:-season]).abs().mean())
    return mae(a, f) / scale


def difference(y, d: int = 1):
    y = _series(y)
    for _ in range(d):
        y = y[1:] - y[:-1]
    return y


def undifference(forecast, history, d: int = 1):
    """Integrate a forecast of the d-times differenced series back to the level of ``history``."""
    f = _series(forecast)
    tails = [_series(history)]
    for _ in range(d - 1):
        tails.append(tails[-1][1:] - tails[-1][:-1])
    for level in reversed(tails[:d]):
        f = level[-1] + torch.cumsum(f, 0)
    return f


# ------------------------------------------------------------------ exponential smoothing
class ExponentialSmoothing:
    """``trend`` / ``season`` switch Holt's and Holt-Winters' additive components on; state after ``fit`` = last level,
    trend and the last ``season`` seasonal terms."""

    def __init__(self, alpha=None, beta=None, gamma=None, trend: bool = False, season: int = 0):
        self.alpha, self.beta, self.gamma, self.trend, self.season = alpha, beta, gamma, trend, season

    def _run(self, y, a, b, g):
        m = self.season
        if m:
            level = float(y[:m].mean())
            seas = [float(v) - level for v in y[:m]]
            tr = float((y[m:2 * m].mean() - y[:m].mean()) / m) if self.trend and len(y) >= 2 * m else 0.0
        else:
            level, seas = float(y[0]), []
            tr = float(y[1] - y[0]) if self.trend and len(y) > 1 else 0.0
        sse, start = 0.0, (m if m else 1)
        for t in range(start, len(y)):
            s = seas[t % m] if m else 0.0
            pred = level + (tr if self.trend else 0.0) + s
            v = float(y[t])
            sse += (v - pred) ** 2
            new_level = a * (v - s) + (1 - a) * (level + (tr if self.trend else 0.0))
            if self.trend:
                tr = b * (new_level - level) + (1 - b) * tr
            if m:
                seas[t % m] = g * (v - new_level) + (1 - g) * s
            level = new_level
        return sse, level, tr, seas

    def fit(self, y):
        y = _series(y)
        if len(y) < max(2, 2 * self.season):
            raise ValueError("the series is too short")
        grid = [0.05, 0.1, 0.2, 0.3, 0.5, 0.7, 0.9]
        choices = itertools.product([self.alpha] if self.alpha is not None else grid,
                                    [self.beta] if self.beta is not None or not self.trend else grid,
                                    [self.gamma] if self.gamma is not None or not self.season else grid)
        best = None
        for a, b, g in choices:
            res = self._run(y, a, b or 0.0, g or 0.0)
            if best is None or res[0] < best[0][0]:
                best = (res, (a, b, g))
        (self.sse, self.level, self.slope, self.seasonal), (self.alpha, self.beta, self.gamma) = best
        self.n = len(y)
        return self

    def forecast(self, steps: int):
        out = []
        for h in range(1, steps + 1):
            s = self.seasonal[(self.n + h - 1) % self.season] if self.season else 0.0
            out.append(self.level + (h * self.slope if self.trend else 0.0) + s)
        return torch.tensor(out, dtype=D)


# ------------------------------------------------------------------ AR / ARIMA
def _lagged(y, lags, start):
    return torch.stack([y[start - k:len(y) - k] for k in range(1, lags + 1)], 1) if lags else torch.zeros(len(y) - start, 0, dtype=D)


class AutoRegression:
    def __init__(self, order: int):
        if order < 1:
            raise ValueError("order >= 1")
        self.p = order

    def fit(self, y):
        y = _series(y)
        if len(y) <= 2 * self.p + 1:
            raise ValueError("the series is too short for this order")
        a = torch.cat([torch.ones(len(y) - self.p, 1, dtype=D), _lagged(y, self.p, self.p)], 1)
        beta = torch.linalg.lstsq(a, y[self.p:, None]).solution[:, 0]
        self.intercept, self.coefficients = float(beta[0]), beta[1:]
        r = y[self.p:] - a @ beta
        self.sigma2 = float((r * r).mean())
        self.history = y
        return self

    def forecast(self, steps: int):
        h = self.history.tolist()
        for _ in range(steps):
            h.append(self.intercept + sum(float(c) * h[-k - 1] for k, c in enumerate(self.coefficients)))
        return torch.tensor(h[-steps:], dtype=D)

    def aic(self) -> float:
        n = len(self.history) - self.p
        return n * math.log(self.sigma2) + 2 * (self.p + 1)


class Arima:
    def __init__(self, p: int, d: int, q: int):
        if min(p, d, q) < 0 or p + q == 0:
            raise ValueError("orders are non-negative and p + q > 0")
        self.p, self.d, self.q = p, d, q

    def fit(self, y):
        self.original = _series(y)
        z = difference(self.original, self.d)
        p, q = self.p, self.q
        long = min(max(p + q + 4, 8), len(z) // 3)
        if len(z) <= long + p + q + 2:
            raise ValueError("the series is too short for these orders")
        e = torch.zeros_like(z)
        if q:
            ar = AutoRegression(long).fit(z)
            a = torch.cat([torch.ones(len(z) - long, 1, dtype=D), _lagged(z, long, long)], 1)
            e[long:] = z[long:] - a @ torch.cat([torch.tensor([ar.intercept], dtype=D), ar.coefficients])
        start = (long + q) if q else p
        cols = [torch.ones(len(z) - start, 1, dtype=D), _lagged(z, p, start)]
        if q:
            cols.append(_lagged(e, q, start))
        a = torch.cat(cols, 1)
        beta = torch.linalg.lstsq(a, z[start:, None]).solution[:, 0]
        self.intercept, self.ar, self.ma = float(beta[0]), beta[1:1 + p], beta[1 + p:]
        res = z[start:] - a @ beta
        self.sigma2 = float((res * res).mean())
        self.z = z
        self.e = torch.cat([e[:start] * 0, res])
        return self

    def forecast(self, steps: int):
        z, e = self.z.tolist(), self.e.tolist()
        for _ in range(steps):
            v = self.intercept + sum(float(c) * z[-k - 1] for k, c in enumerate(self.ar)) + sum(float(c) * e[-k - 1] for k, c in enumerate(self.ma))
            z.append(v)
            e.append(0.0)
        f = torch.tensor(z[-steps:], dtype=D)
        return undifference(f, self.original, self.d) if self.d else f

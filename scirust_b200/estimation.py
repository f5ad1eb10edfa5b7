"""State estimation: extended and unscented Kalman filters, the Rauch-Tung-Striebel smoother, a bootstrap particle
filter and an interacting-multiple-model filter.

* ``ExtendedKalmanFilter``: the Jacobians of the user's transition and measurement functions come from autograd
  (``torch.func.jacrev``), so a model is written once as a plain function; Joseph-form covariance update.
* ``UnscentedKalmanFilter``: scaled sigma points (alpha, beta, kappa), no derivatives needed.
* ``rts_smoother``: backward pass over stored linear-filter results (smoothed means and covariances).
* ``ParticleFilter``: all particles are one tensor ``[particles, state]``; propagation and weighting are batched calls
  of the user's functions, systematic resampling when the effective sample size falls under a fraction of N: on a
  GPU tens of thousands of particles cost one kernel sequence per step.
* ``ImmFilter``: several linear models with a Markov switching matrix: mixing, per-model Kalman step, mode
  probabilities from the innovation likelihoods, moment-matched output.
Reference counterpart: scirust-estimation/src/{kalman,ekf,smoother,particle,imm}.rs and the unscented filter of
scirust-simd/src/dsp/kalman.rs.
"""
from __future__ import annotations

import math

import torch
from torch.func import jacrev

D = torch.float64


def _t(x):
    return torch.as_tensor(x, dtype=D)


def _joseph(p, k, h, r):
    ikh = torch.eye(p.shape[-1], dtype=D) - k @ h
    return ikh @ p @ ikh.t() + k @ r @ k.t()


class ExtendedKalmanFilter:
    def __init__(self, x0, p0):
        self.x, self.p = _t(x0).clone(), _t(p0).clone()

    def predict(self, f, q, *args):
        """``f(x, *args) -> x_next``; the Jacobian df/dx is taken at the current estimate."""
        fx = jacrev(lambda s: f(s, *args))(self.x)
        self.x = f(self.x, *args).detach()
        self.p = fx @ self.p @ fx.t() + _t(q)
        return self.x

    def update(self, z, h, r, *args):
        """``h(x, *args) -> expected measurement``. -> (innovation, innovation covariance)."""
        hx = jacrev(lambda s: h(s, *args))(self.x)
        r = _t(r)
        y = _t(z) - h(self.x, *args).detach()
        s = hx @ self.p @ hx.t() + r
        k = torch.linalg.solve(s, hx @ self.p).t()
        self.x = self.x + k @ y
        self.p = _joseph(self.p, k, hx, r)
        return y, s


class UnscentedKalmanFilter:
    def __init__(self, x0, p0, alpha: float = 1e-1, beta: float = 2.0, kappa: float = 0.0):
        self.x, self.p = _t(x0).clone(), _t(p0).clone()
        n = self.x.numel()
        lam = alpha * alpha * (n + kappa) - n
        self.scale = n + lam
        self.wm = torch.full((2 * n + 1,), 0.5 / self.scale, dtype=D)
        self.wc = self.wm.clone()
        self.wm[0] = lam / self.scale
        self.wc[0] = lam / self.scale + (1 - alpha * alpha + beta)

    def _sigma(self):
        l = torch.linalg.cholesky(self.scale * (0.5 * (self.p + self.p.t()) + 1e-12 * torch.eye(self.x.numel(), dtype=D)))
        return torch.cat([self.x[None], self.x[None] + l.t(), self.x[None] - l.t()])

    def predict(self, f, q, *args):
        pts = torch.stack([f(s, *args) for s in self._sigma()])
        self.x = self.wm @ pts
        d = pts - self.x
        self.p = (self.wc[:, None] * d).t() @ d + _t(q)
        return self.x

    def update(self, z, h, r, *args):
        sig = self._sigma()
        zs = torch.stack([h(s, *args) for s in sig])
        zm = self.wm @ zs
        dz, dx = zs - zm, sig - self.x
        s = (self.wc[:, None] * dz).t() @ dz + _t(r)
        c = (self.wc[:, None] * dx).t() @ dz
        k = torch.linalg.solve(s, c.t()).t()
        y = _t(z) - zm
        self.x = self.x + k @ y
        self.p = self.p - k @ s @ k.t()
        return y, s


def kalman_filter_sequence(zs, f, q, h, r, x0, p0):
    """Linear filter over a whole measurement sequence -> dict of predicted / filtered means and covariances, and the
    log-likelihood of the measurements."""
    f, q, h, r = _t(f), _t(q), _t(h), _t(r)
    x, p = _t(x0), _t(p0)
    out = {"xp": [], "pp": [], "xf": [], "pf": []}
    ll = 0.0
    for z in _t(zs):
        x, p = f @ x, f @ p @ f.t() + q
        out["xp"].append(x)
        out["pp"].append(p)
        y = z - h @ x
        s = h @ p @ h.t() + r
        k = torch.linalg.solve(s, h @ p).t()
        x, p = x + k @ y, _joseph(p, k, h, r)
        ll += float(-0.5 * (y @ torch.linalg.solve(s, y) + torch.logdet(s) + y.numel() * math.log(2 * math.pi)))
        out["xf"].append(x)
        out["pf"].append(p)
    res = {k_: torch.stack(v) for k_, v in out.items()}
    res["log_likelihood"] = ll
    return res


def rts_smoother(filtered: dict, f):
    """-> (smoothed means [T, n], smoothed covariances [T, n, n]) from ``kalman_filter_sequence`` output."""
    f = _t(f)
    xs, ps = filtered["xf"].clone(), filtered["pf"].clone()
    for t in range(xs.shape[0] - 2, -1, -1):
        c = torch.linalg.solve(filtered["pp"][t + 1], f @ filtered["pf"][t]).t()
        xs[t] = filtered["xf"][t] + c @ (xs[t + 1] - filtered["xp"][t + 1])
        ps[t] = filtered["pf"][t] + c @ (ps[t + 1] - filtered["pp"][t + 1]) @ c.t()
    return xs, ps


class ParticleFilter:
    def __init__(self, particles: torch.Tensor, resample_fraction: float = 0.5, seed: int = 0):
        self.x = _t(particles).clone()
        self.n = self.x.shape[0]
        self.logw = torch.full((self.n,), -math.log(self.n), dtype=D, device=self.x.device)
        self.frac = resample_fraction
        self.gen = torch.Generator(device="cpu").manual_seed(seed)
        self.resamples = 0

    def predict(self, propagate):
        """``propagate(particles [N, d], generator) -> particles`` (it adds its own process noise)."""
        self.x = propagate(self.x, self.gen)

    def update(self, log_likelihood):
        """``log_likelihood(particles [N, d]) -> [N]``. -> effective sample size before any resampling."""
        self.logw = self.logw + log_likelihood(self.x)
        self.logw = self.logw - torch.logsumexp(self.logw, 0)
        ess = float(1.0 / torch.exp(2 * self.logw).sum())
        if ess < self.frac * self.n:
            self._resample()
        return ess

    def _resample(self):
        w = torch.exp(self.logw)
        u = (torch.rand((), generator=self.gen, dtype=D) + torch.arange(self.n, dtype=D)) / self.n     # systematic
        idx = torch.searchsorted(torch.cumsum(w, 0).cpu(), u).clamp_max(self.n - 1).to(self.x.device)
        self.x = self.x[idx]
        self.logw = torch.full((self.n,), -math.log(self.n), dtype=D, device=self.x.device)
        self.resamples += 1

    def estimate(self):
        w = torch.exp(self.logw)
        mean = w @ self.x
        d = self.x - mean
        return mean, (w[:, None] * d).t() @ d


class ImmFilter:
    """Models share the measurement model ``(h, r)`` and differ in ``(f_i, q_i)``; ``transition[i, j]`` = P(i -> j)."""

    def __init__(self, models, transition, h, r, x0, p0, mode_probabilities=None):
        self.models = [(_t(f), _t(q)) for f, q in models]
        self.pi, self.h, self.r = _t(transition), _t(h), _t(r)
        m = len(self.models)
        self.mu = _t(mode_probabilities) if mode_probabilities is not None else torch.full((m,), 1.0 / m, dtype=D)
        self.xs = [_t(x0).clone() for _ in range(m)]
        self.ps = [_t(p0).clone() for _ in range(m)]

    def step(self, z):
        z = _t(z)
        m = len(self.models)
        cbar = self.pi.t() @ self.mu                                          # predicted mode probabilities
        mix = self.pi * self.mu[:, None] / cbar[None, :].clamp_min(1e-300)     # mix[i, j] = P(was i | now j)
        x0 = [sum(mix[i, j] * self.xs[i] for i in range(m)) for j in range(m)]
        p0 = [sum(mix[i, j] * (self.ps[i] + torch.outer(self.xs[i] - x0[j], self.xs[i] - x0[j])) for i in range(m)) for j in range(m)]
        like = torch.zeros(m, dtype=D)
        for j, (f, q) in enumerate(self.models):
            x, p = f @ x0[j], f @ p0[j] @ f.t() + q
            y = z - self.h @ x
            s = self.h @ p @ self.h.t() + self.r
            k = torch.linalg.solve(s, self.h @ p).t()
            self.xs[j], self.ps[j] = x + k @ y, _joseph(p, k, self.h, self.r)
            like[j] = torch.exp(-0.5 * (y @ torch.linalg.solve(s, y))) / torch.sqrt(torch.det(2 * math.pi * s))
        self.mu = like * cbar
        self.mu = self.mu / self.mu.sum().clamp_min(1e-300)
        return self.estimate()

    def estimate(self):
        x = sum(w * xi for w, xi in zip(self.mu, self.xs))
        p = sum(w * (pi + torch.outer(xi - x, xi - x)) for w, xi, pi in zip(self.mu, self.xs, self.ps))
        return x, p

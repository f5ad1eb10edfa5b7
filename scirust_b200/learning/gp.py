"""Gaussian-process regression with stationary kernels (RBF, Matern 3/2, Matern 5/2): Cholesky fit, predictive mean and
variance for a whole batch of query points, log marginal likelihood, and a small hyper-parameter search that maximises
it over a log-spaced grid (every grid point is one batched Cholesky).
Reference counterpart: scirust-gp/src/lib.rs (``Kernel``, ``Rbf``, ``Matern32``, ``Matern52``, ``GaussianProcess``)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

D = torch.float64


@dataclass(frozen=True)
class Rbf:
    length_scale: float = 1.0
    variance: float = 1.0

    def __call__(self, a, b):
        return self.variance * torch.exp(-0.5 * (torch.cdist(a, b) / self.length_scale) ** 2)


@dataclass(frozen=True)
class Matern32:
    length_scale: float = 1.0
    variance: float = 1.0

    def __call__(self, a, b):
        r = math.sqrt(3.0) * torch.cdist(a, b) / self.length_scale
        return self.variance * (1 + r) * torch.exp(-r)


@dataclass(frozen=True)
class Matern52:
    length_scale: float = 1.0
    variance: float = 1.0

    def __call__(self, a, b):
        r = math.sqrt(5.0) * torch.cdist(a, b) / self.length_scale
        return self.variance * (1 + r + r * r / 3) * torch.exp(-r)


def _x(x):
    x = torch.as_tensor(x, dtype=D)
    return x[:, None] if x.dim() == 1 else x


class GaussianProcess:
    def __init__(self, kernel=Rbf(), noise: float = 1e-6):
        if noise < 0:
            raise ValueError("the noise variance cannot be negative")
        self.kernel, self.noise = kernel, noise
        self.x = self.l = self.alpha = self.mean = None

    def fit(self, x, y):
        x = _x(x)
        y = torch.as_tensor(y, dtype=D, device=x.device).reshape(-1)
        if x.shape[0] != y.shape[0] or x.shape[0] == 0:
            raise ValueError("x and y need the same non-zero number of rows")
        self.mean = y.mean()
        k = self.kernel(x, x) + (self.noise + 1e-10) * torch.eye(x.shape[0], dtype=D, device=x.device)
        l, info = torch.linalg.cholesky_ex(k)
        if int(info):
            raise ValueError("the kernel matrix is not positive-definite; raise the noise")
        self.x, self.l, self.y = x, l, y
        self.alpha = torch.cholesky_solve((y - self.mean)[:, None], l)[:, 0]
        return self

    def predict_many(self, xq):
        """-> (mean [q], variance [q]) of the latent function at the query points."""
        if self.x is None:
            raise ValueError("fit first")
        xq = _x(xq).to(self.x.device)
        ks = self.kernel(xq, self.x)
        mean = ks @ self.alpha + self.mean
        v = torch.linalg.solve_triangular(self.l, ks.t(), upper=False)
        prior = self.kernel(xq[:1], xq[:1])[0, 0]
        return mean, (prior - (v * v).sum(0)).clamp_min(0.0)

    def predict(self, xq):
        m, v = self.predict_many(torch.as_tensor(xq, dtype=D).reshape(1, -1))
        return float(m[0]), float(v[0])

    def log_marginal_likelihood(self) -> float:
        n = self.x.shape[0]
        return float(-0.5 * (self.y - self.mean) @ self.alpha - torch.log(torch.diagonal(self.l)).sum() - 0.5 * n * math.log(2 * math.pi))

    @staticmethod
    def fit_best(x, y, kernel_type=Rbf, length_scales=None, noises=None):
        """Grid search on the log marginal likelihood -> the fitted process with the best (length scale, noise)."""
        x = _x(x)
        y = torch.as_tensor(y, dtype=D).reshape(-1)
        span = float((x.max(0).values - x.min(0).values).norm()) or 1.0
        length_scales = length_scales or [span * f for f in (0.01, 0.03, 0.1, 0.3, 1.0, 3.0)]
        noises = noises or [1e-6, 1e-4, 1e-2, 1e-1]
        var = float(y.var()) or 1.0
        best = None
        for ls in length_scales:
            for nz in noises:
                try:
                    gp = GaussianProcess(kernel_type(ls, var), nz * var).fit(x, y)
                except ValueError:
                    continue
                lml = gp.log_marginal_likelihood()
                if best is None or lml > best[0]:
                    best = (lml, gp)
        if best is None:
            raise ValueError("no hyper-parameter setting gave a positive-definite kernel matrix")
        return best[1]

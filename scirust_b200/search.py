"""Derivative-free search and self-organising maps (the reference CLI's ``evo``, ``cmaes`` and ``som`` commands;
scirust-cli/src/learning.rs). Deterministic in the seed; numpy only.

* ``evolution_strategy``: (mu + lambda) ES with one self-adapted step size per individual (log-normal mutation).
* ``cma_es``: covariance-matrix adaptation with rank-one and rank-mu updates and cumulative step-size control
  (Hansen's standard parameter settings).
* ``SelfOrganizingMap``: a rectangular Kohonen map with exponentially shrinking neighbourhood and learning rate.
"""
from __future__ import annotations

import math

import numpy as np


def sphere(x):
    return float(np.sum(x * x))


def rosenbrock(x):
    return float(np.sum(100.0 * (x[1:] - x[:-1] ** 2) ** 2 + (1.0 - x[:-1]) ** 2))


def rastrigin(x):
    return float(10.0 * len(x) + np.sum(x * x - 10.0 * np.cos(2 * math.pi * x)))


OBJECTIVES = {"sphere": sphere, "rosenbrock": rosenbrock, "rastrigin": rastrigin}


def evolution_strategy(f, dim: int, mu: int = 8, lam: int = 32, sigma0: float = 0.5, generations: int = 200, seed: int = 0):
    rng = np.random.default_rng(seed)
    tau = 1.0 / math.sqrt(2.0 * dim)
    pop = [(rng.uniform(-2, 2, dim), sigma0) for _ in range(mu)]
    fit = [f(x) for x, _ in pop]
    history = [min(fit)]
    for _ in range(generations):
        kids = []
        for _ in range(lam):
            x, s = pop[rng.integers(mu)]
            s2 = s * math.exp(tau * rng.standard_normal())
            kids.append((x + s2 * rng.standard_normal(dim), s2))
        allp = pop + kids
        allf = fit + [f(x) for x, _ in kids]
        order = np.argsort(allf, kind="stable")[:mu]
        pop, fit = [allp[i] for i in order], [allf[i] for i in order]
        history.append(fit[0])
    return pop[0][0], fit[0], history


def cma_es(f, dim: int, sigma0: float = 0.5, generations: int = 200, seed: int = 0, x0=None, popsize: int | None = None):
    rng = np.random.default_rng(seed)
    lam = popsize or 4 + int(3 * math.log(dim))
    mu = lam // 2
    w = math.log(mu + 0.5) - np.log(np.arange(1, mu + 1))
    w /= w.sum()
    mueff = 1.0 / np.sum(w * w)
    cc = (4 + mueff / dim) / (dim + 4 + 2 * mueff / dim)
    cs = (mueff + 2) / (dim + mueff + 5)
    c1 = 2 / ((dim + 1.3) ** 2 + mueff)
    cmu = min(1 - c1, 2 * (mueff - 2 + 1 / mueff) / ((dim + 2) ** 2 + mueff))
    damps = 1 + 2 * max(0.0, math.sqrt((mueff - 1) / (dim + 1)) - 1) + cs
    chi = math.sqrt(dim) * (1 - 1 / (4 * dim) + 1 / (21 * dim * dim))
    mean = np.array(x0, dtype=float) if x0 is not None else rng.uniform(-2, 2, dim)
    sigma, C = sigma0, np.eye(dim)
    pc, ps = np.zeros(dim), np.zeros(dim)
    best_x, best_f, history = mean.copy(), f(mean), []
    for g in range(generations):
        d2, B = np.linalg.eigh(C)
        D = np.sqrt(np.maximum(d2, 1e-20))
        z = rng.standard_normal((lam, dim))
        y = (z * D) @ B.T
        xs = mean + sigma * y
        fs = np.array([f(x) for x in xs])
        order = np.argsort(fs, kind="stable")
        if fs[order[0]] < best_f:
            best_f, best_x = float(fs[order[0]]), xs[order[0]].copy()
        history.append(best_f)
        ysel = y[order[:mu]]
        yw = w @ ysel
        mean = mean + sigma * yw
        inv_sqrt = (B / D) @ B.T
        ps = (1 - cs) * ps + math.sqrt(cs * (2 - cs) * mueff) * (inv_sqrt @ yw)
        hsig = np.linalg.norm(ps) / math.sqrt(1 - (1 - cs) ** (2 * (g + 1))) / chi < 1.4 + 2 / (dim + 1)
        pc = (1 - cc) * pc + (math.sqrt(cc * (2 - cc) * mueff) * yw if hsig else 0.0)
        C = ((1 - c1 - cmu) * C + c1 * (np.outer(pc, pc) + (0.0 if hsig else cc * (2 - cc)) * C)
             + cmu * (ysel.T * w) @ ysel)
        C = (C + C.T) / 2
        sigma *= math.exp((cs / damps) * (np.linalg.norm(ps) / chi - 1))
        if best_f < 1e-14:
            break
    return best_x, best_f, history


class SelfOrganizingMap:
    def __init__(self, rows: int, cols: int, dim: int, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.rows, self.cols = rows, cols
        self.w = rng.uniform(0, 1, (rows * cols, dim))
        self.grid = np.array([(r, c) for r in range(rows) for c in range(cols)], dtype=float)

    def bmu(self, x) -> int:
        return int(np.argmin(((self.w - x) ** 2).sum(1)))

    def fit(self, data, epochs: int = 20, lr0: float = 0.5, radius0: float | None = None, seed: int = 0):
        rng = np.random.default_rng(seed)
        radius0 = radius0 or max(self.rows, self.cols) / 2
        steps, t = epochs * len(data), 0
        for _ in range(epochs):
            for i in rng.permutation(len(data)):
                frac = t / max(steps - 1, 1)
                lr, rad = lr0 * math.exp(-3 * frac), max(radius0 * math.exp(-3 * frac), 0.5)
                b = self.bmu(data[i])
                h = np.exp(-((self.grid - self.grid[b]) ** 2).sum(1) / (2 * rad * rad))
                self.w += lr * h[:, None] * (data[i] - self.w)
                t += 1
        return self

    def quantization_error(self, data) -> float:
        return float(np.mean([np.sqrt(((self.w[self.bmu(x)] - x) ** 2).sum()) for x in data]))

    def topographic_error(self, data) -> float:
        """Share of samples whose best and second-best units are not grid neighbours."""
        bad = 0
        for x in data:
            d = ((self.w - x) ** 2).sum(1)
            a, b = np.argsort(d)[:2]
            bad += np.abs(self.grid[a] - self.grid[b]).max() > 1
        return bad / len(data)

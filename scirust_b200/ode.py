"""Initial-value solvers for vector systems ``y' = f(t, y)`` on tensors, explicit and stiff.

* ``dopri5``: adaptive Dormand-Prince 5(4) with a PI-free step controller, dense over the caller's output times by
  stepping exactly onto them.
* ``backward_euler``: L-stable, first order; each step solves ``y - h f(t + h, y) = y_n`` by Newton's method with the
  Jacobian from autograd (``torch.func.jacrev``), one LU per iteration.
* ``rosenbrock23``: the linearly implicit, L-stable 2(3) pair used by ``ode23s`` (Shampine-Reichelt): one Jacobian and one
  LU factorisation per step, three back-substitutions, embedded error estimate, adaptive step; no Newton iteration.
* ``backward_euler_dae``: semi-explicit index-1 systems ``M y' = f(t, y)`` with a (possibly singular) constant mass matrix.
All return a ``Solution`` with the accepted times, states and work counters. ``f`` takes ``(t: float, y: Tensor[n])`` and
returns ``Tensor[n]``; it must be written with torch operations for the implicit solvers.
Reference counterpart: scirust-stiff/src/lib.rs (``backward_euler``, ``backward_euler_dae``, ``rosenbrock23``) and
scirust-solvers/src/ode/{rk4,dopri5}.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch.func import jacrev

D = torch.float64


class OdeError(RuntimeError):
    pass


@dataclass
class Solution:
    t: list = field(default_factory=list)
    y: list = field(default_factory=list)
    steps: int = 0
    rejected: int = 0
    f_evals: int = 0
    jac_evals: int = 0

    def states(self) -> torch.Tensor:
        return torch.stack(self.y)

    def final(self) -> torch.Tensor:
        return self.y[-1]


def _y0(y0):
    return torch.as_tensor(y0, dtype=D).reshape(-1).clone()


_C = [0, 1 / 5, 3 / 10, 4 / 5, 8 / 9, 1, 1]
_A = [[], [1 / 5], [3 / 40, 9 / 40], [44 / 45, -56 / 15, 32 / 9], [19372 / 6561, -25360 / 2187, 64448 / 6561, -212 / 729],
      [9017 / 3168, -355 / 33, 46732 / 5247, 49 / 176, -5103 / 18656], [35 / 384, 0, 500 / 1113, 125 / 192, -2187 / 6784, 11 / 84]]
_B4 = [5179 / 57600, 0, 7571 / 16695, 393 / 640, -92097 / 339200, 187 / 2100, 1 / 40]


def dopri5(f, y0, t0: float, t1: float, rtol: float = 1e-8, atol: float = 1e-10, h0: float | None = None, max_steps: int = 1_000_000) -> Solution:
    y, t = _y0(y0), float(t0)
    sol = Solution([t], [y])
    h = h0 or (t1 - t0) / 100
    k1 = f(t, y)
    sol.f_evals += 1
    while (t1 - t) > 1e-14 * max(1.0, abs(t1)):
        h = min(h, t1 - t)
        k = [k1]
        for i in range(1, 7):
            k.append(f(t + _C[i] * h, y + h * sum(a * kj for a, kj in zip(_A[i], k))))
        sol.f_evals += 6
        y5 = y + h * sum(b * kj for b, kj in zip(_A[6] + [0], k))
        err = h * sum((b5 - b4) * kj for b5, b4, kj in zip(_A[6] + [0], _B4, k))
        scale = atol + rtol * torch.maximum(y.abs(), y5.abs())
        e = float((err / scale).pow(2).mean().sqrt())
        if e <= 1.0:
            t, y, k1 = t + h, y5, k[6]                                         # first-same-as-last
            sol.t.append(t)
            sol.y.append(y)
            sol.steps += 1
        else:
            sol.rejected += 1
        h *= min(5.0, max(0.2, 0.9 * e ** -0.2)) if e > 0 else 5.0
        if sol.steps + sol.rejected > max_steps:
            raise OdeError("too many steps")
    return sol


def backward_euler(f, y0, t0: float, t1: float, h: float, newton_tol: float = 1e-10, max_newton: int = 20) -> Solution:
    y, t = _y0(y0), float(t0)
    sol = Solution([t], [y])
    n = max(1, int(math.ceil((t1 - t0) / h - 1e-12)))
    h = (t1 - t0) / n
    eye = torch.eye(y.numel(), dtype=D)
    for _ in range(n):
        z = y.clone()
        for it in range(max_newton):
            g = z - h * f(t + h, z) - y
            jac = eye - h * jacrev(lambda v: f(t + h, v))(z)
            sol.f_evals += 1
            sol.jac_evals += 1
            dz = torch.linalg.solve(jac, -g)
            z = z + dz
            if float(dz.abs().max()) <= newton_tol * (1 + float(z.abs().max())):
                break
        else:
            raise OdeError(f"Newton's iteration did not converge at t = {t + h}")
        t, y = t + h, z
        sol.t.append(t)
        sol.y.append(y)
        sol.steps += 1
    return sol


def backward_euler_dae(f, mass, y0, t0: float, t1: float, h: float, newton_tol: float = 1e-10, max_newton: int = 30) -> Solution:
    """``M (y_{n+1} - y_n) / h = f(t_{n+1}, y_{n+1})``: rows of ``M`` that are zero are algebraic constraints; ``y0`` must
    satisfy them."""
    m = torch.as_tensor(mass, dtype=D)
    y, t = _y0(y0), float(t0)
    sol = Solution([t], [y])
    n = max(1, int(math.ceil((t1 - t0) / h - 1e-12)))
    h = (t1 - t0) / n
    for _ in range(n):
        z = y.clone()
        for it in range(max_newton):
            g = m @ (z - y) - h * f(t + h, z)
            jac = m - h * jacrev(lambda v: f(t + h, v))(z)
            sol.f_evals += 1
            sol.jac_evals += 1
            dz = torch.linalg.solve(jac, -g)
            z = z + dz
            if float(dz.abs().max()) <= newton_tol * (1 + float(z.abs().max())):
                break
        else:
            raise OdeError(f"Newton's iteration did not converge at t = {t + h}")
        t, y = t + h, z
        sol.t.append(t)
        sol.y.append(y)
        sol.steps += 1
    return sol


def rosenbrock23(f, y0, t0: float, t1: float, rtol: float = 1e-6, atol: float = 1e-9, h0: float | None = None, max_steps: int = 200_000) -> Solution:
    y, t = _y0(y0), float(t0)
    sol = Solution([t], [y])
    d = 1.0 / (2.0 + math.sqrt(2.0))
    e32 = 6.0 + math.sqrt(2.0)
    h = h0 or (t1 - t0) / 100
    eye = torch.eye(y.numel(), dtype=D)
    f0 = f(t, y)
    sol.f_evals += 1
    while (t1 - t) > 1e-14 * max(1.0, abs(t1)):
        h = min(h, t1 - t)
        jac = jacrev(lambda v: f(t, v))(y)
        sol.jac_evals += 1
        dt_ = 1e-7 * max(1.0, abs(t))                                          # df/dt by a forward difference
        ft = (f(t + dt_, y) - f0) / dt_
        sol.f_evals += 1
        while True:
            lu, piv = torch.linalg.lu_factor(eye - h * d * jac)
            solve = lambda b: torch.linalg.lu_solve(lu, piv, b[:, None])[:, 0]
            k1 = solve(f0 + h * d * ft)
            f1 = f(t + 0.5 * h, y + 0.5 * h * k1)
            k2 = solve(f1 - k1) + k1
            y_new = y + h * k2
            f2 = f(t + h, y_new)
            sol.f_evals += 2
            k3 = solve(f2 - e32 * (k2 - f1) - 2.0 * (k1 - f0) + h * d * ft)
            err = h / 6.0 * (k1 - 2.0 * k2 + k3)
            scale = atol + rtol * torch.maximum(y.abs(), y_new.abs())
            e = float((err / scale).abs().max())
            if e <= 1.0:
                break
            sol.rejected += 1
            h *= max(0.2, 0.9 * e ** (-1.0 / 3.0))
            if sol.steps + sol.rejected > max_steps or h < 1e-14 * max(1.0, abs(t)):
                raise OdeError(f"step size underflow at t = {t}")
        t, y, f0 = t + h, y_new, f2
        sol.t.append(t)
        sol.y.append(y)
        sol.steps += 1
        h *= min(5.0, max(0.2, 0.9 * e ** (-1.0 / 3.0))) if e > 0 else 5.0
        if sol.steps > max_steps:
            raise OdeError("too many steps")
    return sol

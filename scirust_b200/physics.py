"""Learning and checking mechanical systems: Hamiltonian and Lagrangian neural networks, variational mechanics from a
user-supplied Lagrangian / Hamiltonian, structure-preserving integrators, a physics-informed (PINN) solver for ODE / PDE
residuals, direct optimal control by single shooting, and conservation / consistency checks.

Derivatives are taken by automatic differentiation, batched with ``torch.func`` (``vmap`` over ``grad`` / ``hessian``), so a whole
batch of states costs a few fused passes on the device that holds the model:
* ``HamiltonianNetwork``: an MLP ``H(q, p)``; the learned vector field is ``(dH/dp, -dH/dq)``, symplectic by construction.
* ``LagrangianNetwork``: an MLP ``L(q, qdot)``; accelerations solve ``(d2L/dqdot2) qddot = dL/dq - (d2L/dqdot dq) qdot``.
* ``euler_lagrange_residual`` / ``hamiltonian_vector_field``: the same formulas for any differentiable callable.
* ``rk4_step``, ``leapfrog_step`` (Stoermer-Verlet for separable Hamiltonians), ``rollout``.
* ``PinnSolver``: minimises the mean squared residual at collocation points plus boundary / initial condition terms.
* ``shoot_control``: piecewise-constant controls through an RK4 rollout, optimised by autograd (effort + terminal error).
Reference counterpart: scirust-variational/src/{learning/{hnn,lnn,losses,trainer,dataset,diagnostics},mechanics,pinn,
control/direct,verification}.rs.
"""
from __future__ import annotations

import math

import torch
from torch.func import grad, hessian, jacrev, vmap

D = torch.float64


def _mlp(i, hidden, o, layers=2, act=torch.nn.Softplus):
    mods, d = [], i
    for _ in range(layers):
        mods += [torch.nn.Linear(d, hidden), act()]
        d = hidden
    return torch.nn.Sequential(*mods, torch.nn.Linear(d, o)).to(D)


# ------------------------------------------------------------------ analytic mechanics on callables
def hamiltonian_vector_field(h, state: torch.Tensor) -> torch.Tensor:
    """``state [..., 2n] = (q, p)`` -> ``(dH/dp, -dH/dq)``; ``h`` maps one state vector to a scalar."""
    n = state.shape[-1] // 2
    g = vmap(grad(h))(state.reshape(-1, 2 * n))
    return torch.cat([g[:, n:], -g[:, :n]], 1).reshape(state.shape)


def lagrangian_acceleration(l, q: torch.Tensor, qd: torch.Tensor) -> torch.Tensor:
    """Solve the Euler-Lagrange equations for ``qddot``; ``l(q, qd)`` maps single vectors to a scalar."""
    shape = q.shape
    q2, v2 = q.reshape(-1, shape[-1]), qd.reshape(-1, shape[-1])
    dl_dq = vmap(grad(l, 0))(q2, v2)
    h_vv = vmap(hessian(l, 1))(q2, v2)
    h_vq = vmap(jacrev(grad(l, 1), 0))(q2, v2)
    rhs = dl_dq - (h_vq @ v2[..., None])[..., 0]
    return torch.linalg.solve(h_vv, rhs[..., None])[..., 0].reshape(shape)


def euler_lagrange_residual(l, q, qd, qdd) -> torch.Tensor:
    """``d/dt (dL/dqdot) - dL/dq`` along a path given with its first and second derivative (zero on a true motion)."""
    shape = q.shape
    q2, v2, a2 = (t.reshape(-1, shape[-1]) for t in (q, qd, qdd))
    dl_dq = vmap(grad(l, 0))(q2, v2)
    h_vv = vmap(hessian(l, 1))(q2, v2)
    h_vq = vmap(jacrev(grad(l, 1), 0))(q2, v2)
    return ((h_vv @ a2[..., None])[..., 0] + (h_vq @ v2[..., None])[..., 0] - dl_dq).reshape(shape)


def legendre_energy(l, q, qd) -> torch.Tensor:
    """``qdot . dL/dqdot - L``: the conserved energy of a time-independent Lagrangian."""
    shape = q.shape
    q2, v2 = q.reshape(-1, shape[-1]), qd.reshape(-1, shape[-1])
    p = vmap(grad(l, 1))(q2, v2)
    return ((p * v2).sum(1) - vmap(l)(q2, v2)).reshape(shape[:-1])


# ------------------------------------------------------------------ integrators
def rk4_step(f, x, dt):
    k1 = f(x)
    k2 = f(x + 0.5 * dt * k1)
    k3 = f(x + 0.5 * dt * k2)
    k4 = f(x + dt * k3)
    return x + dt / 6.0 * (k1 + 2 * k2 + 2 * k3 + k4)


def leapfrog_step(dv_dq, q, p, dt, mass=1.0):
    """Kick-drift-kick for ``H = p^2 / 2m + V(q)``; ``dv_dq(q)`` is the potential's gradient. Symplectic and reversible."""
    p = p - 0.5 * dt * dv_dq(q)
    q = q + dt * p / mass
    return q, p - 0.5 * dt * dv_dq(q)


def rollout(f, x0, dt, steps, step=rk4_step):
    out = [x0]
    for _ in range(steps):
        out.append(step(f, out[-1], dt))
    return torch.stack(out, 0)


def trajectory_from_ode(f, x0, dt, steps):
    """-> (states [steps + 1, ...], derivatives at those states): supervised pairs for the networks below."""
    xs = rollout(f, torch.as_tensor(x0, dtype=D), dt, steps)
    return xs, f(xs)


# ------------------------------------------------------------------ learned mechanics
class HamiltonianNetwork(torch.nn.Module):
    def __init__(self, dof: int, hidden: int = 64, layers: int = 2, seed: int = 0):
        super().__init__()
        torch.manual_seed(seed)
        self.dof = dof
        self.net = _mlp(2 * dof, hidden, 1, layers, torch.nn.Tanh)

    def hamiltonian(self, state):
        return self.net(state)[..., 0]

    def vector_field(self, state, create_graph: bool | None = None):
        create_graph = torch.is_grad_enabled() if create_graph is None else create_graph
        with torch.enable_grad():
            s = state if state.requires_grad else state.detach().requires_grad_(True)
            g, = torch.autograd.grad(self.hamiltonian(s).sum(), s, create_graph=create_graph)
        n = self.dof
        return torch.cat([g[..., n:], -g[..., :n]], -1)

    forward = vector_field

    def fit(self, states, derivatives, epochs: int = 500, lr: float = 1e-2) -> list:
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        hist = []
        for _ in range(epochs):
            opt.zero_grad()
            loss = ((self.vector_field(states, True) - derivatives) ** 2).mean()
            loss.backward()
            opt.step()
            hist.append(float(loss.detach()))
        return hist


class LagrangianNetwork(torch.nn.Module):
    def __init__(self, dof: int, hidden: int = 64, layers: int = 2, seed: int = 0):
        super().__init__()
        torch.manual_seed(seed)
        self.dof = dof
        self.net = _mlp(2 * dof, hidden, 1, layers, torch.nn.Softplus)

    def lagrangian(self, q, qd):
        # the explicit kinetic-like term keeps d2L/dqdot2 well conditioned at initialisation
        return self.net(torch.cat([q, qd], -1))[..., 0] + 0.5 * (qd * qd).sum(-1)

    def _derivatives(self, q, qd):
        """dL/dq [B, n], d2L/dqdot2 [B, n, n], d2L/dqdot dq [B, n, n]: 2n + 1 batched backward passes (n = dof)."""
        with torch.enable_grad():
            q = q if q.requires_grad else q.detach().requires_grad_(True)
            qd = qd if qd.requires_grad else qd.detach().requires_grad_(True)
            dl_dq, dl_dv = torch.autograd.grad(self.lagrangian(q, qd).sum(), (q, qd), create_graph=True)
            rows = [torch.autograd.grad(dl_dv[:, k].sum(), (qd, q), create_graph=True) for k in range(self.dof)]
        return dl_dq, torch.stack([r[0] for r in rows], 1), torch.stack([r[1] for r in rows], 1)

    def acceleration(self, q, qd):
        dl_dq, h_vv, h_vq = self._derivatives(q, qd)
        return torch.linalg.solve(h_vv, (dl_dq - (h_vq @ qd[..., None])[..., 0])[..., None])[..., 0]

    def _single(self, q, qd):
        return self.lagrangian(q[None], qd[None])[0]

    def forward(self, q, qd):
        return self.lagrangian(q, qd)

    def fit(self, q, qd, qdd, epochs: int = 500, lr: float = 1e-2, conditioning: float = 0.0) -> list:
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        hist = []
        for _ in range(epochs):
            opt.zero_grad()
            loss = ((self.acceleration(q, qd) - qdd) ** 2).mean()
            if conditioning:
                loss = loss + conditioning * torch.relu(0.1 - torch.linalg.eigvalsh(self._derivatives(q, qd)[1])[..., 0]).mean()
            loss.backward()
            opt.step()
            hist.append(float(loss.detach()))
        return hist


def rollout_errors(model_field, true_field, x0, dt, steps):
    """-> per-step norm of the difference between the model's and the true trajectory from the same start."""
    a, b = rollout(model_field, x0, dt, steps), rollout(true_field, x0, dt, steps)
    return (a - b).reshape(steps + 1, -1).norm(dim=1)


def conservation_drift(quantity, trajectory) -> float:
    """Largest relative deviation of ``quantity(state)`` from its initial value along a trajectory."""
    v = quantity(trajectory)
    return float(((v - v[0]).abs() / v[0].abs().clamp_min(1e-12)).max())


def finite_difference_check(fn, x, eps: float = 1e-6) -> float:
    """Largest gap between autograd's gradient of a scalar function and central differences at ``x``."""
    x = torch.as_tensor(x, dtype=D)
    g = grad(fn)(x)
    fd = torch.stack([(fn(x + eps * e) - fn(x - eps * e)) / (2 * eps) for e in torch.eye(x.numel(), dtype=D).reshape(-1, *x.shape)])
    return float((g.reshape(-1) - fd).abs().max())


# ------------------------------------------------------------------ physics-informed solver
class PinnSolver:
    """``residual(u, x)`` receives the network and collocation points ``x [n, d]`` (requiring grad) and returns the PDE /
    ODE residual per point; ``conditions`` is a list of ``(points, target values)`` the solution must match."""

    def __init__(self, in_dim: int, out_dim: int = 1, hidden: int = 32, layers: int = 3, seed: int = 0):
        torch.manual_seed(seed)
        self.net = _mlp(in_dim, hidden, out_dim, layers, torch.nn.Tanh)

    def __call__(self, x):
        return self.net(torch.as_tensor(x, dtype=D))

    @staticmethod
    def derivative(u, x, order: int = 1, component: int = 0):
        """d^order u / dx_component^order at the collocation points (graph kept for training)."""
        for _ in range(order):
            u = torch.autograd.grad(u.sum(), x, create_graph=True)[0][:, component:component + 1]
        return u

    def fit(self, residual, collocation, conditions, epochs: int = 2000, lr: float = 5e-3, condition_weight: float = 10.0) -> list:
        opt = torch.optim.Adam(self.net.parameters(), lr=lr)
        x = torch.as_tensor(collocation, dtype=D)
        hist = []
        for _ in range(epochs):
            opt.zero_grad()
            xc = x.clone().requires_grad_(True)
            loss = (residual(self.net, xc) ** 2).mean()
            for pts, val in conditions:
                loss = loss + condition_weight * ((self.net(torch.as_tensor(pts, dtype=D)) - torch.as_tensor(val, dtype=D)) ** 2).mean()
            loss.backward()
            opt.step()
            hist.append(float(loss.detach()))
        return hist


# ------------------------------------------------------------------ direct optimal control
def shoot_control(dynamics, x0, target, horizon: int, dt: float, control_dim: int = 1, effort: float = 1e-3, epochs: int = 400,
                  lr: float = 5e-2, u_max: float | None = None):
    """Single shooting: ``dynamics(x, u)`` -> dx/dt; minimise ``|x_T - target|^2 + effort * dt * sum |u|^2``.
    -> (controls [horizon, control_dim], trajectory [horizon + 1, state], final loss)."""
    x0, target = torch.as_tensor(x0, dtype=D), torch.as_tensor(target, dtype=D)
    raw = torch.zeros(horizon, control_dim, dtype=D, requires_grad=True)
    opt = torch.optim.Adam([raw], lr=lr)

    def run():
        u = raw if u_max is None else u_max * torch.tanh(raw)
        xs = [x0]
        for k in range(horizon):
            xs.append(rk4_step(lambda s: dynamics(s, u[k]), xs[-1], dt))
        return u, torch.stack(xs)
    loss = None
    for _ in range(epochs):
        opt.zero_grad()
        u, xs = run()
        loss = ((xs[-1] - target) ** 2).sum() + effort * dt * (u ** 2).sum()
        loss.backward()
        opt.step()
    with torch.no_grad():
        u, xs = run()
    return u.detach(), xs.detach(), float(loss.detach())

"""Variational mechanics, learned Hamiltonians / Lagrangians, integrators, PINN solver, shooting control (CPU)."""
import math

import torch

from scirust_b200 import physics as P

D = torch.float64


def pendulum_h(s):                                           # H = p^2 / 2 + (1 - cos q)
    return 0.5 * s[1] ** 2 + (1 - torch.cos(s[0]))


def pendulum_l(q, v):
    return 0.5 * (v ** 2).sum() - (1 - torch.cos(q)).sum()


def pendulum_field(s):
    return torch.stack([s[..., 1], -torch.sin(s[..., 0])], -1)


def test_variational_formulas_reproduce_the_pendulum():
    g = torch.Generator().manual_seed(0)
    s = torch.randn(16, 2, generator=g, dtype=D)
    assert torch.allclose(P.hamiltonian_vector_field(pendulum_h, s), pendulum_field(s), atol=1e-12)
    q, v = s[:, :1], s[:, 1:]
    acc = P.lagrangian_acceleration(pendulum_l, q, v)
    assert torch.allclose(acc, -torch.sin(q), atol=1e-12)
    assert float(P.euler_lagrange_residual(pendulum_l, q, v, acc).abs().max()) < 1e-12
    assert float(P.euler_lagrange_residual(pendulum_l, q, v, acc + 1.0).abs().min()) > 0.5
    assert torch.allclose(P.legendre_energy(pendulum_l, q, v), 0.5 * v[:, 0] ** 2 + 1 - torch.cos(q[:, 0]), atol=1e-12)
    double = lambda q_, v_: 0.5 * (2 * v_[0] ** 2 + v_[1] ** 2 + 2 * v_[0] * v_[1] * torch.cos(q_[0] - q_[1])) + 2 * torch.cos(q_[0]) + torch.cos(q_[1])
    qq, vv = torch.randn(4, 2, generator=g, dtype=D), torch.randn(4, 2, generator=g, dtype=D)
    aa = P.lagrangian_acceleration(double, qq, vv)                            # coupled, configuration-dependent mass matrix
    assert float(P.euler_lagrange_residual(double, qq, vv, aa).abs().max()) < 1e-10
    assert P.finite_difference_check(pendulum_h, torch.tensor([0.3, -0.8], dtype=D)) < 1e-8


def test_symplectic_integrator_conserves_energy_where_rk4_drifts():
    energy = lambda tr: 0.5 * tr[..., 1] ** 2 + 1 - torch.cos(tr[..., 0])
    x0 = torch.tensor([2.0, 0.0], dtype=D)
    dt, n = 0.3, 1600
    rk = P.rollout(pendulum_field, x0, dt, n)
    q, p, lf = x0[0], x0[1], [x0]
    for _ in range(n):
        q, p = P.leapfrog_step(torch.sin, q, p, dt)
        lf.append(torch.stack([q, p]))
    lf = torch.stack(lf)
    half = n // 2
    lf_trend = abs(float(energy(lf[:half]).mean() - energy(lf[half:]).mean()))
    rk_trend = abs(float(energy(rk[:half]).mean() - energy(rk[half:]).mean()))
    assert P.conservation_drift(energy, lf) < 0.03 and lf_trend < 1e-4         # bounded oscillation, no secular drift
    assert rk_trend > 100 * lf_trend and float(energy(rk[-1])) < float(energy(rk[0])) - 5e-3    # RK4 loses energy steadily
    back_q, back_p = q, -p                                                    # reversibility: run the same steps backwards
    for _ in range(n):
        back_q, back_p = P.leapfrog_step(torch.sin, back_q, back_p, dt)
    assert abs(float(back_q) - 2.0) < 1e-8 and abs(float(back_p)) < 1e-8
    xs, dx = P.trajectory_from_ode(pendulum_field, [1.0, 0.0], 0.05, 100)
    assert xs.shape == (101, 2) and torch.allclose(dx, pendulum_field(xs))


def test_hamiltonian_network_learns_a_conservative_field():
    g = torch.Generator().manual_seed(1)
    states = (torch.rand(512, 2, generator=g, dtype=D) - 0.5) * 4
    hnn = P.HamiltonianNetwork(1, hidden=48, seed=0)
    hist = hnn.fit(states, pendulum_field(states), epochs=600, lr=1e-2)
    assert hist[-1] < 2e-3 < hist[0]
    test = (torch.rand(200, 2, generator=g, dtype=D) - 0.5) * 3
    assert float((hnn.vector_field(test) - pendulum_field(test)).abs().mean()) < 0.05
    traj = P.rollout(lambda s: hnn.vector_field(s).detach(), torch.tensor([1.0, 0.0], dtype=D), 0.05, 400)
    assert P.conservation_drift(lambda tr: hnn.hamiltonian(tr).detach(), traj) < 0.02          # its own energy is conserved
    err = P.rollout_errors(lambda s: hnn.vector_field(s).detach(), pendulum_field, torch.tensor([1.0, 0.0], dtype=D), 0.05, 100)
    assert float(err[-1]) < 0.2 and float(err[0]) == 0.0
    # the learned field is divergence-free (Hamiltonian by construction), whatever the weights
    s = torch.tensor([0.3, -0.4], dtype=D)
    jac = torch.autograd.functional.jacobian(lambda x: P.HamiltonianNetwork(1, seed=5).vector_field(x, True), s)
    assert abs(float(jac[0, 0] + jac[1, 1])) < 1e-10


def test_lagrangian_network_learns_accelerations():
    g = torch.Generator().manual_seed(2)
    q = (torch.rand(256, 1, generator=g, dtype=D) - 0.5) * 3
    v = (torch.rand(256, 1, generator=g, dtype=D) - 0.5) * 3
    lnn = P.LagrangianNetwork(1, hidden=32, seed=0)
    before = float(((lnn.acceleration(q, v) + torch.sin(q)) ** 2).mean())
    hist = lnn.fit(q, v, -torch.sin(q), epochs=300, lr=1e-2)
    assert hist[-1] < 0.05 * before
    qt = torch.linspace(-1, 1, 21, dtype=D)[:, None]
    assert float((lnn.acceleration(qt, torch.zeros_like(qt)).detach() + torch.sin(qt)).abs().max()) < 0.15


def test_pinn_solves_an_oscillator_and_shooting_steers_a_double_integrator():
    def residual(net, x):                                                     # u'' + u = 0, u(0) = 0, u'(0) = 1 -> sin x
        u = net(x)
        return P.PinnSolver.derivative(u, x, 2) + u
    pinn = P.PinnSolver(1, hidden=24, layers=3, seed=0)
    x = torch.linspace(0, math.pi, 64, dtype=D)[:, None]
    eps = 1e-3
    hist = pinn.fit(residual, x, [([[0.0]], [[0.0]]), ([[eps]], [[math.sin(eps)]]), ([[math.pi / 2]], [[1.0]])], epochs=1500, lr=5e-3)
    assert hist[-1] < 1e-3 < hist[0]
    assert float((pinn(x).detach()[:, 0] - torch.sin(x[:, 0])).abs().max()) < 0.03
    dyn = lambda s, u: torch.stack([s[1], u[0]])                               # position, velocity; force as control
    u, xs, loss = P.shoot_control(dyn, [0.0, 0.0], [1.0, 0.0], horizon=20, dt=0.1, effort=1e-3, epochs=300, lr=0.1)
    assert float((xs[-1] - torch.tensor([1.0, 0.0], dtype=D)).abs().max()) < 0.02 and loss < 0.01
    assert float(u[:5].mean()) > 0 > float(u[-5:].mean())                      # accelerate, then brake
    ub, xb, _ = P.shoot_control(dyn, [0.0, 0.0], [1.0, 0.0], horizon=20, dt=0.1, u_max=1.5, epochs=300, lr=0.1)
    assert float(ub.abs().max()) <= 1.5 and float((xb[-1, 0] - 1.0).abs()) < 0.05

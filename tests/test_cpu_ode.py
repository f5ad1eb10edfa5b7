"""Explicit and stiff initial-value solvers (CPU)."""
import math

import pytest
import torch

from scirust_b200 import ode as O

D = torch.float64


def test_dopri5_meets_its_tolerance_on_an_oscillator():
    f = lambda t, y: torch.stack([y[1], -y[0]])
    sol = O.dopri5(f, [1.0, 0.0], 0.0, 10.0, rtol=1e-9, atol=1e-12)
    want = torch.tensor([math.cos(10.0), -math.sin(10.0)], dtype=D)
    assert float((sol.final() - want).abs().max()) < 1e-7 and sol.t[-1] == pytest.approx(10.0) and sol.steps < 400
    loose = O.dopri5(f, [1.0, 0.0], 0.0, 10.0, rtol=1e-4, atol=1e-6)
    assert loose.steps < sol.steps and float((loose.final() - want).abs().max()) < 1e-2
    assert sol.states().shape == (sol.steps + 1, 2)


def test_stiff_solvers_take_large_steps_where_the_explicit_one_cannot():
    lam = 1000.0
    f = lambda t, y: -lam * (y - torch.cos(torch.as_tensor(t, dtype=D)))
    exact = lambda t: (lam * lam * math.cos(t) + lam * math.sin(t)) / (1 + lam * lam)          # the slow manifold (transient gone)
    ros = O.rosenbrock23(f, [0.0], 0.0, 2.0, rtol=1e-3, atol=1e-6)             # a loose tolerance: stability, not accuracy, would bind
    exp = O.dopri5(f, [0.0], 0.0, 2.0, rtol=1e-3, atol=1e-6)
    assert abs(float(ros.final()[0]) - exact(2.0)) < 2e-3 and abs(float(exp.final()[0]) - exact(2.0)) < 2e-3
    assert ros.steps < 0.2 * exp.steps and ros.jac_evals == ros.steps                            # stability does not limit the step
    be = O.backward_euler(f, [0.0], 0.0, 2.0, h=0.05)                                            # h * lambda = 50: far outside explicit stability
    assert abs(float(be.final()[0]) - exact(2.0)) < 5e-3 and be.steps == 40
    vdp = lambda t, y: torch.stack([y[1], 50.0 * (1 - y[0] ** 2) * y[1] - y[0]])                   # Van der Pol, mu = 50
    a = O.rosenbrock23(vdp, [2.0, 0.0], 0.0, 20.0, rtol=1e-5, atol=1e-8)
    b = O.dopri5(vdp, [2.0, 0.0], 0.0, 20.0, rtol=1e-8, atol=1e-10)
    assert float((a.final() - b.final()).abs().max()) < 5e-3 and a.steps < b.steps
    with pytest.raises(O.OdeError):
        O.backward_euler(lambda t, y: y ** 2 + 1e6, [0.0], 0.0, 1.0, h=1.0, max_newton=3)


def test_robertson_kinetics_conserve_mass_and_the_dae_form_enforces_the_constraint():
    def rob(t, y):
        return torch.stack([-0.04 * y[0] + 1e4 * y[1] * y[2], 0.04 * y[0] - 1e4 * y[1] * y[2] - 3e7 * y[1] ** 2, 3e7 * y[1] ** 2])
    sol = O.rosenbrock23(rob, [1.0, 0.0, 0.0], 0.0, 40.0, rtol=1e-5, atol=1e-10)
    y = sol.final()
    assert abs(float(y.sum()) - 1.0) < 1e-6
    assert abs(float(y[0]) - 0.7158) < 2e-3 and abs(float(y[1]) - 9.185e-6) < 2e-7 and abs(float(y[2]) - 0.2842) < 2e-3    # reference values at t = 40
    assert sol.steps < 400
    def rob_dae(t, y):                                                        # third equation replaced by the conservation law
        return torch.stack([-0.04 * y[0] + 1e4 * y[1] * y[2], 0.04 * y[0] - 1e4 * y[1] * y[2] - 3e7 * y[1] ** 2, y[0] + y[1] + y[2] - 1.0])
    mass = torch.diag(torch.tensor([1.0, 1.0, 0.0], dtype=D))
    dae = O.backward_euler_dae(rob_dae, mass, [1.0, 0.0, 0.0], 0.0, 40.0, h=0.1)
    assert float((dae.states().sum(1) - 1.0).abs().max()) < 1e-12                                 # the constraint holds at every step
    assert abs(float(dae.final()[0]) - 0.7158) < 5e-3

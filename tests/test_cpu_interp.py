"""Interpolants against scipy.interpolate and their defining properties (CPU)."""
import numpy as np
import pytest
import torch

from scirust_b200 import interp as I

si = pytest.importorskip("scipy.interpolate")


def _data():
    g = np.random.default_rng(0)
    x = np.sort(g.uniform(0, 10, 12))
    y = np.stack([np.sin(x), g.normal(size=12)])
    return x, y, np.linspace(x[0], x[-1], 201)


def test_splines_pchip_and_akima_match_scipy_on_batched_values():
    x, y, q = _data()
    for ours, ref in ((I.CubicSpline(x, y), si.CubicSpline(x, y, axis=1)), (I.CubicSpline(x, y, "natural"), si.CubicSpline(x, y, axis=1, bc_type="natural")),
                      (I.Pchip(x, y), si.PchipInterpolator(x, y, axis=1)), (I.Akima(x, y), si.Akima1DInterpolator(x, y, axis=1))):
        assert np.abs(ours(q).numpy() - ref(q)).max() < 1e-10
        assert np.abs(ours.derivative(q).numpy() - ref(q, 1)).max() < 1e-8
    assert I.CubicSpline(x, y)(torch.tensor(q).reshape(3, 67)).shape == (2, 3, 67)            # query shape is kept
    far = np.array([x[0] - 1.0, x[-1] + 1.0])
    assert np.abs(I.CubicSpline(x, y)(far).numpy() - si.CubicSpline(x, y, axis=1)(far)).max() < 1e-9     # end polynomials extrapolate
    held = I.CubicSpline(x, y, clamp=True)(far).numpy()
    assert np.allclose(held[:, 0], y[:, 0]) and np.allclose(held[:, 1], y[:, -1])
    assert np.abs(I.CubicSpline(x[:3], y[:, :3])(q[:20]).numpy() - si.CubicSpline(x[:3], y[:, :3], axis=1)(q[:20])).max() < 1e-10
    assert np.abs(I.CubicSpline(x[:2], y[:, :2])(q[:5]).numpy() - si.interp1d(x[:2], y[:, :2], fill_value="extrapolate")(q[:5])).max() < 1e-10


def test_linear_nearest_and_shape_preservation():
    x, y, q = _data()
    assert np.abs(I.LinearInterp(x, y)(q).numpy() - np.stack([np.interp(q, x, r) for r in y])).max() < 1e-12
    assert I.LinearInterp([0, 1], [0, 2])(3.0).item() == 6.0 and I.LinearInterp([0, 1], [0, 2], clamp=True)(3.0).item() == 2.0
    assert I.NearestInterp([0, 1, 2], [10, 20, 30])([0.4, 0.5, 0.6, 1.9, -5, 9]).tolist() == [10, 10, 20, 30, 10, 30]
    steps_x, steps_y = [0, 1, 2, 3, 4, 5], [0, 0, 0, 1, 1, 1]
    dense = torch.linspace(0, 5, 501, dtype=torch.float64)
    p = I.Pchip(steps_x, steps_y)(dense)
    assert float(p.min()) >= 0.0 and float(p.max()) <= 1.0 and bool((p[1:] >= p[:-1] - 1e-15).all())    # monotone, no overshoot
    s = I.CubicSpline(steps_x, steps_y)(dense)
    assert float(s.min()) < -0.01 and float(s.max()) > 1.01                                           # the spline overshoots the step
    for bad in (([0, 0, 1], [1, 2, 3]), ([0], [1]), ([0, 1], [1, 2, 3])):
        with pytest.raises(ValueError):
            I.LinearInterp(*bad)


def test_barycentric_polynomial_on_chebyshev_nodes():
    f = lambda t: 1.0 / (1.0 + 25.0 * t * t)                                                         # Runge's function
    nodes = I.chebyshev_nodes(60)
    q = torch.linspace(-1, 1, 1001, dtype=torch.float64)
    assert float((I.Barycentric(nodes, f(nodes))(q) - f(q)).abs().max()) < 1e-4
    equi = torch.linspace(-1, 1, 21, dtype=torch.float64)
    assert float((I.Barycentric(equi, f(equi))(q) - f(q)).abs().max()) > 1.0                         # equispaced nodes diverge
    poly = lambda t: 3 * t ** 3 - t + 2
    b = I.Barycentric([-1.0, 0.0, 0.5, 2.0], poly(torch.tensor([-1.0, 0.0, 0.5, 2.0], dtype=torch.float64)))
    assert float((b(q) - poly(q)).abs().max()) < 1e-12 and b(0.5).item() == poly(torch.tensor(0.5, dtype=torch.float64)).item()
    with pytest.raises(ValueError):
        I.Barycentric([0, 0, 1], [1, 2, 3])

"""Quaternions, dual quaternions, SE(2), Cayley-Dickson algebras, dual numbers, attitude filter, curves (CPU)."""
import math

import pytest
import torch

from scirust_b200 import geometry as G

D = torch.float64


def _rand_q(n, seed):
    return G.q_normalize(torch.randn(n, 4, dtype=D, generator=torch.Generator().manual_seed(seed)))


def _same_rotation(a, b):
    return float(torch.minimum((a - b).abs().amax(-1), (a + b).abs().amax(-1)).max())


def test_quaternion_conversions_round_trip():
    q, v = _rand_q(64, 0), torch.randn(64, 3, dtype=D, generator=torch.Generator().manual_seed(1))
    r = G.q_to_matrix(q)
    assert float((G.q_rotate(q, v) - (r @ v[..., None])[..., 0]).abs().max()) < 1e-12
    assert float((r @ r.transpose(-1, -2) - torch.eye(3, dtype=D)).abs().max()) < 1e-12
    assert float((torch.linalg.det(r) - 1).abs().max()) < 1e-12
    assert _same_rotation(G.q_from_matrix(r), q) < 1e-12
    assert _same_rotation(G.q_from_euler(*G.q_to_euler(q)), q) < 1e-12
    axis, angle = G.q_to_axis_angle(q)
    assert _same_rotation(G.q_from_axis_angle(axis, angle), q) < 1e-12
    assert float((G.q_mul(q, G.q_inverse(q)) - G.q_identity(64)).abs().max()) < 1e-12
    lock = G.q_from_euler(torch.tensor(0.3, dtype=D), torch.tensor(math.pi / 2, dtype=D), torch.tensor(0.5, dtype=D))
    roll, pitch, yaw = G.q_to_euler(lock)
    assert float(roll) == 0.0 and abs(float(pitch) - math.pi / 2) < 1e-12              # yaw carries what is left
    assert float((G.q_to_matrix(G.q_from_euler(roll, pitch, yaw)) - G.q_to_matrix(lock)).abs().max()) < 1e-9
    yaw90 = G.q_from_euler(torch.tensor(0.0, dtype=D), torch.tensor(0.0, dtype=D), torch.tensor(math.pi / 2, dtype=D))
    assert float((G.q_rotate(yaw90, torch.tensor([1.0, 0, 0], dtype=D)) - torch.tensor([0.0, 1, 0], dtype=D)).abs().max()) < 1e-12


def test_slerp_has_constant_speed_and_squad_passes_through_its_keys():
    a, b = _rand_q(16, 2), _rand_q(16, 3)
    assert _same_rotation(G.q_slerp(a, b, 0.0), a) < 1e-12 and _same_rotation(G.q_slerp(a, b, 1.0), b) < 1e-12
    ts = [0.0, 0.25, 0.5, 0.75, 1.0]
    pts = [G.q_slerp(a, b, t) for t in ts]
    steps = torch.stack([torch.acos(((pts[i] * pts[i + 1]).sum(-1)).abs().clamp(max=1)) for i in range(4)])
    assert float((steps - steps[0]).abs().max()) < 1e-9
    assert _same_rotation(G.q_slerp(a, a, 0.3), a) < 1e-12                               # parallel inputs: no division by zero
    assert _same_rotation(G.q_nlerp(a, b, 0.5), G.q_slerp(a, b, 0.5)) < 1e-9             # the midpoint coincides
    keys = [G.q_from_axis_angle([0.0, 0, 1], 0.3 * i + 0.05 * i * i) for i in range(4)]
    s1, s2 = G.q_squad_setup(keys[0], keys[1], keys[2]), G.q_squad_setup(keys[1], keys[2], keys[3])
    assert _same_rotation(G.q_squad(keys[1], keys[2], s1, s2, 0.0), keys[1]) < 1e-12
    assert _same_rotation(G.q_squad(keys[1], keys[2], s1, s2, 1.0), keys[2]) < 1e-12
    mid_angle = float(G.q_to_axis_angle(G.q_squad(keys[1], keys[2], s1, s2, 0.5))[1])
    assert float(G.q_to_axis_angle(keys[1])[1]) < mid_angle < float(G.q_to_axis_angle(keys[2])[1])
    assert float((G.q_exp(G.q_log(a)) - torch.where(a[..., :1] < 0, -a, a)).abs().max()) < 1e-12


def test_dual_quaternions_compose_and_interpolate_rigid_motions():
    g = torch.Generator().manual_seed(4)
    qa, qb = _rand_q(32, 5), _rand_q(32, 6)
    ta, tb, v = (torch.randn(32, 3, dtype=D, generator=g) for _ in range(3))
    a, b = G.dq_from_rotation_translation(qa, ta), G.dq_from_rotation_translation(qb, tb)
    assert float((G.dq_transform_point(a, v) - (G.q_rotate(qa, v) + ta)).abs().max()) < 1e-12
    ab = G.dq_mul(a, b)
    assert float((G.dq_transform_point(ab, v) - G.dq_transform_point(a, G.dq_transform_point(b, v))).abs().max()) < 1e-12
    inv = G.dq_mul(a, G.dq_conjugate(a))
    assert float((G.dq_transform_point(inv, v) - v).abs().max()) < 1e-12
    l, m, th, d = G.dq_to_screw(a)
    back = G.dq_from_screw(l, m, th, d)
    assert float((G.dq_transform_point(back, v) - G.dq_transform_point(a, v)).abs().max()) < 1e-10
    for t, want in ((0.0, a), (1.0, b)):
        got = G.dq_sclerp(a, b, t)
        assert float((G.dq_transform_point(got, v) - G.dq_transform_point(want, v)).abs().max()) < 1e-10
    half = G.dq_sclerp(a, b, 0.5)
    twice = G.dq_mul(G.dq_mul(half, G.dq_conjugate(a)), half)                             # (half a^-1) half = b
    assert float((G.dq_transform_point(twice, v) - G.dq_transform_point(b, v)).abs().max()) < 1e-9
    shift = G.dq_from_rotation_translation(G.q_identity(), torch.tensor([2.0, 0, 0], dtype=D))
    halfway = G.dq_pow(shift, 0.5)
    assert float((G.dq_transform_point(halfway, torch.zeros(3, dtype=D)) - torch.tensor([1.0, 0, 0], dtype=D)).abs().max()) < 1e-12


def test_se2_cayley_dickson_and_dual_numbers():
    a, b = G.Se2(0.4, [1.0, 2.0]), G.Se2(-1.1, [0.5, -0.3])
    p = torch.tensor([0.7, -0.2], dtype=D)
    assert float((a.compose(b).transform_point(p) - a.transform_point(b.transform_point(p))).abs().max()) < 1e-12
    assert float((a.inverse().transform_point(a.transform_point(p)) - p).abs().max()) < 1e-12
    q, r = _rand_q(8, 7), _rand_q(8, 8)
    assert float((G.cayley_dickson_mul(q, r) - G.q_mul(q, r)).abs().max()) < 1e-12
    g = torch.Generator().manual_seed(9)
    o1, o2, o3 = (torch.randn(8, dtype=D, generator=g) for _ in range(3))
    prod = G.cayley_dickson_mul(o1, o2)
    assert abs(float(G.cd_norm_sqr(prod) - G.cd_norm_sqr(o1) * G.cd_norm_sqr(o2))) < 1e-10            # octonions: composition algebra
    assoc = G.cayley_dickson_mul(prod, o3) - G.cayley_dickson_mul(o1, G.cayley_dickson_mul(o2, o3))
    assert float(assoc.abs().max()) > 1e-3                                                           # ... but not associative
    alt = G.cayley_dickson_mul(G.cayley_dickson_mul(o1, o1), o2) - G.cayley_dickson_mul(o1, G.cayley_dickson_mul(o1, o2))
    assert float(alt.abs().max()) < 1e-10                                                            # alternative
    one = torch.zeros(8, dtype=D)
    one[0] = 1.0
    assert float((G.cayley_dickson_mul(o1, G.cd_inverse(o1)) - one).abs().max()) < 1e-12
    e = torch.eye(16, dtype=D)
    zero_div = G.cayley_dickson_mul(e[3] + e[10], e[6] - e[15])
    assert float(zero_div.abs().max()) < 1e-12                                                       # sedenions have zero divisors
    assert float((G.cd_exp(G.cd_ln(o1)) - o1).abs().max()) < 1e-10
    assert float((G.cayley_dickson_mul(G.cd_powf(o1, 0.5), G.cd_powf(o1, 0.5)) - o1).abs().max()) < 1e-10
    with pytest.raises(ValueError):
        G.cayley_dickson_mul(torch.zeros(3), torch.zeros(3))
    x = G.Dual.variable(torch.tensor(0.7, dtype=D))
    f = (x * x).sin() / x.exp() + x.sqrt().ln() + 2.0 * x.powf(1.5) - 1.0 / x
    xx = torch.tensor(0.7, dtype=D, requires_grad=True)
    ff = torch.sin(xx * xx) / torch.exp(xx) + torch.log(torch.sqrt(xx)) + 2.0 * xx ** 1.5 - 1.0 / xx
    ff.backward()
    assert abs(float(f.re - ff)) < 1e-12 and abs(float(f.eps - xx.grad)) < 1e-12


def test_attitude_filter_converges_and_curves_interpolate():
    truth = G.q_from_euler(torch.tensor(0.4, dtype=D), torch.tensor(-0.3, dtype=D), torch.tensor(0.0, dtype=D))
    accel = G.q_rotate(G.q_conj(truth), torch.tensor([0.0, 0, 1], dtype=D))              # gravity seen from the body
    ahrs = G.MahonyAhrs(kp=2.0)
    for _ in range(1500):
        ahrs.update_imu(torch.zeros(3, dtype=D), accel, 0.01)
    roll, pitch, _ = G.q_to_euler(ahrs.orientation)
    assert abs(float(roll) - 0.4) < 1e-3 and abs(float(pitch) + 0.3) < 1e-3               # yaw is unobservable without a compass
    truth = G.q_from_euler(torch.tensor(0.2, dtype=D), torch.tensor(0.1, dtype=D), torch.tensor(0.9, dtype=D))
    north = torch.tensor([0.5, 0.0, -0.8], dtype=D)
    accel, mag = G.q_rotate(G.q_conj(truth), torch.tensor([0.0, 0, 1], dtype=D)), G.q_rotate(G.q_conj(truth), north)
    ahrs = G.MahonyAhrs(kp=2.0)
    for _ in range(3000):
        ahrs.update_marg(torch.zeros(3, dtype=D), accel, mag, 0.01)
    assert _same_rotation(ahrs.orientation, truth) < 2e-3
    bias = torch.tensor([0.02, -0.01, 0.0], dtype=D)
    ahrs = G.MahonyAhrs(kp=1.0, ki=0.3)
    for _ in range(6000):
        ahrs.update_imu(bias, torch.tensor([0.0, 0, 1], dtype=D), 0.01)
    assert float((ahrs.bias[:2] + bias[:2]).abs().max()) < 2e-3                           # the integral term cancels a constant bias
    p = [torch.tensor(v, dtype=D) for v in ([0.0, 0], [1.0, 2], [3.0, 2], [4.0, 0])]
    assert torch.equal(G.bezier_cubic(*p, 0.0), p[0]) and torch.equal(G.bezier_cubic(*p, 1.0), p[3])
    assert float((G.bezier_cubic_tangent(*p, 0.0) - 3 * (p[1] - p[0])).abs().max()) < 1e-12
    assert float((G.catmull_rom(*p, 0.0) - p[1]).abs().max()) < 1e-12 and float((G.catmull_rom(*p, 1.0) - p[2]).abs().max()) < 1e-12
    assert G.bezier_cubic(*p, torch.linspace(0, 1, 5, dtype=D)).shape == (5, 2)
    line = [torch.tensor([float(i), 2.0 * i], dtype=D) for i in range(4)]
    assert float((G.catmull_rom(*line, 0.5) - torch.tensor([1.5, 3.0], dtype=D)).abs().max()) < 1e-12

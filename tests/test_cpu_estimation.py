"""Extended / unscented Kalman filters, RTS smoother, particle filter and IMM (CPU)."""
import math

import torch

from scirust_b200 import estimation as E

D = torch.float64


def _g(seed):
    return torch.Generator().manual_seed(seed)


def test_ekf_and_ukf_track_a_pendulum_from_nonlinear_measurements():
    dt = 0.05
    f = lambda s: torch.stack([s[0] + dt * s[1], s[1] - dt * 9.81 * torch.sin(s[0])])
    h = lambda s: torch.sin(s[0])[None]                                       # horizontal position of the bob
    g = _g(0)
    truth, zs, s = [], [], torch.tensor([1.2, 0.0], dtype=D)
    for _ in range(300):
        s = f(s)
        truth.append(s)
        zs.append(h(s) + 0.1 * torch.randn(1, generator=g, dtype=D))
    truth = torch.stack(truth)
    q, r = torch.eye(2, dtype=D) * 1e-5, torch.eye(1, dtype=D) * 0.01
    for make in (lambda: E.ExtendedKalmanFilter([0.8, 0.5], torch.eye(2, dtype=D)), lambda: E.UnscentedKalmanFilter([0.8, 0.5], torch.eye(2, dtype=D))):
        kf, est = make(), []
        for z in zs:
            kf.predict(f, q)
            kf.update(z, h, r)
            est.append(kf.x.clone())
        est = torch.stack(est)
        err = (est[100:] - truth[100:]).abs()
        assert float(err[:, 0].mean()) < 0.05 and float(err[:, 1].mean()) < 0.25           # the unobserved velocity is recovered too
        assert float(torch.linalg.eigvalsh(kf.p).min()) > 0 and float(kf.p[0, 0]) < 0.01
    lin = E.ExtendedKalmanFilter([0.0, 0.0], torch.eye(2, dtype=D))
    fm, hm = torch.tensor([[1.0, 1.0], [0.0, 1.0]], dtype=D), torch.tensor([[1.0, 0.0]], dtype=D)
    ref = E.kalman_filter_sequence(torch.tensor([[1.0], [2.1], [2.9]], dtype=D), fm, q, hm, r, [0.0, 0.0], torch.eye(2, dtype=D))
    for z in ([1.0], [2.1], [2.9]):                                           # on a linear model the EKF is the Kalman filter
        lin.predict(lambda s_: fm @ s_, q)
        lin.update(z, lambda s_: hm @ s_, r)
    assert torch.allclose(lin.x, ref["xf"][-1], atol=1e-12) and torch.allclose(lin.p, ref["pf"][-1], atol=1e-12)


def test_smoother_reduces_error_and_variance():
    g = _g(1)
    f, h = torch.tensor([[1.0, 1.0], [0.0, 1.0]], dtype=D), torch.tensor([[1.0, 0.0]], dtype=D)
    q, r = torch.diag(torch.tensor([1e-4, 1e-3], dtype=D)), torch.tensor([[1.0]], dtype=D)
    x, truth, zs = torch.tensor([0.0, 0.3], dtype=D), [], []
    for _ in range(200):
        x = f @ x + torch.randn(2, generator=g, dtype=D) * torch.sqrt(torch.diagonal(q))
        truth.append(x)
        zs.append(h @ x + torch.randn(1, generator=g, dtype=D))
    truth = torch.stack(truth)
    filt = E.kalman_filter_sequence(torch.stack(zs), f, q, h, r, [0.0, 0.0], torch.eye(2, dtype=D) * 10)
    xs, ps = E.rts_smoother(filt, f)
    fe, se = (filt["xf"] - truth)[:, 0].pow(2).mean(), (xs - truth)[:, 0].pow(2).mean()
    assert float(se) < 0.8 * float(fe)
    assert bool((torch.diagonal(ps, dim1=1, dim2=2) <= torch.diagonal(filt["pf"], dim1=1, dim2=2) + 1e-12).all())
    assert torch.allclose(xs[-1], filt["xf"][-1]) and math.isfinite(filt["log_likelihood"])
    worse = E.kalman_filter_sequence(torch.stack(zs), f, q, h, r * 100, [0.0, 0.0], torch.eye(2, dtype=D) * 10)
    assert worse["log_likelihood"] < filt["log_likelihood"]                   # the true noise level explains the data better


def test_particle_filter_handles_a_bimodal_measurement():
    g = _g(2)
    # the sensor sees |x| only: the posterior has two modes until the drift reveals the sign
    x, truth, zs = 2.0, [], []
    for _ in range(60):
        x = x + 0.15 + 0.05 * float(torch.randn((), generator=g, dtype=D))
        truth.append(x)
        zs.append(abs(x) + 0.2 * float(torch.randn((), generator=g, dtype=D)))
    pf = E.ParticleFilter(torch.randn(4000, 1, generator=g, dtype=D) * 3, seed=3)
    prop = lambda p, gen: p + 0.15 + 0.05 * torch.randn(p.shape, generator=gen, dtype=D)
    first = None
    for i, z in enumerate(zs):
        pf.predict(prop)
        ess = pf.update(lambda p: -0.5 * ((p[:, 0].abs() - z) / 0.2) ** 2)
        if i == 0:
            first = pf.x[:, 0].clone()
    assert float((first > 0).double().mean()) > 0.2 and float((first < 0).double().mean()) > 0.2      # both signs alive at first
    mean, cov = pf.estimate()
    assert abs(float(mean[0]) - truth[-1]) < 0.3 and float(cov[0, 0]) < 0.1 and pf.resamples > 3 and 0 < ess <= 4000


def test_imm_switches_between_cruise_and_manoeuvre_models():
    g = _g(4)
    dt = 1.0
    f = torch.tensor([[1.0, dt], [0.0, 1.0]], dtype=D)
    gq = torch.tensor([[dt ** 4 / 4, dt ** 3 / 2], [dt ** 3 / 2, dt ** 2]], dtype=D)
    h, r = torch.tensor([[1.0, 0.0]], dtype=D), torch.tensor([[1.0]], dtype=D)
    imm = E.ImmFilter([(f, gq * 1e-4), (f, gq * 4.0)], [[0.95, 0.05], [0.05, 0.95]], h, r, [0.0, 1.0], torch.eye(2, dtype=D) * 10)
    single = [E.kalman_filter_sequence, None]
    x, v, mode_prob, errs_imm, zs, truth = 0.0, 1.0, [], [], [], []
    for t in range(120):
        a = 2.0 * math.sin(0.5 * t) if 40 <= t < 80 else 0.0                      # a manoeuvre in the middle third
        x, v = x + v * dt + 0.5 * a * dt * dt, v + a * dt
        z = torch.tensor([x + float(torch.randn((), generator=g, dtype=D))], dtype=D)
        est, _ = imm.step(z)
        mode_prob.append(float(imm.mu[1]))
        errs_imm.append(abs(float(est[0]) - x))
        zs.append(z)
        truth.append(x)
    mp = torch.tensor(mode_prob)
    assert float(mp[15:40].mean()) < 0.2 and float(mp[45:80].mean()) > 0.7 and float(mp[100:].mean()) < 0.3
    quiet = E.kalman_filter_sequence(torch.stack(zs), f, gq * 1e-4, h, r, [0.0, 1.0], torch.eye(2, dtype=D) * 10)
    quiet_err = (quiet["xf"][:, 0] - torch.tensor(truth, dtype=D)).abs()
    assert sum(errs_imm[45:85]) < 0.5 * float(quiet_err[45:85].sum())           # the cruise-only filter lags in the manoeuvre
    loud = E.kalman_filter_sequence(torch.stack(zs), f, gq * 4.0, h, r, [0.0, 1.0], torch.eye(2, dtype=D) * 10)
    loud_err = (loud["xf"][:, 0] - torch.tensor(truth, dtype=D)).abs()
    assert sum(errs_imm[10:40]) < float(loud_err[10:40].sum())                  # ... and the manoeuvre-only filter is noisy in cruise
    assert abs(float(imm.mu.sum()) - 1.0) < 1e-12

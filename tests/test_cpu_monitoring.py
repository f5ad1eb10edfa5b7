"""Control charts, robust covariance, seasonal decomposition, change points and RUL (CPU)."""
import math

import pytest
import torch

from scirust_b200 import monitoring as M

D = torch.float64


def _g(seed):
    return torch.Generator().manual_seed(seed)


def test_shewhart_cusum_and_ewma_charts():
    x = 10 + 0.5 * torch.randn(200, generator=_g(0), dtype=D)
    chart = M.ControlChart.from_individuals(x)
    assert abs(chart.center - 10) < 0.1 and abs(chart.sigma - 0.5) < 0.07 and chart.ucl - chart.lcl == pytest.approx(6 * chart.sigma)
    probe = x.clone()
    probe[50] = 13.0
    assert 50 in chart.out_of_control(probe) and len(chart.out_of_control(x)) <= 2
    sub = M.ControlChart.from_subgroups(x.reshape(40, 5))
    assert abs(sub.sigma - 0.5 / math.sqrt(5)) < 0.04
    runs = torch.cat([torch.full((5,), 10.0, dtype=D), torch.full((8,), 10.2, dtype=D), torch.tensor([11.2, 11.3], dtype=D)])
    we = M.ControlChart(10.0, 0.5).western_electric(runs)
    assert we[4] == [12, 13, 14] and we[2] == [14] and we[1] == []              # 8 on one side; 2 of 3 beyond 2 sigma
    shifted = torch.cat([x[:100], x[100:] + 0.5])                              # a one-sigma shift: too small for 3-sigma limits
    assert len(M.ControlChart(10.0, 0.5).out_of_control(shifted)) <= 3
    alarms = M.CusumChart(10.0, 0.5).run(shifted)
    assert alarms and alarms[0][1] == "up" and 100 < alarms[0][0] < 130 and M.CusumChart(10.0, 0.5).run(x[:100]) == []
    vals, half, out = M.EwmaChart(10.0, 0.5, lam=0.2).run(shifted)
    assert out and 100 < out[0] < 125 and float(half[0]) < float(half[-1]) == pytest.approx(3 * 0.5 * math.sqrt(0.2 / 1.8), rel=1e-6)


def test_hotelling_and_minimum_covariance_determinant():
    g = _g(1)
    cov = torch.tensor([[1.0, 0.9], [0.9, 1.0]], dtype=D)
    ref = torch.randn(300, 2, generator=g, dtype=D) @ torch.linalg.cholesky(cov).t()
    t2 = M.HotellingT2(ref)
    odd = torch.tensor([[1.5, -1.5]], dtype=D)                                  # inside each marginal range, against the correlation
    assert float(t2.statistic(odd)) > t2.limit() > 11 and 20 in t2.out_of_control(torch.cat([ref[:20], odd])) and len(t2.out_of_control(ref)) <= 5
    bad = torch.randn(60, 2, generator=g, dtype=D) * 0.3 + torch.tensor([6.0, -6.0], dtype=D)
    x = torch.cat([ref, bad])
    mu, c, inl = M.mcd_covariance(x)
    assert float(mu.abs().max()) < 0.15 and float((c - cov).abs().max()) < 0.2 and int(inl[300:].sum()) == 0 and int(inl[:300].sum()) > 270
    classical = torch.cov(x.t())
    assert float((classical - cov).abs().max()) > 3.0                            # the cluster wrecks the ordinary estimate
    d = M.robust_mahalanobis(x)
    assert float(d[300:].min()) > 10 and float(d[:300].median()) < 1.6


def test_period_detection_decomposition_and_harmonics():
    n = torch.arange(240, dtype=D)
    x = 5 + 0.05 * n + 3 * torch.sin(2 * math.pi * n / 12) + 0.3 * torch.randn(240, generator=_g(2), dtype=D)
    period, strength = M.detect_period(x)
    assert period == 12 and strength > 0.7
    assert M.detect_period(torch.randn(200, generator=_g(3), dtype=D))[0] is None
    spiky = x.clone()
    spiky[[40, 41, 150]] += 25.0
    trend, seasonal, resid = M.stl_decompose(spiky, 12)
    assert torch.allclose(trend + seasonal + resid, spiky)
    assert float((seasonal[:12] - 3 * torch.sin(2 * math.pi * n[:12] / 12)).abs().max()) < 0.4        # spikes do not leak into the season
    assert float(seasonal[:12].sum().abs()) < 1e-9 and float((trend[24:-24] - (5 + 0.05 * n[24:-24])).abs().median()) < 0.3
    assert sorted(resid.abs().topk(3).indices.tolist()) == [40, 41, 150]
    fitted, amps = M.harmonic_fit(x, 12.0, harmonics=3)
    assert abs(amps[0] - 3.0) < 0.15 and amps[1] < 0.15 and float((fitted - x).std()) < 0.4
    with pytest.raises(ValueError):
        M.stl_decompose(x[:20], 12)


def test_change_points_and_remaining_useful_life():
    g = _g(4)
    x = torch.cat([torch.randn(120, generator=g, dtype=D), 2.0 + torch.randn(80, generator=g, dtype=D), -1.0 + torch.randn(100, generator=g, dtype=D)])
    cps = M.cusum_change_points(x)
    assert len(cps) == 2 and abs(cps[0] - 120) <= 6 and abs(cps[1] - 200) <= 6
    assert M.cusum_change_points(torch.randn(300, generator=g, dtype=D)) == []
    ph = M.page_hinkley(torch.cat([torch.randn(150, generator=g, dtype=D) * 0.2, 1.0 + torch.randn(50, generator=g, dtype=D) * 0.2]), lam=3.0)
    assert ph is not None and 150 <= ph < 165 and M.page_hinkley(torch.randn(200, generator=g, dtype=D) * 0.2, lam=5.0) is None
    t = torch.arange(300, dtype=D)
    vib = 1.0 + 0.05 * torch.randn(300, generator=g, dtype=D) + torch.where(t > 100, 0.01 * (t - 100), torch.zeros_like(t))
    hi = M.health_index(vib, healthy=80)
    assert bool((hi[1:] >= hi[:-1]).all()) and float(hi[90]) < 4.0 < float(hi[-1])
    slope = float(hi[-1] - hi[-31]) / 30
    rul, lo, up = M.estimate_rul(hi, threshold=float(hi[-1]) + 50 * slope, window=30)
    assert lo <= rul <= up and abs(rul - 50) < 12
    assert M.estimate_rul(torch.ones(50, dtype=D), 2.0)[0] == math.inf
    grow = torch.exp(0.02 * t[:200])
    r, _, _ = M.estimate_rul(grow, threshold=math.exp(0.02 * 260), window=40, model="exponential")
    assert abs(r - 61) < 1.0

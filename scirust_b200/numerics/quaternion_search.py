"""Joint (chart, accumulation) search on a second kernel: averaging noisy unit quaternions.

The estimate of a fixed orientation from N noisy observations depends on two choices that interact: the CHART in which
the samples are averaged (``componentwise``: mean of the raw (w, x, y, z) in R^4, renormalised, cheap but biased at high
noise; ``log-chart``: a Karcher-style mean, i.e. log-map every sample to the tangent space at the current estimate,
average the tangent vectors, exp-map back, repeated a fixed number of times) and the ACCUMULATION method that sums each
component column (narrowed to fp32 for the sum, chart arithmetic in float64). ``sequential_baseline`` fixes the cheapest
chart and tunes only the accumulator; ``joint_search`` feeds the Cartesian product to the same selection harness
(choose on a development set, validate on a held-out set), so on the development set it can never do worse. All
trials of one plan are evaluated as one batched torch computation (``[trials, samples, 4]``); the accumulators are
applied per column through the scalar reference implementations so their rounding behaviour is exactly the tuned one.
Reference counterpart: scirust-core/src/representation_graph_quaternion.rs:81-420 (the quaternion type it uses lives in
scirust-simd/src/geometry/quaternion.rs).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .accumulate import NAIVE, AccumMethod, accumulate, autotune_by, default_accumulators


# ------------------------------------------------------------------ quaternion algebra, batched, (w, x, y, z) last
def q_normalize(q):
    return q / q.norm(dim=-1, keepdim=True).clamp_min(1e-300)


def q_conj(q):
    return q * q.new_tensor([1.0, -1.0, -1.0, -1.0])


def q_mul(a, b):
    aw, ax, ay, az = a.unbind(-1)
    bw, bx, by, bz = b.unbind(-1)
    return torch.stack([aw * bw - ax * bx - ay * by - az * bz,
                        aw * bx + ax * bw + ay * bz - az * by,
                        aw * by - ax * bz + ay * bw + az * bx,
                        aw * bz + ax * by - ay * bx + az * bw], -1)


def q_from_axis_angle(axis, angle):
    axis = torch.as_tensor(axis, dtype=torch.float64)
    angle = torch.as_tensor(angle, dtype=torch.float64)
    axis = axis / axis.norm(dim=-1, keepdim=True).clamp_min(1e-300)
    h = angle[..., None] * 0.5
    return torch.cat([h.cos(), axis * h.sin()], -1)


def log_relative(reference, q):
    """Tangent vector at ``reference`` whose exp map gives ``q`` (shorter arc: norm at most pi)."""
    d = q_mul(q_conj(reference), q)
    d = torch.where(d[..., :1] < 0, -d, d)
    v = d[..., 1:]
    s = v.norm(dim=-1, keepdim=True)
    angle = 2.0 * torch.atan2(s, d[..., :1])
    return torch.where(s > 1e-12, v / s.clamp_min(1e-300) * angle, 2.0 * v)


def exp_relative(reference, v):
    angle = v.norm(dim=-1, keepdim=True)
    h = angle * 0.5
    delta = torch.cat([h.cos(), torch.where(angle > 1e-12, v / angle.clamp_min(1e-300) * h.sin(), 0.5 * v)], -1)
    return q_mul(reference, delta)


def angular_error_degrees(a, b):
    """Rotation angle between two unit quaternions; q and -q are the same rotation."""
    d = (a * b).sum(-1).abs().clamp(max=1.0)
    return 2.0 * torch.acos(d) * (180.0 / math.pi)


# ------------------------------------------------------------------ the chart axis
@dataclass(frozen=True)
class Chart:
    kind: str                     # componentwise | log
    iterations: int = 0

    def name(self) -> str:
        return "componentwise" if self.kind == "componentwise" else f"log-chart(iters={self.iterations})"

    def cost(self) -> int:
        return 0 if self.kind == "componentwise" else 4 * self.iterations


COMPONENTWISE = Chart("componentwise")


def default_chart_dictionary():
    return [COMPONENTWISE, Chart("log", 2)]


def _column_means(accum: AccumMethod, cols: torch.Tensor) -> torch.Tensor:
    """``cols [trials, samples, k]`` -> ``[trials, k]``: every column summed in fp32 by ``accum``, divided by the count."""
    t, n, k = cols.shape
    arr = cols.to(torch.float32).numpy()
    out = np.empty((t, k))
    for i in range(t):
        for j in range(k):
            out[i, j] = float(accumulate(accum, arr[i, :, j])) / n
    return torch.from_numpy(out)


def average(chart: Chart, accum: AccumMethod, samples) -> torch.Tensor:
    """``samples [trials, n, 4]`` (or ``[n, 4]``) unit quaternions -> one estimate per trial."""
    q = torch.as_tensor(samples, dtype=torch.float64)
    single = q.dim() == 2
    q = q[None] if single else q
    ref = q[:, :1]
    q = torch.where(((q * ref).sum(-1, keepdim=True)) < 0, -q, q)               # one hemisphere: no cancellation
    if chart.kind == "componentwise":
        est = q_normalize(_column_means(accum, q))
    else:
        est = q_normalize(q.mean(1))
        for _ in range(chart.iterations):
            est = exp_relative(est, _column_means(accum, log_relative(est[:, None], q)))
    return est[0] if single else est


# ------------------------------------------------------------------ data
def noisy_trials(truth, sigma: float, trials: int, n: int, seed: int) -> torch.Tensor:
    """Each observation = (rotation by N(0, sigma) radians about a uniformly random axis) * truth."""
    g = torch.Generator().manual_seed(seed)
    axis = torch.randn(trials, n, 3, generator=g, dtype=torch.float64)
    angle = torch.randn(trials, n, generator=g, dtype=torch.float64) * sigma
    return q_mul(q_from_axis_angle(axis, angle), torch.as_tensor(truth, dtype=torch.float64).expand(trials, n, 4))


# ------------------------------------------------------------------ search
@dataclass(frozen=True)
class QuatPlan:
    chart: Chart
    accumulation: AccumMethod


@dataclass
class QuatSearchReport:
    plan: QuatPlan
    eval_mean_error_degrees: float


def score_plan(plan: QuatPlan, truth, _fit, score_on):
    """Negative mean angular error in degrees (higher is better); charts and accumulators have nothing to fit."""
    if score_on is None or len(score_on) == 0:
        return None
    est = average(plan.chart, plan.accumulation, score_on)
    return -float(angular_error_degrees(est, torch.as_tensor(truth, dtype=torch.float64)).mean())


def _base(truth):
    def f(fit, scr):
        s = score_plan(QuatPlan(COMPONENTWISE, NAIVE), truth, fit, scr)
        return -math.inf if s is None else s
    return f


def sequential_baseline(truth, dev, held_out, accumulators=None):
    out = autotune_by(dev, held_out, accumulators or default_accumulators(),
                      lambda a, fit, scr: score_plan(QuatPlan(COMPONENTWISE, a), truth, fit, scr), _base(truth))
    return None if out.chosen is None else QuatSearchReport(QuatPlan(COMPONENTWISE, out.chosen), -out.chosen_eval_score)


def joint_search(truth, dev, held_out, charts=None, accumulators=None):
    cands = [QuatPlan(c, a) for c in (charts or default_chart_dictionary()) for a in (accumulators or default_accumulators())]
    out = autotune_by(dev, held_out, cands, lambda p, fit, scr: score_plan(p, truth, fit, scr), _base(truth))
    return None if out.chosen is None else QuatSearchReport(out.chosen, -out.chosen_eval_score)

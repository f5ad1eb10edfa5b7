"""Post-hoc reliability tools behind the ``calibrate`` / ``conformal`` / ``certify`` commands of the
reference CLI (scirust-cli/src/lib.rs:653-760 lists them; the implementations live in its
``scirust-learning`` / ``scirust-core`` crates): temperature scaling with expected calibration error,
split conformal prediction sets, and interval-arithmetic output bounds for ReLU networks."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def expected_calibration_error(probs: torch.Tensor, labels: torch.Tensor, bins: int = 15) -> float:
    conf, pred = probs.max(-1)
    correct = (pred == labels).float()
    ece = 0.0
    edges = torch.linspace(0, 1, bins + 1)
    for lo, hi in zip(edges[:-1], edges[1:]):
        m = (conf > lo) & (conf <= hi)
        if m.any():
            ece += m.float().mean().item() * abs(correct[m].mean().item() - conf[m].mean().item())
    return ece


def fit_temperature(logits: torch.Tensor, labels: torch.Tensor, iters: int = 60) -> float:
    """Temperature T > 0 minimising the NLL of softmax(logits / T) (golden-section search on log T:
    deterministic, no optimiser state)."""
    def nll(log_t):
        return F.cross_entropy(logits.double() / math.exp(log_t), labels).item()
    lo, hi = math.log(0.05), math.log(20.0)
    g = (math.sqrt(5) - 1) / 2
    a, b = hi - g * (hi - lo), lo + g * (hi - lo)
    fa, fb = nll(a), nll(b)
    for _ in range(iters):
        if fa < fb:
            hi, b, fb = b, a, fa
            a = hi - g * (hi - lo)
            fa = nll(a)
        else:
            lo, a, fa = a, b, fb
            b = lo + g * (hi - lo)
            fb = nll(b)
    return math.exp((lo + hi) / 2)


def conformal_threshold(cal_probs: torch.Tensor, cal_labels: torch.Tensor, alpha: float = 0.1) -> float:
    """Split conformal: score = 1 - p(true class); returns the ceil((n+1)(1-alpha))/n empirical quantile."""
    scores = 1.0 - cal_probs.gather(1, cal_labels[:, None]).squeeze(1)
    n = scores.numel()
    k = min(n, math.ceil((n + 1) * (1 - alpha)))
    return float(torch.sort(scores).values[k - 1])


def conformal_sets(probs: torch.Tensor, threshold: float):
    """Prediction sets {y : 1 - p(y) <= threshold} as a boolean mask."""
    return (1.0 - probs) <= threshold


def interval_bounds(layers, lo: torch.Tensor, hi: torch.Tensor):
    """Sound output bounds of an affine/ReLU stack under the input box [lo, hi] (interval arithmetic).
    ``layers``: [(W [in, out], b [out]) ...], ReLU between consecutive layers."""
    for i, (w, b) in enumerate(layers):
        wp, wn = w.clamp(min=0), w.clamp(max=0)
        lo, hi = lo @ wp + hi @ wn + b, hi @ wp + lo @ wn + b
        if i + 1 < len(layers):
            lo, hi = lo.clamp(min=0), hi.clamp(min=0)
    return lo, hi

"""Attribution by integrated gradients (Sundararajan et al., 2017): the path integral of the model's gradient along
the straight line from a baseline to the input, times ``(input - baseline)``. All ``steps + 1`` interpolated inputs
go through the model as ONE batch (one forward, one backward), the Riemann average over the ``steps + 1`` points
``alpha = i / steps`` is the estimate. With a linear model the attributions equal ``w * (x - baseline)`` exactly, and
they sum (approximately, exactly in the limit) to ``f(x) - f(baseline)``: ``completeness_gap`` reports the difference.
Reference counterpart: scirust-core/src/xai.rs:8-41 (one tape per interpolation step).
"""
from __future__ import annotations

import torch


def integrated_gradients(input, baseline, steps: int, model_fn, batch: int | None = None) -> torch.Tensor:
    """``model_fn`` maps a batch ``[n, ...]`` to one scalar per row (or to a tensor that is summed per row)."""
    x = torch.as_tensor(input, dtype=torch.float32)
    b = torch.as_tensor(baseline, dtype=torch.float32, device=x.device)
    if x.shape != b.shape:
        raise ValueError("integrated_gradients: input and baseline shapes differ")
    if steps < 1:
        raise ValueError("integrated_gradients: steps must be >= 1")
    diff = x - b
    alphas = torch.arange(steps + 1, dtype=torch.float32, device=x.device) / steps
    total = torch.zeros_like(x)
    batch = batch or steps + 1
    for i in range(0, steps + 1, batch):
        a = alphas[i:i + batch].reshape(-1, *([1] * x.dim()))
        pts = (b[None] + a * diff[None]).detach().requires_grad_(True)
        out = model_fn(pts)
        out = out.reshape(out.shape[0], -1).sum()
        total += torch.autograd.grad(out, pts)[0].sum(0)
    return total / (steps + 1) * diff


def completeness_gap(attributions, input, baseline, model_fn) -> float:
    """``sum(attributions) - (f(input) - f(baseline))``: tends to 0 as the number of steps grows."""
    with torch.no_grad():
        pair = torch.stack([torch.as_tensor(input, dtype=torch.float32), torch.as_tensor(baseline, dtype=torch.float32)])
        f = model_fn(pair).reshape(2, -1).sum(1)
    return float(attributions.sum() - (f[0] - f[1]))

"""Certified (verified) training by differentiable interval bound propagation: the IBP end of the CROWN-IBP
schedule (Zhang et al., 2020). The network trains on a bound of the WORST-CASE loss over an L-infinity ball around
each input, so its certified radius grows instead of only its clean accuracy.

For ``y = x W + b`` a box (centre, radius) maps to ``(centre W + b, radius |W|)``; a ReLU maps ``[l, u]`` to
``[relu(l), relu(u)]``; the robust logits put the true class at its lower bound and every other class at its upper
bound, and a cross-entropy on those is small only if the true class wins everywhere in the ball. Both box products
of a layer are issued as one stacked product (centre and radius rows against ``W`` and ``|W|``) and everything is
differentiable, so the optimiser is any of the framework's. The bound is sound (never a false certificate) but
looser than a full CROWN back-substitution, which is not part of this trainer; ``to_ibp_mlp`` hands the weights to
the verifiers of ``scirust_b200.certify`` / ``scirust_b200.verify`` for measuring what was achieved.
Reference counterpart: scirust-core/src/nn/crown_ibp.rs:45-360 (N-D tape, ``|W| = relu(W) + relu(-W)``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..certify import IbpLinear, IbpMlp
from .rng import PcgEngine


class CrownIbpMlp(torch.nn.Module):
    def __init__(self, dims, rng: PcgEngine | None = None):
        super().__init__()
        if len(dims) < 2 or any(d <= 0 for d in dims):
            raise ValueError("CrownIbpMlp needs at least an input and an output width, all positive")
        rng = rng or PcgEngine(0)
        self.weights = torch.nn.ParameterList()
        self.biases = torch.nn.ParameterList()
        for a, b in zip(dims[:-1], dims[1:]):
            self.weights.append(torch.nn.Parameter(rng.fill_uniform_signed((a, b), 1.0 / math.sqrt(a))))
            self.biases.append(torch.nn.Parameter(torch.zeros(1, b)))

    @property
    def input_dim(self):
        return self.weights[0].shape[0]

    @property
    def output_dim(self):
        return self.weights[-1].shape[1]

    def forward(self, x):
        h = x
        for i, (w, b) in enumerate(zip(self.weights, self.biases)):
            h = h @ w + b
            if i + 1 < len(self.weights):
                h = torch.relu(h)
        return h

    @staticmethod
    def _check_eps(eps):
        if not math.isfinite(eps) or eps < 0.0:
            raise ValueError("certified IBP epsilon must be finite and >= 0")

    def ibp_propagate(self, x, eps: float):
        """(centre, radius) of the output box for the L-infinity ball of radius ``eps`` around each row of x."""
        centre, radius = x, torch.full_like(x, eps)
        n = len(self.weights)
        for i, (w, b) in enumerate(zip(self.weights, self.biases)):
            nc = centre @ w + b
            nr = radius @ w.abs()
            if i + 1 < n:
                lo, hi = torch.relu(nc - nr), torch.relu(nc + nr)
                centre, radius = 0.5 * (lo + hi), 0.5 * (hi - lo)
            else:
                centre, radius = nc, nr
        return centre, radius

    def robust_loss(self, x, eps: float, targets):
        self._check_eps(eps)
        if x.dim() != 2:
            raise ValueError(f"CrownIbpMlp robust_loss expects rank-2 input, got rank {x.dim()}")
        if x.shape[0] == 0:
            raise ValueError("CrownIbpMlp robust_loss requires a non-empty batch")
        if x.shape[1] != self.input_dim:
            raise ValueError(f"CrownIbpMlp input width mismatch: expected {self.input_dim}, got {x.shape[1]}")
        t = torch.as_tensor(targets, dtype=torch.int64, device=x.device).reshape(-1)
        if t.numel() != x.shape[0]:
            raise ValueError(f"CrownIbpMlp target count mismatch: expected {x.shape[0]}, got {t.numel()}")
        if int(t.max()) >= self.output_dim or int(t.min()) < 0:
            raise ValueError(f"CrownIbpMlp target class out of range for {self.output_dim} classes")
        centre, radius = self.ibp_propagate(x, eps)
        sign = torch.ones_like(centre).scatter_(1, t[:, None], -1.0)
        return F.cross_entropy(centre + radius * sign, t)

    @torch.no_grad()
    def certified_box(self, x, eps: float):
        self._check_eps(eps)
        x = torch.as_tensor(x, dtype=torch.float32).reshape(1, -1)
        if x.shape[1] != self.input_dim:
            raise ValueError(f"CrownIbpMlp certified_box input size mismatch: expected {self.input_dim}, got {x.shape[1]}")
        if not bool(torch.isfinite(x).all()):
            raise ValueError("CrownIbpMlp certified_box input must be finite")
        c, r = self.ibp_propagate(x.to(self.weights[0].device), eps)
        return (c - r)[0].cpu(), (c + r)[0].cpu()

    def to_ibp_mlp(self) -> IbpMlp:
        return IbpMlp([IbpLinear(w.detach().cpu(), b.detach().cpu()) for w, b in zip(self.weights, self.biases)])

    @torch.no_grad()
    def certified_accuracy(self, x, targets, eps: float) -> float:
        """Fraction of rows whose true class provably wins over the whole ball."""
        t = torch.as_tensor(targets, dtype=torch.int64, device=x.device)
        c, r = self.ibp_propagate(x, eps)
        lo_t = (c - r).gather(1, t[:, None])
        hi = (c + r).scatter(1, t[:, None], -math.inf)
        return float((lo_t.squeeze(1) > hi.max(1).values).float().mean())

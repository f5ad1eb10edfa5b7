"""Lipschitz certificates for linear heads: the spectral norm by power iteration (an estimate from below), a
sound upper bound ``sqrt(||W||_1 ||W||_inf)`` accumulated in float64 with a relative safety margin, spectral
normalisation, and the GloRo-style certificate: with ``L = sqrt(2) * sigma_max(W)`` bounding every logit
DIFFERENCE, the prediction cannot change inside the L2 ball of radius ``margin / L``.
Reference counterpart: scirust-core/src/nn/lipschitz.rs:37-347.
"""
from __future__ import annotations

import math

import torch


def _mat(w, rows=None, cols=None) -> torch.Tensor:
    t = torch.as_tensor(w, dtype=torch.float32)
    if rows is not None:
        if t.numel() != rows * cols:
            raise ValueError("spectral_norm: size mismatch")
        t = t.reshape(rows, cols)
    return t


def spectral_norm(w, rows=None, cols=None, iters: int = 50) -> float:
    """Largest singular value by ``iters`` rounds of power iteration from the uniform unit vector."""
    W = _mat(w, rows, cols)
    if W.numel() == 0:
        return 0.0
    v = torch.full((W.shape[1],), 1.0 / math.sqrt(W.shape[1]))
    sigma = 0.0
    for _ in range(iters):
        u = W @ v
        sigma = float(u.norm())
        vn = W.t() @ u
        nrm = float(vn.norm())
        if nrm <= 0.0:
            return 0.0
        v = vn / nrm
    return sigma


def spectral_norm_upper_bound(w, rows=None, cols=None) -> float:
    """``sigma_max <= sqrt(max row abs-sum * max column abs-sum)``, never below the true value after the
    narrowing to float32 (float64 sums, margin 1e-6 relative)."""
    W = _mat(w, rows, cols).double().abs()
    if W.numel() == 0:
        return 0.0
    bound = math.sqrt(float(W.sum(1).max()) * float(W.sum(0).max())) * (1.0 + 1e-6)
    return float(torch.tensor(bound, dtype=torch.float32))


def spectral_normalize(w, rows=None, cols=None, iters: int = 50) -> torch.Tensor:
    W = _mat(w, rows, cols)
    sn = spectral_norm(W, iters=iters)
    return W.clone() if sn <= 0.0 else W / sn


class GloroClassifier:
    """Linear classifier ``logits = W x`` (``W [classes, features]``) with a certified L2 radius per input."""

    def __init__(self, w, num_classes: int, in_features: int, iters: int = 50):
        if num_classes < 2:
            raise ValueError("GloRo certification requires at least two classes")
        if in_features == 0:
            raise ValueError("GloRo in_features must be > 0")
        W = torch.as_tensor(w, dtype=torch.float32)
        if W.numel() != num_classes * in_features:
            raise ValueError(f"GloRo weight size mismatch: expected {num_classes * in_features}, got {W.numel()}")
        if not bool(torch.isfinite(W).all()):
            raise ValueError("GloRo weights must be finite")
        self.w = W.reshape(num_classes, in_features)
        self.num_classes, self.in_features = num_classes, in_features
        self.lip = math.sqrt(2.0) * spectral_norm_upper_bound(self.w)
        self.lip_estimate = math.sqrt(2.0) * spectral_norm(self.w, iters=iters)

    def logits(self, x) -> torch.Tensor:
        x = torch.as_tensor(x, dtype=torch.float32)
        if x.shape[-1] != self.in_features:
            raise ValueError(f"GloRo input size mismatch: expected {self.in_features}, got {x.shape[-1]}")
        if not bool(torch.isfinite(x).all()):
            raise ValueError("GloRo input must contain only finite values")
        return x @ self.w.t()

    def certify(self, x):
        """(predicted class, certified radius >= 0) for one input; batched inputs give two tensors."""
        z = self.logits(x)
        top2 = z.topk(2, dim=-1)
        margin = top2.values[..., 0] - top2.values[..., 1]
        radius = (margin / self.lip).clamp_min(0) if self.lip > 0 else torch.zeros_like(margin)
        cls = z.argmax(-1)
        if z.dim() == 1:
            return int(cls), float(radius)
        return cls, radius

    def lipschitz(self) -> float:
        return self.lip

    def lipschitz_estimate(self) -> float:
        return self.lip_estimate

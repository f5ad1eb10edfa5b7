"""Verifying an inference ACROSS machines whose floating-point sums differ.

Bit-exact re-execution (``io/proof.py``) only works when the verifier reproduces the prover's arithmetic exactly; with
other vector widths, fused multiply-adds or thread counts an honest fp32 output differs in the last bits. DiFR recomputes
a canonical reference (products and sums in float64: order-independent to far below fp32 resolution) and accepts a claimed
output iff it lies inside a SOUND error envelope of it: per layer the dot-product rounding bound
``slack * (n + 1) * u * (sum |w_i x_i| + |b|)`` plus the propagated input error ``sum |w_i| delta_i`` (ReLU is 1-Lipschitz,
so it passes the bound through). Any fp32 evaluation in any summation order is inside the envelope; the envelope is a
few parts per million of the activation scale, so meaningful tampering is outside it.
Whole BATCHES of claims are verified in one pass of float64 matrix products on the tensors' device.
Reference counterpart: scirust-runtime/src/difr.rs:25-236 (one input vector, scalar loops, ``reproducible_dot``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

DEFAULT_SLACK = 4.0
F32_U = 2.0 ** -24


@dataclass
class DifrLayer:
    w: torch.Tensor          # [in, out]
    b: torch.Tensor          # [out]

    @property
    def in_f(self):
        return self.w.shape[0]

    @property
    def out_f(self):
        return self.w.shape[1]


@dataclass
class DifrVerdict:
    accepted: bool
    reference: torch.Tensor
    envelope: torch.Tensor
    deviation: torch.Tensor
    accepted_rows: torch.Tensor | None = None


@torch.no_grad()
def difr_verify(layers, inputs, claimed, slack: float = DEFAULT_SLACK) -> DifrVerdict:
    """``inputs [in]`` or ``[batch, in]``; ``claimed`` of matching shape. ReLU after every layer but the last."""
    x = torch.as_tensor(inputs, dtype=torch.float32)
    single = x.dim() == 1
    ref = x.reshape(1, -1).double() if single else x.double()
    delta = torch.zeros_like(ref)
    for li, l in enumerate(layers):
        if ref.shape[1] != l.in_f:
            raise ValueError("difr: layer input width mismatch")
        w, b = l.w.double().to(ref.device), l.b.double().to(ref.device)
        out = (ref @ w + b).float().double()                                  # canonical value, rounded to fp32 once
        scale = ref.abs() @ w.abs() + b.abs()
        delta = slack * (l.in_f + 1.0) * F32_U * scale + delta @ w.abs()
        ref = out.clamp_min(0) if li + 1 < len(layers) else out
    c = torch.as_tensor(claimed, dtype=torch.float32).reshape(ref.shape).double().to(ref.device)
    dev = (c - ref).abs()
    rows = (dev <= delta).all(1)
    fin = torch.isfinite(c).all(1)
    rows = rows & fin
    sq = (lambda t: t[0].float()) if single else (lambda t: t.float())
    return DifrVerdict(bool(rows.all()), sq(ref), sq(delta), sq(dev), None if single else rows)

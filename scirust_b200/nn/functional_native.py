"""Autograd wrappers over native kernels for callers that hold plain tensors (the N-D tape, layer zoo)."""
from __future__ import annotations

import torch

from .. import ops


class _RmsUnit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        w = torch.ones(shape[-1], dtype=x.dtype, device=x.device)
        y, inv = ops.rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, w, inv)
        ctx.shape = shape
        return y.reshape(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, inv = ctx.saved_tensors
        dx, _ = ops.rmsnorm_bwd(dy.reshape(x2.shape).contiguous(), x2, w, inv)
        return dx.reshape(ctx.shape), None


def rmsnorm_unit_gain(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis on the native RMSNorm kernels (bf16 CUDA tensors)."""
    return _RmsUnit.apply(x, eps)

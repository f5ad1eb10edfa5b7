"""Linear layers fused with what follows them: ``matmul_silu``, ``matmul_relu``, ``matmul_gelu`` (tanh form),
``matmul_layernorm``, ``matmul_silu_layernorm`` (a two-layer MLP block) and ``matmul_scale``. ``x [batch, in]``,
``w [in, out]`` (the framework's x.W layout), ``bias [out]``.

On CUDA bf16 operands the product runs on the tcgen05 GEMM (``scirust_b200.ops.gemm``) and the activation /
normalisation is applied to its output rows; elsewhere one fp32 statement. The op-graph pass that finds these
patterns is ``scirust_b200.fusion``. Reference counterpart: scirust-core/src/nn/fused_ops.rs:22-276 (scalar CPU
loops; ``FusedKernelOp`` lists the same six).
"""
from __future__ import annotations

import enum
import math

import torch
import torch.nn.functional as F


class FusedKernelOp(enum.Enum):
    MATMUL_SILU = "matmul_silu"
    MATMUL_RELU = "matmul_relu"
    MATMUL_GELU = "matmul_gelu"
    MATMUL_LAYERNORM = "matmul_layernorm"
    MATMUL_SILU_LAYERNORM = "matmul_silu_layernorm"
    MATMUL_SCALE = "matmul_scale"


def _affine(x, w, bias):
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from ..ops import gemm as G
        y = G.matmul_nn(x.contiguous(), w.contiguous()).float()
    else:
        y = x.float() @ w.float()
    return y if bias is None else y + bias.float().reshape(1, -1)


def _layernorm(y, gamma, beta, eps):
    mean = y.mean(-1, keepdim=True)
    var = ((y - mean) ** 2).mean(-1, keepdim=True)
    return (y - mean) / torch.sqrt(var + eps) * gamma.float() + beta.float()


def matmul_silu(x, w, bias=None):
    return F.silu(_affine(x, w, bias))


def matmul_relu(x, w, bias=None):
    return _affine(x, w, bias).clamp_min(0)


def gelu_tanh(y):
    return 0.5 * y * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (y + 0.044715 * y ** 3)))


def matmul_gelu(x, w, bias=None):
    return gelu_tanh(_affine(x, w, bias))


def matmul_layernorm(x, w, bias, gamma, beta, eps: float = 1e-5):
    return _layernorm(_affine(x, w, bias), gamma, beta, eps)


def matmul_silu_layernorm(x, w1, w2, b1, b2, gamma, beta, eps: float = 1e-5):
    h = F.silu(_affine(x, w1, b1))
    return _layernorm(_affine(h.to(x.dtype), w2, b2), gamma, beta, eps)


def matmul_scale(x, w, scale):
    """``(x w) * scale`` with a per-output-column ``scale`` (or one scalar)."""
    s = torch.as_tensor(scale, dtype=torch.float32, device=x.device)
    return _affine(x, w, None) * (s.reshape(1, -1) if s.dim() else s)


def run(op: FusedKernelOp, *args, **kw):
    return {FusedKernelOp.MATMUL_SILU: matmul_silu, FusedKernelOp.MATMUL_RELU: matmul_relu,
            FusedKernelOp.MATMUL_GELU: matmul_gelu, FusedKernelOp.MATMUL_LAYERNORM: matmul_layernorm,
            FusedKernelOp.MATMUL_SILU_LAYERNORM: matmul_silu_layernorm,
            FusedKernelOp.MATMUL_SCALE: matmul_scale}[op](*args, **kw)

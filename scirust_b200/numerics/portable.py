"""Bit-portable fp32 elementary functions and GEMM (scirust-core/src/portable_f32.rs:88, 1005,
1033, 1058). The reference defines ``exp_f32`` / ``ln_f32`` / ``tanh_f32`` / ``sigmoid_f32`` as the
*correctly rounded* fp32 results (fp64 evaluation plus tables for the hard cases), which makes the
answer a mathematical fact independent of any libm. Here the same values are obtained by an fp64
evaluation whose result is re-decided with 60-digit decimal arithmetic whenever it lies close to
an fp32 rounding boundary. ``softmax_f32`` composes ``exp_f32`` with the order-independent sum;
``gemm_f32`` accumulates exact products in fp64 in ascending k and rounds once."""
from __future__ import annotations

import ctypes as C
import decimal
import math

import numpy as np
import torch

from ..ops import _lib
from .reproducible import reproducible_sum

_CTX = decimal.Context(prec=60)


def _round_f32_checked(x64: float, exact_fn) -> np.float32:
    """Round an fp64 approximation to fp32, re-deciding near-ties with ``exact_fn() -> Decimal``."""
    f = np.float32(x64)
    if not np.isfinite(f) or f == 0:
        return f
    lo = np.nextafter(f, np.float32(-np.inf), dtype=np.float32)
    hi = np.nextafter(f, np.float32(np.inf), dtype=np.float32)
    for nb in (lo, hi):
        mid = (float(f) + float(nb)) / 2.0
        if abs(x64 - mid) <= abs(mid) * 1e-13:
            ex = exact_fn()
            dm = decimal.Decimal(mid)
            if ex == dm:
                return f  # exact tie cannot occur for transcendental results; keep nearest-even pick
            closer_to_f = (ex > dm) == (float(f) > mid)
            return f if closer_to_f else np.float32(nb)
    return f


def exp_f32(x) -> np.float32:
    x = np.float32(x)
    if np.isnan(x):
        return np.float32(np.nan)
    if x >= 89.0:
        return np.float32(np.inf)
    if x <= -105.0:
        return np.float32(0.0)
    return _round_f32_checked(math.exp(float(x)), lambda: _CTX.exp(decimal.Decimal(float(x))))


def ln_f32(x) -> np.float32:
    x = np.float32(x)
    if np.isnan(x) or x < 0:
        return np.float32(np.nan)
    if x == 0:
        return np.float32(-np.inf)
    if np.isinf(x):
        return np.float32(np.inf)
    return _round_f32_checked(math.log(float(x)), lambda: _CTX.ln(decimal.Decimal(float(x))))


def sigmoid_f32(x) -> np.float32:
    x = np.float32(x)
    if np.isnan(x):
        return np.float32(np.nan)
    if x >= 30.0:
        return np.float32(1.0)
    if x <= -120.0:
        return np.float32(0.0)
    y = float(x)

    def exact():
        e = _CTX.exp(decimal.Decimal(-y))
        return _CTX.divide(decimal.Decimal(1), _CTX.add(decimal.Decimal(1), e))
    approx = 1.0 / (1.0 + math.exp(-y)) if y >= 0 else math.exp(y) / (1.0 + math.exp(y))
    return _round_f32_checked(approx, exact)


def tanh_f32(x) -> np.float32:
    x = np.float32(x)
    if np.isnan(x):
        return np.float32(np.nan)
    if abs(x) >= 10.0:
        return np.float32(math.copysign(1.0, float(x)))
    y = float(x)

    def exact():
        e2 = _CTX.exp(decimal.Decimal(2 * y))
        return _CTX.divide(_CTX.subtract(e2, decimal.Decimal(1)), _CTX.add(e2, decimal.Decimal(1)))
    return _round_f32_checked(math.tanh(y), exact)


def softmax_f32(xs) -> np.ndarray:
    xs = np.asarray(xs, dtype=np.float32)
    m = np.float32(-np.inf)
    for v in xs:
        m = max(m, v)
    e = np.array([exp_f32(np.float32(v - m)) for v in xs], dtype=np.float32)
    s = np.float32(reproducible_sum(e))
    return (e / s).astype(np.float32)


def dot_f32(a, b) -> np.float32:
    acc = 0.0
    for x, y in zip(np.asarray(a, dtype=np.float32).tolist(), np.asarray(b, dtype=np.float32).tolist()):
        acc += x * y
    return np.float32(acc)


def gemm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    a = a.detach().float().cpu().contiguous()
    b = b.detach().float().cpu().contiguous()
    M, K = a.shape
    K2, N = b.shape
    if K != K2:
        raise ValueError("gemm_f32: inner dimensions differ")
    lib = _lib.rt()
    lib.sbrt_gemm_f32_portable.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
    lib.sbrt_gemm_f32_portable.restype = None
    c = torch.empty((M, N), dtype=torch.float32)
    lib.sbrt_gemm_f32_portable(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, K, N)
    return c


class PortableExp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = torch.tensor([float(exp_f32(v)) for v in x.detach().cpu().reshape(-1).tolist()],
                         dtype=torch.float32).reshape(x.shape).to(x.device)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return g * y


class PortableMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm_f32(a, b).to(a.device)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        return gemm_f32(g, b.t().contiguous()).to(a.device), gemm_f32(a.t().contiguous(), g).to(a.device)


class PortableLn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = torch.tensor([float(ln_f32(v)) for v in x.detach().cpu().reshape(-1).tolist()],
                         dtype=torch.float32).reshape(x.shape).to(x.device)
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return g / x


class PortableSoftmax(torch.autograd.Function):
    """Row softmax through the libm-free kernels; the vector-Jacobian product is ``y * (g - sum(g * y))``."""

    @staticmethod
    def forward(ctx, x):
        rows = [softmax_f32(r) for r in x.detach().cpu().numpy()]
        y = torch.tensor(np.stack(rows), dtype=torch.float32).to(x.device)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, g):
        (y,) = ctx.saved_tensors
        return y * (g - (g * y).sum(1, keepdim=True))

"""Canonical operator set with bit-exact agreement between the CPU statement and the CUDA kernels
(scirust-gpu/src/cuda_reference.rs:498-520, 684-890): relu, scale, add, sub, mul, div, shape-copy and
permute over fp32 tensors. ``exp`` and ``log`` are refused, as in the reference: no implementation of
them is bit-reproducible across targets.

``run(op, *operands, **attrs)`` executes on the operands' device; on CPU tensors it is the plain
statement that the GPU tests compare against word for word.
"""
from __future__ import annotations

import ctypes as C
import struct

import torch

from . import _lib
from . import gemm as _g

OPS = {"relu": 0, "scale": 1, "add": 2, "sub": 3, "mul": 4, "div": 5, "copy": 6}
ARITY = {"relu": 1, "scale": 1, "copy": 1, "permute": 1, "add": 2, "sub": 2, "mul": 2, "div": 2}

_lib.register("sb_canon_elementwise", [_lib.i32, _lib.vp, _lib.vp, _lib.vp, C.c_longlong, C.c_uint32, _lib.vp])
_lib.register("sb_canon_permute", [_lib.vp, _lib.vp, _lib.i32, _lib.vp, _lib.vp, _lib.vp])


class Unsupported(ValueError):
    pass


def _f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _cpu(op, a, b, factor, perm, shape):
    if op == "relu":
        # NaN and strictly positive values pass through untouched; -0.0 becomes +0.0
        keep = torch.isnan(a) | (a > 0)
        return torch.where(keep, a, torch.zeros_like(a))
    if op == "scale":
        return a * torch.tensor(factor, dtype=torch.float32)
    if op == "add":
        return a + b
    if op == "sub":
        return a - b
    if op == "mul":
        return a * b
    if op == "div":
        return a / b
    if op == "copy":
        return a.reshape(shape if shape is not None else a.shape).clone()
    return a.permute(perm).contiguous()


def run(op: str, a: torch.Tensor, b: torch.Tensor | None = None, *, factor: float = 1.0, perm=None, shape=None):
    """One canonical operator on fp32 tensors. ``copy`` may carry a new ``shape`` of the same size."""
    if op in ("exp", "log"):
        raise Unsupported("exp and log have no bit-reproducible implementation and are not executed")
    if op not in ARITY:
        raise Unsupported(f"no canonical kernel for {op!r}")
    if a.dtype != torch.float32 or (b is not None and b.dtype != torch.float32):
        raise ValueError("canonical operators take fp32 tensors")
    if ARITY[op] == 2 and (b is None or b.shape != a.shape):
        raise ValueError(f"{op} takes two operands of one shape")
    if op == "permute" and sorted(perm) != list(range(a.dim())):
        raise ValueError("perm must be a permutation of the axes")
    if not a.is_cuda:
        return _cpu(op, a, b, factor, perm, shape)
    a = a.contiguous()
    if op == "permute":
        out = _lib.empty([a.shape[p] for p in perm], torch.float32, a.device)
        shp = (C.c_longlong * a.dim())(*a.shape)
        prm = (C.c_int * a.dim())(*perm)
        _lib.call("sb_canon_permute", a.data_ptr(), out.data_ptr(), a.dim(), C.addressof(shp), C.addressof(prm),
                  _lib.stream())
    else:
        out = _lib.empty(shape if (op == "copy" and shape is not None) else a.shape, torch.float32, a.device)
        if out.numel() != a.numel():
            raise ValueError("copy keeps the number of elements")
        bb = b.contiguous() if b is not None else None
        _lib.call("sb_canon_elementwise", OPS[op], a.data_ptr(), _lib.ptr(bb), out.data_ptr(), a.numel(),
                  _f32_bits(factor), _lib.stream())
    _g.launch_count += 1
    return out

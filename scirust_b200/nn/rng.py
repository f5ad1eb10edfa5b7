"""Seeded generators with the reference's exact streams.

``PcgEngine`` is PCG-XSH-RR 64/32 with the reference's ``float`` / ``float_signed`` / Box-Muller
``normal`` draws (scirust-core/src/nn/rng.rs:9-53); the fp32 arithmetic runs in the native CPU
runtime so that a seed reproduces the same weights bit for bit. ``Philox4x32`` is the counter-based
generator of scirust-core/src/philox.rs:24-201 (random access: value = f(seed, stream, index)).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ..ops import _lib


class _PcgState(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


_configured = False


def _rt():
    global _configured
    lib = _lib.rt()
    if not _configured:
        P = C.POINTER(_PcgState)
        lib.sbrt_pcg_new.argtypes = [P, C.c_uint64]
        lib.sbrt_pcg_new.restype = None
        lib.sbrt_pcg_next_u32.argtypes = [P]
        lib.sbrt_pcg_next_u32.restype = C.c_uint32
        for f in ("sbrt_pcg_float", "sbrt_pcg_float_signed"):
            getattr(lib, f).argtypes = [P]
            getattr(lib, f).restype = C.c_float
        lib.sbrt_pcg_normal.argtypes = [P, C.c_float, C.c_float]
        lib.sbrt_pcg_normal.restype = C.c_float
        lib.sbrt_pcg_fill_normal.argtypes = [P, C.c_float, C.c_float, C.c_void_p, C.c_size_t]
        lib.sbrt_pcg_fill_normal.restype = None
        lib.sbrt_pcg_fill_uniform_signed.argtypes = [P, C.c_float, C.c_void_p, C.c_size_t]
        lib.sbrt_pcg_fill_uniform_signed.restype = None
        lib.sbrt_pcg_fill_float.argtypes = [P, C.c_void_p, C.c_size_t]
        lib.sbrt_pcg_fill_float.restype = None
        lib.sbrt_pcg_shuffle.argtypes = [P, C.c_void_p, C.c_size_t]
        lib.sbrt_pcg_shuffle.restype = None
        lib.sbrt_philox4x32_10.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        lib.sbrt_philox4x32_10.restype = None
        _configured = True
    return lib


class PcgEngine:
    def __init__(self, seed: int):
        self._s = _PcgState()
        _rt().sbrt_pcg_new(C.byref(self._s), seed & 0xFFFFFFFFFFFFFFFF)

    def clone(self) -> "PcgEngine":
        e = PcgEngine.__new__(PcgEngine)
        e._s = _PcgState(self._s.state, self._s.inc)
        return e

    def next_u32(self) -> int:
        return int(_rt().sbrt_pcg_next_u32(C.byref(self._s)))

    def float(self) -> float:
        return float(_rt().sbrt_pcg_float(C.byref(self._s)))

    def float_signed(self) -> float:
        return float(_rt().sbrt_pcg_float_signed(C.byref(self._s)))

    def normal(self, mean: float = 0.0, stddev: float = 1.0) -> float:
        return float(_rt().sbrt_pcg_normal(C.byref(self._s), mean, stddev))

    def fill_normal(self, shape, mean: float = 0.0, stddev: float = 1.0) -> torch.Tensor:
        t = torch.empty(shape, dtype=torch.float32)
        _rt().sbrt_pcg_fill_normal(C.byref(self._s), mean, stddev, t.data_ptr(), t.numel())
        return t

    def fill_uniform_signed(self, shape, bound: float) -> torch.Tensor:
        t = torch.empty(shape, dtype=torch.float32)
        _rt().sbrt_pcg_fill_uniform_signed(C.byref(self._s), bound, t.data_ptr(), t.numel())
        return t

    def fill_float(self, shape) -> torch.Tensor:
        t = torch.empty(shape, dtype=torch.float32)
        _rt().sbrt_pcg_fill_float(C.byref(self._s), t.data_ptr(), t.numel())
        return t

    def shuffle(self, n: int) -> torch.Tensor:
        """Fisher-Yates permutation of range(n) driven by the u32 stream."""
        idx = torch.arange(n, dtype=torch.int64)
        _rt().sbrt_pcg_shuffle(C.byref(self._s), idx.data_ptr(), n)
        return idx


class Philox4x32:
    def __init__(self, seed: int):
        self.key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint32)

    def block(self, counter) -> np.ndarray:
        c = np.asarray(counter, dtype=np.uint32)
        out = np.empty(4, dtype=np.uint32)
        _rt().sbrt_philox4x32_10(c.ctypes.data, self.key.ctypes.data, out.ctypes.data)
        return out

    def u32_at(self, stream: int, index: int) -> int:
        i = index // 4
        return int(self.block([i & 0xFFFFFFFF, (i >> 32) & 0xFFFFFFFF, stream, 0])[index % 4])

    def f32_at(self, stream: int, index: int) -> float:
        return float(np.float32(self.u32_at(stream, index) >> 8) * np.float32(1.0 / 16777216.0))

    def fill_f32(self, stream: int, start: int, n: int) -> np.ndarray:
        return np.array([self.f32_at(stream, start + j) for j in range(n)], dtype=np.float32)

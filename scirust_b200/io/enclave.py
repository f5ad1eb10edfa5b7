"""Length-checked raw-buffer inference (``csrc/rt_enclave.cpp``): the entry point a C host or a trusted-execution shim
calls with pointers. Every buffer travels with its element count, the counts are checked against the layout before any
pointer is touched, output may not alias an input, and the pointer-only predecessor always refuses.
``EnclaveRuntime.infer`` is the safe wrapper; ``raw_infer_v1`` exposes the ABI itself (for tests of the refusals).
Reference counterpart: scirust-runtime/src/enclave.rs:24-300.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ..ops import _lib

OK, ERR_NULL, ERR_LENGTH, ERR_OVERFLOW, ERR_VERSION, ERR_FLAG, ERR_LEGACY, ERR_ALIAS = range(8)
ABI_VERSION = 1
_NAMES = {ERR_NULL: "null pointer", ERR_LENGTH: "buffer length does not match the layout", ERR_OVERFLOW: "layout overflows",
          ERR_VERSION: "unknown ABI version", ERR_FLAG: "invalid bias flag", ERR_LEGACY: "pointer-only entry point is closed",
          ERR_ALIAS: "output overlaps an input"}


class EnclaveLayout(C.Structure):
    _fields_ = [("batch", C.c_size_t), ("in_features", C.c_size_t), ("out_features", C.c_size_t), ("has_bias", C.c_uint8)]

    @staticmethod
    def new(batch: int, in_features: int, out_features: int, has_bias: bool) -> "EnclaveLayout":
        return EnclaveLayout(batch, in_features, out_features, int(bool(has_bias)))

    def uses_bias(self) -> bool:
        return self.has_bias == 1


class EnclaveError(RuntimeError):
    def __init__(self, code: int):
        super().__init__(f"enclave inference refused: {_NAMES.get(code, 'error')} (code {code})")
        self.code = code


_ready = False


def _rt():
    global _ready
    lib = _lib.rt()
    if not _ready:
        fp = C.POINTER(C.c_float)
        lib.sbrt_enclave_infer_v1.argtypes = [C.c_uint32, fp, C.c_size_t, fp, C.c_size_t, fp, C.c_size_t, fp, C.c_size_t, EnclaveLayout]
        lib.sbrt_enclave_infer_v1.restype = C.c_int32
        lib.sbrt_enclave_infer.argtypes = [fp, fp, fp, fp, EnclaveLayout]
        lib.sbrt_enclave_infer.restype = C.c_int32
        lib.sbrt_enclave_abi_version.restype = C.c_uint32
        _ready = True
    return lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def raw_infer_v1(version, weights, weights_len, inp, input_len, out, output_len, bias, bias_len, dims: EnclaveLayout) -> int:
    """The ABI as a C caller sees it: arrays (or None) with separately stated element counts."""
    return int(_rt().sbrt_enclave_infer_v1(version, _p(weights), weights_len, _p(inp), input_len, _p(out), output_len,
                                           _p(bias), bias_len, dims))


def legacy_infer(weights, inp, out, bias, dims: EnclaveLayout) -> int:
    return int(_rt().sbrt_enclave_infer(_p(weights), _p(inp), _p(out), _p(bias), dims))


def abi_version() -> int:
    return int(_rt().sbrt_enclave_abi_version())


class EnclaveRuntime:
    def infer(self, weights, inp, bias=None, dims: EnclaveLayout | None = None) -> np.ndarray:
        """``weights [out, in]``, ``inp [batch, in]`` -> ``[batch, out]`` (fp32, fixed accumulation order)."""
        w = np.ascontiguousarray(weights, dtype=np.float32)
        x = np.ascontiguousarray(inp, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        if dims is None:
            if w.ndim != 2 or x.ndim != 2:
                raise ValueError("give 2-D weights and inputs, or an explicit layout")
            dims = EnclaveLayout.new(x.shape[0], w.shape[1], w.shape[0], b is not None)
        out = np.empty(dims.batch * dims.out_features, dtype=np.float32)
        code = raw_infer_v1(ABI_VERSION, w, w.size, x, x.size, out, out.size, b, 0 if b is None else b.size, dims)
        if code != OK:
            raise EnclaveError(code)
        return out.reshape(dims.batch, dims.out_features)

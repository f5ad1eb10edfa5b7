"""Host (CPU) transformer kernels of the native runtime (csrc/rt_cpu_kernels.cpp): blockwise flash attention, the
W8A8 dynamic linear layer, an int8 decoder block and a KV cache with fp32 or int8 rows.

They stand where the reference has its SIMD crate (scirust-simd/src/attention.rs:194-389, qtransformer.rs:99-229,
kv_cache.rs, quant.rs): the same arithmetic as one portable C++ statement, thread-count independent, used as oracles
for the device kernels and for deployments without a GPU. Inputs and outputs are contiguous fp32 CPU tensors."""
from __future__ import annotations

import ctypes as C
import os

import torch

from .ops import _lib

_cfg = False
i64, f32, vp, i32 = C.c_int64, C.c_float, C.c_void_p, C.c_int


def _rt():
    global _cfg
    lib = _lib.rt()
    if not _cfg:
        lib.sbrt_flash_attention_f32.argtypes = [vp, vp, vp, vp, i64, i64, i32, i32, i32, i32, i32, i32]
        lib.sbrt_w8a8_linear.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, vp, i32]
        lib.sbrt_int8_decoder_block.argtypes = [vp, vp, i64, i32, i32, i32, i32, f32, f32, vp, vp] + [vp] * 14 + [i32]
        lib.sbrt_kv_new.restype = vp
        lib.sbrt_kv_new.argtypes = [i32, i64, i32]
        lib.sbrt_kv_free.argtypes = [vp]
        lib.sbrt_kv_len.argtypes = [vp]
        lib.sbrt_kv_len.restype = i64
        lib.sbrt_kv_bytes.argtypes = [vp]
        lib.sbrt_kv_bytes.restype = i64
        lib.sbrt_kv_append.argtypes = [vp, vp, vp]
        lib.sbrt_kv_attend.argtypes = [vp, vp, vp, i32]
        lib.sbrt_sos_filter_f64.argtypes = [vp, i32, vp, vp, vp, i64, i64, i32]
        _cfg = True
    return lib


def _threads(n):
    return int(n) if n else min(8, os.cpu_count() or 1)


def _f(t):
    return torch.as_tensor(t, dtype=torch.float32).contiguous()


def flash_attention(q, k, v, causal: bool = True, block: int = 64, threads: int = 0) -> torch.Tensor:
    """``q [B, S, H, dh]``, ``k`` / ``v [B, S, Hkv, dh]`` -> ``[B, S, H, dh]``."""
    q, k, v = _f(q), _f(k), _f(v)
    B, S, H, dh = q.shape
    out = torch.empty_like(q)
    rc = _rt().sbrt_flash_attention_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, S, H, k.shape[2],
                                        dh, int(causal), block, _threads(threads))
    if rc:
        raise ValueError("flash_attention: bad shapes")
    return out


def quantize_weight(w):
    """``w [K, N]`` fp32 -> (int8 codes, fp32 per-column scales), round half away from zero."""
    w = _f(w)
    amax = w.abs().amax(0)
    s = torch.where(amax == 0, torch.ones_like(amax), amax / 127.0)
    v = w / s
    q = torch.where(v >= 0, torch.floor(v + 0.5), torch.ceil(v - 0.5)).clamp(-128, 127).to(torch.int8)
    return q.contiguous(), s.contiguous()


def w8a8_linear(x, wq, w_scale, bias=None, threads: int = 0) -> torch.Tensor:
    x = _f(x)
    M, K = x.shape
    N = wq.shape[1]
    y = torch.empty((M, N), dtype=torch.float32)
    b = _f(bias) if bias is not None else None
    rc = _rt().sbrt_w8a8_linear(x.data_ptr(), wq.data_ptr(), w_scale.data_ptr(), b.data_ptr() if b is not None else None,
                                y.data_ptr(), M, K, N, None, _threads(threads))
    if rc:
        raise ValueError("w8a8_linear: bad shapes")
    return y


class Int8DecoderBlock:
    """Quantises the seven matrices of a decoder block once; ``forward(x [S, d])`` runs the block in C++."""

    def __init__(self, n_heads, n_kv_heads, theta, eps, g1, g2, wq, wk, wv, wo, wg, wu, wd):
        self.H, self.Hkv, self.theta, self.eps = n_heads, n_kv_heads, float(theta), float(eps)
        self.g1, self.g2 = _f(g1).reshape(-1), _f(g2).reshape(-1)
        self.q = [quantize_weight(w) for w in (wq, wk, wv, wo, wg, wu, wd)]
        self.d, self.ff = wq.shape[0], wg.shape[1]

    def forward(self, x, threads: int = 0) -> torch.Tensor:
        x = _f(x)
        out = torch.empty_like(x)
        args = []
        for codes, scale in self.q:
            args += [codes.data_ptr(), scale.data_ptr()]
        rc = _rt().sbrt_int8_decoder_block(x.data_ptr(), out.data_ptr(), x.shape[0], self.d, self.H, self.Hkv, self.ff,
                                           self.theta, self.eps, self.g1.data_ptr(), self.g2.data_ptr(), *args,
                                           _threads(threads))
        if rc:
            raise ValueError("Int8DecoderBlock: bad shapes")
        return out


class NativeKvCache:
    """One head's keys and values in native memory: fp32 rows or int8 rows with one scale per row."""

    def __init__(self, dim: int, capacity: int, quantized: bool = False):
        self._lib = _rt()
        self._h = self._lib.sbrt_kv_new(dim, capacity, int(quantized))
        if not self._h:
            raise ValueError("dim and capacity must be positive")
        self.dim = dim

    def append(self, k, v) -> None:
        k, v = _f(k).reshape(-1), _f(v).reshape(-1)
        if k.numel() != self.dim or v.numel() != self.dim:
            raise ValueError("row has the wrong dimension")
        if self._lib.sbrt_kv_append(self._h, k.data_ptr(), v.data_ptr()):
            raise MemoryError("KV cache is full")

    def attend(self, q, block: int = 64) -> torch.Tensor:
        q = _f(q).reshape(-1)
        out = torch.empty(self.dim, dtype=torch.float32)
        if self._lib.sbrt_kv_attend(self._h, q.data_ptr(), out.data_ptr(), block):
            raise ValueError("attention over an empty cache")
        return out

    def __len__(self):
        return int(self._lib.sbrt_kv_len(self._h))

    def nbytes(self) -> int:
        return int(self._lib.sbrt_kv_bytes(self._h))

    def __del__(self):
        try:
            if self._h:
                self._lib.sbrt_kv_free(self._h)
                self._h = None
        except Exception:
            pass


def sos_filter_native(sos, x, state, threads: int = 0) -> torch.Tensor:
    """Cascade of second-order sections (direct form I) over the rows of ``x [rows, n]`` (float64); ``sos [sections, 5]``
    = (b0, b1, b2, a1, a2); ``state [rows, sections, 4]`` is read and updated in place (it must be contiguous)."""
    assert x.dtype == torch.float64 and sos.dtype == torch.float64 and state.dtype == torch.float64
    assert x.is_contiguous() and sos.is_contiguous() and state.is_contiguous()
    y = torch.empty_like(x)
    _rt().sbrt_sos_filter_f64(sos.data_ptr(), sos.shape[0], x.data_ptr(), y.data_ptr(), state.data_ptr(), x.shape[0],
                              x.shape[1], _threads(threads))
    return y

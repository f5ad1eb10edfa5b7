"""Token sampling with the reference's decode policy and RNG stream
(scirust-sciagent/src/generate.rs:10-36, 202-337): repetition penalty -> greedy arg-max when
``temperature <= 0`` -> ``softmax(logits / T)`` -> top-k -> top-p -> renormalise -> inverse-CDF draw
from a splitmix64-seeded xorshift64 stream. One ``sample_row`` serves every decoder (CPU, CUDA,
paged, tensor-parallel) so a seed gives the same tokens on all of them. Token 0 is the stop id.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from .ops import _lib

_M64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    repetition_window: int = 64


def seed_to_state(seed: int) -> int:
    z = (seed + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return z if z != 0 else 0x9E3779B97F4A7C15


class SamplerRng:
    """xorshift64 state shared across calls (mutated by ``sample_row``)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed_to_state(seed))

    def next_uniform(self) -> float:
        lib = _lib.rt()
        lib.sbrt_next_uniform.argtypes = [C.POINTER(C.c_uint64)]
        lib.sbrt_next_uniform.restype = C.c_float
        return float(lib.sbrt_next_uniform(C.byref(self.state)))


_cfg = False


def sample_row(logits, params: SamplingParams, recent, rng: SamplerRng) -> int:
    """Pick the next token from one ``[vocab]`` logits row."""
    global _cfg
    lib = _lib.rt()
    if not _cfg:
        lib.sbrt_sample_row.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_int64, C.c_float, C.c_float,
                                        C.c_int64, C.c_void_p, C.c_int64, C.POINTER(C.c_uint64)]
        lib.sbrt_sample_row.restype = C.c_int64
        _cfg = True
    row = torch.as_tensor(logits).detach().to(torch.float32).cpu().contiguous().reshape(-1)
    rec = np.asarray(list(recent), dtype=np.int64)
    return int(lib.sbrt_sample_row(row.data_ptr(), row.numel(), params.temperature, params.top_k, params.top_p,
                                   params.repetition_penalty, params.repetition_window,
                                   rec.ctypes.data if rec.size else None, rec.size, C.byref(rng.state)))


def greedy_argmax(row) -> int:
    """First maximum (ties -> lower id), the rule every device arg-max kernel reproduces."""
    r = torch.as_tensor(row).float().reshape(-1)
    best, best_val = 0, float(r[0])
    vals = r.tolist()
    for j in range(1, len(vals)):
        if vals[j] > best_val:
            best_val, best = vals[j], j
    return best

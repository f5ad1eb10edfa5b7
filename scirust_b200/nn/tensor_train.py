"""Tensor-train compression of dense layers: TT-SVD of a weight ``[in, out]`` whose axes are factorised into modes
``in = prod(in_dims)``, ``out = prod(out_dims)``. Mode k pairs (in_k, out_k); sweeping left to right, each step
reshapes the remainder to ``[r_k * in_k * out_k, rest]``, takes an SVD (on the weight's device: cuSOLVER on a GPU)
and keeps the singular values above ``tolerance * sigma_max`` up to ``max_rank``. ``tt_decompose`` returns a
``zoo.TTLinear`` whose cores reproduce the weight to the truncation error; ``tt_decompose_auto`` picks balanced
mode sizes. Reference counterpart: scirust-core/src/nn/tt_linear.rs:32-360 (``TTLinear``, ``tt_decompose``,
``tt_decompose_auto``, ``auto_factorize``).
"""
from __future__ import annotations

import math

import torch

from .zoo import TTLinear


def auto_factorize(n: int, n_factors: int) -> list:
    """``n_factors`` integers with product ``n``, as balanced as the prime factorisation allows (ascending)."""
    if n_factors < 1 or n < 1:
        raise ValueError("auto_factorize: n and n_factors must be positive")
    primes, m, p = [], n, 2
    while p * p <= m:
        while m % p == 0:
            primes.append(p)
            m //= p
        p += 1
    if m > 1:
        primes.append(m)
    dims = [1] * n_factors
    for q in sorted(primes, reverse=True):
        dims[dims.index(min(dims))] *= q
    return sorted(dims)


def tt_svd(weight: torch.Tensor, in_dims, out_dims, max_rank: int, tolerance: float = 0.0):
    """Cores ``[r_k, in_k, out_k, r_{k+1}]`` and the rank list."""
    in_dims, out_dims = list(in_dims), list(out_dims)
    d = len(in_dims)
    if len(out_dims) != d:
        raise ValueError("in/out_dims must have the same length")
    if math.prod(in_dims) != weight.shape[0] or math.prod(out_dims) != weight.shape[1]:
        raise ValueError(f"mode products {math.prod(in_dims)} x {math.prod(out_dims)} != weight {tuple(weight.shape)}")
    # [i0..id, o0..od] -> [(i0 o0), (i1 o1), ...]
    t = weight.float().reshape(*in_dims, *out_dims)
    perm = [x for k in range(d) for x in (k, d + k)]
    t = t.permute(*perm).reshape([in_dims[k] * out_dims[k] for k in range(d)])
    cores, ranks, r = [], [1], 1
    rest = t.reshape(1, -1)
    for k in range(d - 1):
        nk = in_dims[k] * out_dims[k]
        mat = rest.reshape(r * nk, -1)
        u, s, vh = torch.linalg.svd(mat, full_matrices=False)
        keep = int((s > tolerance * s[0]).sum()) if tolerance > 0 else s.numel()
        keep = max(1, min(keep, max_rank, s.numel()))
        cores.append(u[:, :keep].reshape(r, in_dims[k], out_dims[k], keep))
        rest = s[:keep, None] * vh[:keep]
        r = keep
        ranks.append(r)
    cores.append(rest.reshape(r, in_dims[-1], out_dims[-1], 1))
    ranks.append(1)
    return cores, ranks


def tt_decompose(linear, in_dims, out_dims, max_rank: int, tolerance: float = 0.0) -> TTLinear:
    """``linear`` has ``weight [in, out]`` (the framework's Linear) or is a ``torch.nn.Linear`` (``[out, in]``)."""
    w = linear.weight.detach()
    if isinstance(linear, torch.nn.Linear):
        w = w.t()
    cores, ranks = tt_svd(w, in_dims, out_dims, max_rank, tolerance)
    tt = TTLinear(in_dims, out_dims, rank=max(ranks))
    tt.cores = torch.nn.ParameterList([torch.nn.Parameter(c.contiguous()) for c in cores])
    bias = getattr(linear, "bias", None)
    with torch.no_grad():
        if bias is not None:
            tt.bias.copy_(bias.detach().reshape(-1))
    tt.ranks = ranks
    return tt


def tt_decompose_auto(linear, n_factors: int, max_rank: int, tolerance: float = 0.0) -> TTLinear:
    w = linear.weight
    fin, fout = (w.shape[1], w.shape[0]) if isinstance(linear, torch.nn.Linear) else (w.shape[0], w.shape[1])
    return tt_decompose(linear, auto_factorize(fin, n_factors), auto_factorize(fout, n_factors), max_rank, tolerance)


def num_params(tt: TTLinear) -> int:
    return sum(c.numel() for c in tt.cores) + tt.bias.numel()


def compression_ratio(tt: TTLinear) -> float:
    dense = math.prod(tt.in_modes) * math.prod(tt.out_modes) + tt.bias.numel()
    return dense / num_params(tt)

"""Post-training quantisation methods beyond the core set of ``quantization.py`` and the fake-quant op of QAT.

* ``SqueezeLlmCodebook``  non-uniform ``2^bits`` codebook fitted by sensitivity-weighted k-means (quantile start,
  fixed number of Lloyd iterations): code points go where they reduce the loss, not where weights are dense.
* ``SpqrOutliers``        the fraction of weights with the largest dense-quantisation error kept in full precision
  (sparse side channel), ties broken by index.
* ``omniquant_quantize``  per-output-channel symmetric codes with a searched clip factor gamma in (0, 1] (the grid
  contains 1, so the result is never worse than round-to-nearest).
* ``quantize_aqlm``       additive quantisation: each group of ``g`` weights is the SUM of one codeword from each of
  ``M`` codebooks, learned by residual k-means initialisation and alternating beam-1 re-assignment / codebook update.
* ``quantize_quip``       QuIP#-style: a seeded random sign + blockwise Hadamard transform makes the weights
  incoherent, blocks of 8 are rounded to the nearest point of the E8 lattice, the inverse transform reconstructs.
* ``fake_quantize``       symmetric quantise-dequantise with a straight-through gradient (identity inside the clip
  range, zero outside): the QAT op of the tape.

Counterparts: scirust-core/src/quantization.rs:1237-1420 (SqueezeLLM), :1430-1560 (SpQR), :1960-2170 (OmniQuant),
:2180-2560 (AQLM), :2560-2806 (QuIP#: ``nearest_e8`` :2572, ``random_hadamard_transform`` :2592); the STE op is
scirust-core/src/autodiff/reverse.rs:3525-3565. Everything is deterministic: fixed iteration counts, fixed orders,
seeded sign patterns.
"""
from __future__ import annotations

import torch


# --------------------------------------------------------------------------------------- SqueezeLLM
class SqueezeLlmCodebook:
    def __init__(self, levels: torch.Tensor):
        self.levels = levels

    @staticmethod
    def fit(weights, sensitivity, bits: int, iters: int = 20) -> "SqueezeLlmCodebook":
        w = torch.as_tensor(weights, dtype=torch.float32).reshape(-1)
        s = torch.as_tensor(sensitivity, dtype=torch.float32).reshape(-1)
        if w.numel() != s.numel():
            raise ValueError("SqueezeLLM: weights / sensitivity length mismatch")
        if not 1 <= bits <= 8:
            raise ValueError("SqueezeLLM: bits must be in 1..=8")
        if bool((s < 0).any()):
            raise ValueError("SqueezeLLM: sensitivities must be non-negative")
        k = 1 << bits
        sw = torch.sort(w).values
        # quantile initialisation: the centre of each of the k equal-count slices
        q = ((torch.arange(k, dtype=torch.float32) + 0.5) / k * (w.numel() - 1)).round().long()
        levels = sw[q].clone()
        for _ in range(iters):
            assign = (w[:, None] - levels[None, :]).abs().argmin(1)
            num = torch.zeros(k).index_add_(0, assign, w * s)
            den = torch.zeros(k).index_add_(0, assign, s)
            upd = den > 0
            levels = torch.where(upd, num / den.clamp_min(1e-30), levels)
        return SqueezeLlmCodebook(torch.sort(levels).values)

    def quantize(self, weights) -> torch.Tensor:
        w = torch.as_tensor(weights, dtype=torch.float32)
        return (w.reshape(-1, 1) - self.levels[None, :]).abs().argmin(1).reshape(w.shape).to(torch.uint8)

    def dequantize(self, codes) -> torch.Tensor:
        return self.levels[torch.as_tensor(codes).long()]


# --------------------------------------------------------------------------------------------- SpQR
class SpqrOutliers:
    def __init__(self, indices: torch.Tensor, values: torch.Tensor):
        self.indices, self.values = indices, values

    @staticmethod
    def extract(weights, quantized, outlier_frac: float) -> "SpqrOutliers":
        w = torch.as_tensor(weights, dtype=torch.float32).reshape(-1)
        q = torch.as_tensor(quantized, dtype=torch.float32).reshape(-1)
        if w.numel() != q.numel():
            raise ValueError("SpQR: weights / quantized length mismatch")
        if not 0.0 <= outlier_frac <= 1.0:
            raise ValueError("SpQR: outlier_frac must be in [0, 1]")
        k = int(round(w.numel() * outlier_frac))
        err = (w - q).abs()
        order = torch.sort(-err, stable=True).indices[:k]          # largest error first, lower index on ties
        idx = torch.sort(order).values
        return SpqrOutliers(idx, w[idx].clone())

    def apply(self, quantized) -> torch.Tensor:
        """The dense reconstruction with the outliers restored to their exact values."""
        q = torch.as_tensor(quantized, dtype=torch.float32).clone()
        flat = q.reshape(-1)
        flat[self.indices] = self.values
        return q

    def overhead_bytes(self) -> int:
        return int(self.indices.numel()) * (4 + 4)


# ----------------------------------------------------------------------------------------- OmniQuant
class OmniQuantResult:
    def __init__(self, codes, scales, gammas, in_features, out_features):
        self.codes, self.scales, self.gammas = codes, scales, gammas
        self.in_features, self.out_features = in_features, out_features

    def dequantize(self) -> torch.Tensor:
        return self.codes.float() * self.scales[None, :]


def omniquant_quantize(weight, bits: int = 4, grid: int = 32) -> OmniQuantResult:
    """``weight [in, out]``; per output channel the clip factor of the grid ``{1/grid, ..., 1}`` with the least
    squared error (ties: the larger gamma)."""
    w = torch.as_tensor(weight, dtype=torch.float32)
    if w.dim() != 2 or not 2 <= bits <= 8:
        raise ValueError("omniquant_quantize: 2-D weight and 2 <= bits <= 8")
    qmax = float((1 << (bits - 1)) - 1)
    amax = w.abs().amax(0).clamp_min(1e-12)
    best_err = torch.full((w.shape[1],), float("inf"))
    best_g = torch.ones(w.shape[1])
    for j in range(grid, 0, -1):                                   # gamma = 1 first: kept on ties
        g = j / grid
        scale = amax * g / qmax
        q = torch.clamp(torch.round(w / scale[None, :]), -qmax, qmax)
        err = (w - q * scale[None, :]).pow(2).sum(0)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best_g = torch.where(better, torch.full_like(best_g, g), best_g)
    scales = amax * best_g / qmax
    codes = torch.clamp(torch.round(w / scales[None, :]), -qmax, qmax).to(torch.int8)
    return OmniQuantResult(codes, scales, best_g, w.shape[0], w.shape[1])


# ---------------------------------------------------------------------------------------------- AQLM
class AqlmResult:
    def __init__(self, codebooks, codes, group_size, n_weights, shape):
        self.codebooks, self.codes, self.group_size, self.n_weights, self.shape = codebooks, codes, group_size, n_weights, shape

    def dequantize(self) -> torch.Tensor:
        rec = sum(cb[self.codes[:, m]] for m, cb in enumerate(self.codebooks))
        return rec.reshape(-1)[:self.n_weights].reshape(self.shape)

    def bits_per_weight(self) -> float:
        import math
        return sum(math.log2(cb.shape[0]) for cb in self.codebooks) / self.group_size


def _kmeans(x: torch.Tensor, k: int, iters: int) -> torch.Tensor:
    n = x.shape[0]
    order = torch.sort(x.pow(2).sum(1), stable=True).indices       # spread the start along the norm ordering
    cent = x[order[((torch.arange(k, dtype=torch.float32) + 0.5) / k * (n - 1)).round().long()]].clone()
    for _ in range(iters):
        assign = torch.cdist(x, cent).argmin(1)
        num = torch.zeros_like(cent).index_add_(0, assign, x)
        cnt = torch.zeros(k).index_add_(0, assign, torch.ones(n))
        cent = torch.where((cnt > 0)[:, None], num / cnt.clamp_min(1)[:, None], cent)
    return cent


def quantize_aqlm(weight, group_size: int = 8, num_codebooks: int = 2, codebook_size: int = 16, iters: int = 8
                  ) -> AqlmResult:
    w = torch.as_tensor(weight, dtype=torch.float32)
    flat = w.reshape(-1)
    n = flat.numel()
    pad = (-n) % group_size
    x = torch.cat([flat, torch.zeros(pad)]).reshape(-1, group_size)
    k = min(codebook_size, x.shape[0])
    codebooks, codes = [], torch.zeros((x.shape[0], num_codebooks), dtype=torch.long)
    resid = x.clone()
    for m in range(num_codebooks):                                  # residual initialisation
        cb = _kmeans(resid, k, iters)
        codes[:, m] = torch.cdist(resid, cb).argmin(1)
        resid = resid - cb[codes[:, m]]
        codebooks.append(cb)
    for _ in range(iters):                                          # alternate: re-assign one codebook at a time, refit it
        for m in range(num_codebooks):
            others = sum(codebooks[j][codes[:, j]] for j in range(num_codebooks) if j != m)
            target = x - others if num_codebooks > 1 else x
            codes[:, m] = torch.cdist(target, codebooks[m]).argmin(1)
            num = torch.zeros_like(codebooks[m]).index_add_(0, codes[:, m], target)
            cnt = torch.zeros(k).index_add_(0, codes[:, m], torch.ones(x.shape[0]))
            codebooks[m] = torch.where((cnt > 0)[:, None], num / cnt.clamp_min(1)[:, None], codebooks[m])
    return AqlmResult(codebooks, codes, group_size, n, tuple(w.shape))


# --------------------------------------------------------------------------------------------- QuIP#
def fwht8(block: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform of the last axis (length 8); its own inverse."""
    x = block
    h = 1
    while h < 8:
        x = x.reshape(*x.shape[:-1], 8 // (2 * h), 2, h)
        x = torch.stack([x[..., 0, :] + x[..., 1, :], x[..., 0, :] - x[..., 1, :]], -2).reshape(*block.shape)
        h *= 2
    return x / (8 ** 0.5)


def nearest_e8(x: torch.Tensor) -> torch.Tensor:
    """Nearest point of the E8 lattice (D8 union D8 + 1/2) to each row of ``x [n, 8]``."""
    def nearest_d8(v):
        r = torch.round(v)
        odd = (r.sum(-1).long() % 2) != 0
        diff = v - r
        j = diff.abs().argmax(-1)
        step = torch.where(diff.gather(-1, j[:, None]).squeeze(-1) >= 0, 1.0, -1.0)
        fix = torch.zeros_like(r).scatter_(-1, j[:, None], step[:, None])
        return torch.where(odd[:, None], r + fix, r)
    a = nearest_d8(x)
    b = nearest_d8(x - 0.5) + 0.5
    return torch.where(((x - a).pow(2).sum(-1) <= (x - b).pow(2).sum(-1))[:, None], a, b)


def _signs(n: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.where(torch.randint(0, 2, (n,), generator=g) == 0, 1.0, -1.0)


def random_hadamard_transform(w: torch.Tensor, seed: int) -> torch.Tensor:
    flat = w.reshape(-1).float()
    pad = (-flat.numel()) % 8
    x = torch.cat([flat, torch.zeros(pad)])
    return fwht8((x * _signs(x.numel(), seed)).reshape(-1, 8)).reshape(-1)


def inverse_random_hadamard_transform(wr: torch.Tensor, seed: int, length: int) -> torch.Tensor:
    x = fwht8(wr.reshape(-1, 8)).reshape(-1) * _signs(wr.numel(), seed)
    return x[:length]


class QuipResult:
    def __init__(self, codes, scale, seed, n_weights, shape):
        self.codes, self.scale, self.seed, self.n_weights, self.shape = codes, scale, seed, n_weights, shape

    def dequantize(self) -> torch.Tensor:
        pts = self.codes.float() / 2.0 * self.scale                 # codes hold 2 x the lattice coordinates
        return inverse_random_hadamard_transform(pts, self.seed, self.n_weights).reshape(self.shape)


def quantize_quip(weight, bits: int = 2, seed: int = 0) -> QuipResult:
    """``bits`` sets the lattice scale: the transformed weights are scaled so that their largest magnitude maps to
    ``2^(bits-1)`` lattice units."""
    w = torch.as_tensor(weight, dtype=torch.float32)
    wr = random_hadamard_transform(w, seed)
    amax = float(wr.abs().max())
    scale = amax / float(1 << (bits - 1)) if amax > 0 else 1.0
    pts = nearest_e8((wr / scale).reshape(-1, 8))
    return QuipResult(torch.round(pts * 2).to(torch.int16).reshape(-1), scale, seed, w.numel(), tuple(w.shape))


# ------------------------------------------------------------------------------------- fake quant (STE)
class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, qmax):
        q = torch.clamp(torch.round(x / scale), -qmax, qmax)
        ctx.save_for_backward((x / scale).abs() <= qmax)
        return q * scale

    @staticmethod
    def backward(ctx, dy):
        (inside,) = ctx.saved_tensors
        return dy * inside.to(dy.dtype), None, None


def fake_quantize(x: torch.Tensor, bits: int = 8, scale: float | None = None) -> torch.Tensor:
    """Quantise-dequantise on a symmetric ``bits``-bit grid; gradient passes straight through inside the clip range
    and is zero outside. ``scale`` defaults to ``max|x| / qmax`` (detached)."""
    qmax = float((1 << (bits - 1)) - 1)
    if scale is None:
        m = float(x.detach().abs().max())
        scale = m / qmax if m > 0 else 1.0
    return _FakeQuant.apply(x, float(scale), qmax)

"""Weight / activation quantisation (scirust-core/src/quantization.rs:8-190 core, :265-2806 methods).

Core (bit-compatible with the reference's integer arithmetic): symmetric per-tensor INT8
(``compute_scale`` / ``quantize_tensor`` / ``dequantize_tensor``), per-output-channel weights for the
x.W layout (``quantize_per_channel``), ``matmul_int8`` (wide accumulation, saturated to i32) and the
W8A8-dynamic ``quantized_linear_forward``. Methods: SmoothQuant scale migration, GPTQ
(Hessian-ordered error feedback), AWQ (activation-aware per-channel scaling search), ternary /
BitNet b1.58, NF4 (normal-float 4-bit, blockwise absmax), group-wise INT4 and KV-cache
quantisation. On CUDA the per-channel weight path uses the native kernels of ``ops.decode``.
"""
from __future__ import annotations

import numpy as np
import torch

from .io.artifacts import quantize_tensor as _quantize_np
from .ops.decode import QuantWeight, gemv, quantize_per_channel as quantize_per_channel_t  # noqa: F401


def compute_scale(x) -> float:
    m = float(np.abs(np.asarray(x, dtype=np.float32)).max()) if np.size(x) else 0.0
    return 1.0 if m == 0.0 else float(np.float32(m) / np.float32(127.0))


def quantize_tensor(x, scale: float) -> np.ndarray:
    return _quantize_np(np.asarray(x, dtype=np.float32), scale)


def dequantize_tensor(q, scale: float) -> np.ndarray:
    return np.asarray(q, dtype=np.int8).astype(np.float32) * np.float32(scale)


def quantize_per_channel(weight, in_features: int, out_features: int):
    """weight: flat or (in, out) fp32 in x.W layout -> (int8 codes (in*out,), fp32 scales (out,))."""
    w = np.asarray(weight, dtype=np.float32).reshape(in_features, out_features)
    mx = np.abs(w).max(0)
    scales = np.where(mx == 0, np.float32(1.0), mx / np.float32(127.0)).astype(np.float32)
    q = np.empty_like(w, dtype=np.int8)
    for o in range(out_features):
        q[:, o] = _quantize_np(w[:, o], scales[o])
    return q.reshape(-1), scales


def matmul_int8(a, b, m: int, k: int, n: int) -> np.ndarray:
    acc = np.asarray(a, dtype=np.int8).reshape(m, k).astype(np.int64) @ np.asarray(b, dtype=np.int8).reshape(k, n).astype(np.int64)
    return np.clip(acc, -2**31, 2**31 - 1).astype(np.int32).reshape(-1)


def quantized_linear_forward(x, batch: int, in_features: int, w_q, w_scales, bias, out_features: int) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    if x.size != batch * in_features:
        raise ValueError(f"quantized_linear_forward: input has {x.size} values, expected {batch * in_features}")
    if np.size(w_q) != in_features * out_features or np.size(w_scales) != out_features or np.size(bias) != out_features:
        raise ValueError("quantized_linear_forward: weight / scale / bias sizes do not match the layer")
    s_in = np.float32(compute_scale(x))
    acc = matmul_int8(quantize_tensor(x, s_in), w_q, batch, in_features, out_features).reshape(batch, out_features)
    return (acc.astype(np.float32) * s_in * np.asarray(w_scales, dtype=np.float32)[None, :]
            + np.asarray(bias, dtype=np.float32)[None, :]).reshape(-1)


# ----------------------------------------------------------------------------- methods
def smoothquant_scales(act_absmax: torch.Tensor, weight: torch.Tensor, alpha: float = 0.5) -> torch.Tensor:
    """Per-input-channel s_j = max|X_j|^alpha / max|W_j|^(1-alpha); use X/s and s*W."""
    w_absmax = weight.abs().amax(1).clamp_min(1e-5)
    return (act_absmax.clamp_min(1e-5) ** alpha / w_absmax ** (1 - alpha)).clamp_min(1e-5)


def smoothquant_apply(x: torch.Tensor, weight: torch.Tensor, alpha: float = 0.5):
    s = smoothquant_scales(x.abs().amax(0), weight, alpha)
    return x / s[None, :], weight * s[:, None], s


def _rtn(w: torch.Tensor, bits: int, scale: torch.Tensor) -> torch.Tensor:
    qmax = 2 ** (bits - 1) - 1
    return torch.clamp(torch.round(w / scale), -qmax - 1, qmax) * scale


def gptq_quantize(weight: torch.Tensor, x_calib: torch.Tensor, bits: int = 4, damp: float = 0.01) -> torch.Tensor:
    """GPTQ on an (in, out) weight: quantise input rows one at a time and push each row's rounding
    error onto the not-yet-quantised rows through the inverse Hessian of the calibration inputs."""
    W = weight.double().clone()
    H = 2.0 * x_calib.double().t() @ x_calib.double()
    H += damp * torch.diag(H).mean() * torch.eye(H.shape[0], dtype=torch.float64)
    Hinv = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(H)), upper=True)
    qmax = 2 ** (bits - 1) - 1
    scale = (W.abs().amax(0) / qmax).clamp_min(1e-12)
    Q = torch.zeros_like(W)
    for i in range(W.shape[0]):
        q = _rtn(W[i], bits, scale)
        Q[i] = q
        err = (W[i] - q) / Hinv[i, i]
        if i + 1 < W.shape[0]:
            W[i + 1:] -= Hinv[i, i + 1:, None] * err[None, :]
    return Q.to(weight.dtype)


def awq_quantize(weight: torch.Tensor, x_calib: torch.Tensor, bits: int = 4, grid: int = 20):
    """AWQ: search s = mean|X|^a (a in [0,1]) minimising ||X W - (X/s) Q(s W)||; returns (Q(sW)/s, s)."""
    a_mean = x_calib.abs().mean(0).clamp_min(1e-5)
    ref = x_calib @ weight
    qmax = 2 ** (bits - 1) - 1
    best = (None, None, float("inf"))
    for g in range(grid + 1):
        s = (a_mean ** (g / grid)).clamp_min(1e-4)
        s = s / (s.max() * s.min()).sqrt()
        ws = weight * s[:, None]
        sc = (ws.abs().amax(0) / qmax).clamp_min(1e-12)
        wq = _rtn(ws, bits, sc) / s[:, None]
        err = float(((x_calib @ wq) - ref).pow(2).mean())
        if err < best[2]:
            best = (wq, s, err)
    return best[0], best[1]


def ternary_quantize(weight: torch.Tensor):
    """BitNet b1.58: codes in {-1, 0, +1} with scale = mean |W|."""
    scale = weight.abs().mean().clamp_min(1e-12)
    return torch.clamp(torch.round(weight / scale), -1, 1).to(torch.int8), float(scale)


_NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                     0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                     0.7229568362236023, 1.0])


def nf4_quantize(weight: torch.Tensor, block: int = 64):
    """Normal-float 4-bit: blockwise absmax scaling, nearest of the 16 normal-quantile levels."""
    flat = weight.reshape(-1).float()
    pad = (-flat.numel()) % block
    x = torch.cat([flat, flat.new_zeros(pad)]).reshape(-1, block)
    absmax = x.abs().amax(1, keepdim=True).clamp_min(1e-12)
    codes = ((x / absmax)[..., None] - _NF4).abs().argmin(-1).to(torch.uint8)
    return codes, absmax.reshape(-1), weight.shape, pad


def nf4_dequantize(codes, absmax, shape, pad):
    x = _NF4[codes.long()] * absmax[:, None]
    flat = x.reshape(-1)
    return (flat[: flat.numel() - pad] if pad else flat).reshape(shape)


def int4_group_quantize(weight: torch.Tensor, group: int = 32):
    """Group-wise symmetric INT4 along the flattened weight (the SciAgent model quantiser,
    scirust-sciagent/src/quantize.rs:9-260): two codes per byte, one fp32 scale per group."""
    flat = weight.reshape(-1).float()
    pad = (-flat.numel()) % group
    x = torch.cat([flat, flat.new_zeros(pad)]).reshape(-1, group)
    scale = (x.abs().amax(1, keepdim=True) / 7.0)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round(x / scale), -8, 7).to(torch.int8).reshape(-1)
    packed = ((q[0::2] & 0xF) | ((q[1::2] & 0xF) << 4)).to(torch.uint8)
    return packed, scale.reshape(-1), weight.shape, pad


def int4_group_dequantize(packed, scale, shape, pad, group: int = 32):
    lo = (packed & 0xF).to(torch.int8)
    hi = ((packed >> 4) & 0xF).to(torch.int8)
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    q = torch.stack([lo, hi], 1).reshape(-1).float().reshape(-1, group) * scale[:, None]
    flat = q.reshape(-1)
    return (flat[: flat.numel() - pad] if pad else flat).reshape(shape)


def kv_quantize(x: torch.Tensor, bits: int = 8, per_channel: bool = True):
    """KVQuant-style: keys per channel, values per token."""
    qmax = 2 ** (bits - 1) - 1
    dim = 0 if per_channel else 1
    scale = (x.abs().amax(dim, keepdim=True) / qmax).clamp_min(1e-12)
    return torch.clamp(torch.round(x / scale), -qmax - 1, qmax).to(torch.int8), scale

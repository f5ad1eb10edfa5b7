"""Green-list text watermark (Kirchenbauer et al., 2023): a keyed hash of (previous token, token) marks a
``gamma`` fraction of the vocabulary green at every position, generation adds ``delta`` to the green logits,
and detection needs only the key: the count of green transitions is binomial under the null, so its z-score
exposes watermarked text without access to the model. The hash is a SplitMix64 finaliser whose top 24 bits
become a uniform in [0, 1). Reference counterpart: scirust-core/src/nn/watermark.rs:14-62. Whole rows are
hashed at once (uint64 NumPy arithmetic), so biasing a 128 k-entry logit row costs one vector pass.
"""
from __future__ import annotations

import math

import numpy as np
import torch

_M1, _M2 = np.uint64(0x9E3779B97F4A7C15), np.uint64(0xD1B54A32D192ED03)
_F1, _F2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)


def green_hash(seed: int, prev_token, token) -> np.ndarray:
    """Uniform [0, 1) value of each (prev_token, token) pair (broadcasting, float32)."""
    with np.errstate(over="ignore"):
        z = (np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + np.asarray(prev_token, dtype=np.uint64) * _M1
             + np.asarray(token, dtype=np.uint64) * _M2)
        z = (z ^ (z >> np.uint64(30))) * _F1
        z = (z ^ (z >> np.uint64(27))) * _F2
        z = z ^ (z >> np.uint64(31))
    return (z >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)


def is_green(seed: int, prev_token: int, token: int, gamma: float) -> bool:
    return bool(green_hash(seed, prev_token, token) < np.float32(gamma))


def green_mask(seed: int, prev_token: int, vocab: int, gamma: float) -> np.ndarray:
    return green_hash(seed, prev_token, np.arange(vocab, dtype=np.uint64)) < np.float32(gamma)


def apply_green_bias(logits, seed: int, prev_token: int, gamma: float, delta: float):
    """Add ``delta`` to the green tokens of one logit row, in place; returns the row."""
    if isinstance(logits, torch.Tensor):
        mask = torch.from_numpy(green_mask(seed, prev_token, logits.shape[-1], gamma)).to(logits.device)
        logits[..., mask] += delta
        return logits
    arr = np.asarray(logits)
    arr[green_mask(seed, prev_token, arr.shape[-1], gamma)] += delta
    return arr


def detect_z(seed: int, tokens, gamma: float) -> float:
    """z = (green - gamma n) / sqrt(n gamma (1 - gamma)) over the n = len - 1 transitions."""
    t = np.asarray(tokens, dtype=np.uint64).reshape(-1)
    if t.size < 2:
        return 0.0
    n = float(t.size - 1)
    green = float((green_hash(seed, t[:-1], t[1:]) < np.float32(gamma)).sum())
    return (green - gamma * n) / math.sqrt(n * gamma * (1.0 - gamma))


def detect_p_value(seed: int, tokens, gamma: float) -> float:
    """One-sided p-value of the z statistic under the no-watermark null."""
    return 0.5 * math.erfc(detect_z(seed, tokens, gamma) / math.sqrt(2.0))

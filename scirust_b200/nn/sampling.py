"""Seeded token sampling for autoregressive generation on the PCG stream: greedy, temperature, top-k and
nucleus (top-p). The same seed and logits always give the same token; greedy consumes no random draw.
Reference counterpart: scirust-core/src/nn/sampling.rs:11-134 (``SamplingConfig``, ``sample_token``); the
decoder's own sampler (splitmix-seeded xorshift, repetition penalty) is ``scirust_b200.generate``.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .rng import PcgEngine


@dataclass
class SamplingConfig:
    temperature: float = 1.0     # <= 0: greedy arg-max
    top_k: int = 0               # 0 disables; 1 is greedy
    top_p: float = 1.0           # >= 1 disables

    @staticmethod
    def greedy() -> "SamplingConfig":
        return SamplingConfig(temperature=0.0, top_k=0, top_p=1.0)


def _argmax(logits: np.ndarray) -> int:
    """First maximum (ties to the lowest index); NaNs never win."""
    best, best_v = 0, -np.inf
    for i, v in enumerate(logits):
        if v > best_v:
            best, best_v = i, v
    return best


def sample_token(logits, cfg: SamplingConfig, rng: PcgEngine) -> int:
    x = np.asarray(torch.as_tensor(logits).detach().float().cpu().numpy() if isinstance(logits, torch.Tensor)
                   else logits, dtype=np.float32).reshape(-1)
    if x.size == 0:
        return 0
    if cfg.temperature <= 0.0 or cfg.top_k == 1:
        return _argmax(x)
    inv_t = np.float32(1.0 / cfg.temperature)
    probs = np.exp((x - x.max()) * inv_t, dtype=np.float32)
    # descending probability, ascending index among equals
    order = np.lexsort((np.arange(x.size), -probs))
    if 0 < cfg.top_k < x.size:
        probs[order[cfg.top_k:]] = 0.0
    if cfg.top_p < 1.0:
        total = np.float32(0.0)
        for p in probs:
            total += p
        if total > 0.0:
            cum, cutoff = np.float32(0.0), x.size
            for rank, i in enumerate(order):
                cum += probs[i] / total
                if cum >= cfg.top_p:
                    cutoff = rank + 1
                    break
            probs[order[cutoff:]] = 0.0
    s = np.float32(0.0)
    for p in probs:
        s += p
    if s <= 0.0:
        return _argmax(x)
    r = np.float32(rng.float()) * s
    cum = np.float32(0.0)
    for i, p in enumerate(probs):
        cum += p
        if r < cum:
            return i
    return int(order[0])

"""Memory planner for the SciAgent decoder (scirust-sciagent/src/planning.rs:23-156): bytes needed
for weights, optimizer state, activations (with naive S x S attention, with flash attention, with
activation checkpointing) and the KV cache, and whether a configuration fits a device. Sized for a
180 GB B200 by default."""
from __future__ import annotations

from dataclasses import dataclass

B200_HBM_BYTES = 180 * 10 ** 9


@dataclass
class MemoryPlan:
    weights: int
    optimizer: int
    grads: int
    activations_naive: int
    activations_flash: int
    activations_checkpointed: int
    kv_cache: int

    def total(self, mode: str = "flash") -> int:
        act = {"naive": self.activations_naive, "flash": self.activations_flash,
               "checkpointed": self.activations_checkpointed}[mode]
        return self.weights + self.optimizer + self.grads + act

    def fits(self, mode: str = "flash", capacity: int = B200_HBM_BYTES, headroom: float = 0.9) -> bool:
        return self.total(mode) <= capacity * headroom


def n_params(cfg) -> int:
    d, ff, L = cfg.d_model, cfg.d_ff, cfg.n_layers
    per = d * cfg.qkv_dim + cfg.n_heads * cfg.head_dim * d + 3 * d * ff + 2 * d
    head = 0 if cfg.tie_embeddings else cfg.vocab_size * d
    return cfg.vocab_size * d + L * per + d + head


def plan(cfg, batch: int, seq: int, tp: int = 1, kv_batch: int = 0, kv_seq: int = 0) -> MemoryPlan:
    P = n_params(cfg)
    T = batch * seq
    d, ff, L, H = cfg.d_model, cfg.d_ff, cfg.n_layers, cfg.n_heads
    weights = 2 * P // tp
    optimizer = 12 * P // tp                      # fp32 master + two Adam moments
    grads = 2 * P // tp
    # saved per layer by the block's backward: x, h1, qkv, a, x2, h2, gu, hm (bf16) + lse/inv (fp32)
    per_layer = 2 * T * (3 * d + cfg.qkv_dim // tp + H * cfg.head_dim // tp + 3 * ff // tp) + 4 * T * (2 + H // tp)
    logits = 2 * min(T, 4096) * cfg.vocab_size
    flash = L * per_layer + logits
    naive = flash + L * 2 * batch * (H // tp) * seq * seq * 2        # scores + probabilities
    ckpt = L * 2 * T * d + per_layer + logits                          # block inputs only + one live block
    kv = 2 * 2 * L * kv_batch * kv_seq * cfg.n_kv_heads * cfg.head_dim // max(1, min(tp, cfg.n_kv_heads))
    return MemoryPlan(weights, optimizer, grads, naive, flash, ckpt, kv)

"""Held-out evaluation of a decoder checkpoint: mean next-token cross-entropy and perplexity over a directory of token
shards, no gradient step and no shuffling: a deterministic measurement. Shards load in file-name order, windows of
the model's ``max_seq_len`` are taken in order, exactly one pass (or ``max_batches``); the mean is weighted by rows so
a short batch does not bias it. On a GPU each batch is one fused forward (the loss head produces only the loss when no
gradient is wanted). Reference counterpart: scirust-sciagent/src/bin/sciagent-eval.rs (CLI `sciagent-eval`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..data.corpus import PretrainDataset, ShardLoader


@dataclass
class EvalReport:
    tokens: int
    sequences: int
    batches: int
    mean_loss: float
    perplexity: float


@torch.no_grad()
def evaluate_tokens(model, tokens, seq_len: int, vocab_size: int, batch_size: int = 8, max_batches: int = 0) -> EvalReport:
    ds = PretrainDataset(tokens, seq_len, vocab_size)
    full = len(ds) // max(batch_size, 1)
    target = min(full, max_batches) if max_batches > 0 else full
    dev = model.flat.device if hasattr(model, "flat") else next(model.parameters()).device
    total, rows, batches = 0.0, 0, 0
    while batches < target:
        nb = ds.next_batch(batch_size)
        if nb is None:
            break
        xs, ys = nb
        x = torch.tensor(xs, dtype=torch.int64).reshape(batch_size, seq_len).to(dev)
        y = torch.tensor(ys, dtype=torch.int64).reshape(batch_size, seq_len).to(dev)
        loss = float(model(x, y))
        total += loss * x.numel()
        rows += x.numel()
        batches += 1
    mean = total / rows if rows else math.nan
    return EvalReport(len(ds.data), len(ds), batches, mean, math.exp(mean) if rows else math.nan)


def evaluate_shards(model, data_dir, batch_size: int = 8, max_batches: int = 0, seq_len: int | None = None) -> EvalReport:
    loader = ShardLoader()
    loader.load_dir(data_dir)
    cfg = model.cfg
    return evaluate_tokens(model, loader.tokens(), seq_len or cfg.max_seq_len, cfg.vocab_size, batch_size, max_batches)

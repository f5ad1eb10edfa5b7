"""Vocabulary-parallel embedding, LM head, cross-entropy and arg-max for tensor-parallel ranks: rank r
owns the vocabulary ids [r * V / W, (r + 1) * V / W) of the embedding table and of the head.

The reference runs these on one device (embedding gather / scatter-add, softmax cross-entropy and the
LM-head arg-max: scirust-sciagent/src/cuda_model.rs:560-640, 1010-1080; scirust-cuda/src/chain.rs:
embed_fwd, embed_bwd, softmax_ce); here the vocabulary axis is sharded so that no rank ever holds a
[tokens, V] matrix or the whole table:

* embedding: a local lookup that yields zero rows for ids of other shards, then a sum over ranks;
  the gradient of a row goes to the shard that owns its id only
* cross-entropy: per-row (max, sum-exp, target logit) of the local logits, one small all-gather of
  those three numbers, combined in rank order (bitwise repeatable), then the local gradient
  (exp(x - lse) - onehot) * scale from the global log-sum-exp
* arg-max: local (value, id) pairs gathered; the largest value wins, ties go to the smallest id

Collectives go through ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks), so the same code is
tested on CPU ranks; the per-row statistics and the gradient are native kernels on CUDA tensors.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import basic, gemm


def shard_range(vocab: int, rank: int, world: int):
    if vocab % world:
        raise ValueError("vocabulary size must divide by the number of ranks")
    per = vocab // world
    return rank * per, per


class VocabParallelEmbedding:
    """``table`` is this rank's [V / W, d] slice. ``forward`` returns the full [n, d] activations on every
    rank (sum over ranks); ``backward`` accumulates this shard's table gradient."""

    def __init__(self, table: torch.Tensor, vocab: int, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.v0, self.per = shard_range(vocab, self.rank, self.world)
        if table.shape[0] != self.per:
            raise ValueError("table must hold this rank's vocabulary shard")
        self.table = table

    def _local(self, tokens):
        loc = tokens.reshape(-1) - self.v0
        own = (loc >= 0) & (loc < self.per)
        return loc.clamp(0, self.per - 1), own

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        loc, own = self._local(tokens)
        out = basic.embed_fwd(self.table, loc)
        out = out * own[:, None].to(out.dtype)
        acc = out.float()                      # sum in fp32: exactly one rank contributes a non-zero row
        dist.all_reduce(acc, group=self.group)
        return acc.to(self.table.dtype)

    def backward(self, dy: torch.Tensor, tokens: torch.Tensor, dtable: torch.Tensor, accumulate: bool = True):
        loc, own = self._local(tokens)
        return basic.embed_bwd(dy * own[:, None].to(dy.dtype), loc, dtable, accumulate=accumulate)


def vocab_parallel_logits(h: torch.Tensor, head_shard: torch.Tensor) -> torch.Tensor:
    """Logits of this rank's vocabulary shard: h [n, d] times head_shard [V / W, d]^T."""
    return gemm.matmul_nt(h, head_shard)


def vocab_parallel_ce(logits_local: torch.Tensor, targets: torch.Tensor, v0: int, grad_scale: float, group=None,
                      in_place: bool = True):
    """Returns (per-row loss fp32, gradient w.r.t. the local logits). Every rank gets the same loss."""
    world = dist.get_world_size(group)
    stats = basic.ce_shard_stats(logits_local, targets, v0)
    allst = [torch.empty_like(stats) for _ in range(world)]
    dist.all_gather(allst, stats, group=group)
    m = allst[0][:, 0]
    for r in range(1, world):
        m = torch.maximum(m, allst[r][:, 0])
    s = torch.zeros_like(m)
    t = torch.zeros_like(m)
    for r in range(world):                      # rank order: the same bits on every rank and every run
        s = s + allst[r][:, 1] * torch.exp(allst[r][:, 0] - m)
        t = t + allst[r][:, 2]
    lse = m + torch.log(s)
    loss = torch.where(targets.reshape(-1) < 0, torch.zeros_like(lse), lse - t)
    d = basic.ce_shard_grad(logits_local, targets, v0, lse, grad_scale, in_place=in_place)
    return loss, d


def vocab_parallel_argmax(logits_local: torch.Tensor, v0: int, group=None) -> torch.Tensor:
    """Global arg-max id per row; ties go to the smallest id."""
    world = dist.get_world_size(group)
    val, idx = logits_local.float().max(-1)
    pair = torch.stack([val, (idx + v0).float()], 1)
    allp = [torch.empty_like(pair) for _ in range(world)]
    dist.all_gather(allp, pair, group=group)
    best_v, best_i = allp[0][:, 0], allp[0][:, 1]
    for r in range(1, world):
        better = allp[r][:, 0] > best_v          # strictly larger: an equal value keeps the smaller id
        best_v = torch.where(better, allp[r][:, 0], best_v)
        best_i = torch.where(better, allp[r][:, 1], best_i)
    return best_i.long()

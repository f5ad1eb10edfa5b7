"""Context parallelism: ring attention over a sequence that is sharded across ranks.

Rank ``r`` of ``W`` holds tokens ``[r * S_l, (r + 1) * S_l)`` of every sequence as a fused ``qkv`` matrix
``[B * S_l, (H + 2 Hkv) * dh]`` (the layout of ``ops.attention``). Forward: the K/V shards travel around the ring;
at hop ``t`` a rank attends its queries to the shard of rank ``r - t`` with the ordinary flash kernel — causal on its
own shard (hop 0), unmasked on earlier shards, skipped for later ones — and folds the block's (O, LSE) into the
running result with the log-sum-exp merge, so nothing of size S x S exists anywhere and no rank ever holds the whole
sequence. Backward: the same ring; every block is differentiated with the flash backward written on the MERGED
normaliser and output (``P = exp(S - lse)``, ``delta = rowsum(dO * O)``), which yields that block's share of dQ and
the dK/dV of the visiting shard; dK/dV travel on with their shard and arrive home after W hops.

The blocks are visited in the same order on every run and merged in hop order, so results are repeatable bit for
bit at a fixed world size. Transfers are ``torch.distributed`` point-to-point operations (NCCL between GPUs, gloo
between CPU ranks), issued before the block's kernels so that the copy of hop t + 1 runs under the math of hop t.
Long-context surface of the reference: its blockwise attention oracle and planner
(scirust-sciagent/src/flash_attention.rs:1-321); the reference itself is single-device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import attention as att


def _ring_exchange(send: torch.Tensor, group, rank: int, world: int) -> torch.Tensor:
    """Send ``send`` to rank + 1, receive the same shape from rank - 1 (one hop of the ring)."""
    recv = torch.empty_like(send)
    g = (lambda r: dist.get_global_rank(group, r)) if group is not dist.group.WORLD else (lambda r: r)
    ops_ = [dist.P2POp(dist.isend, send, g((rank + 1) % world), group),
            dist.P2POp(dist.irecv, recv, g((rank - 1) % world), group)]
    for w in dist.batch_isend_irecv(ops_):
        w.wait()
    return recv


def _merge(o, lse, o_b, lse_b):
    """Fold a block's (O, LSE) into the running pair; fp32. o: [B*S, H*dh] fp32, lse: [B, H, S]."""
    new = torch.logaddexp(lse, lse_b)
    B, H, S = lse.shape
    wa = torch.exp(lse - new).permute(0, 2, 1).reshape(B * S, H, 1)
    wb = torch.exp(lse_b - new).permute(0, 2, 1).reshape(B * S, H, 1)
    wa, wb = torch.nan_to_num(wa, nan=0.0), torch.nan_to_num(wb, nan=0.0)
    dh = o.shape[1] // H
    out = o.view(B * S, H, dh) * wa + o_b.float().view(B * S, H, dh) * wb
    return out.view(B * S, H * dh), new


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, H, Hkv, dh, group, causal):
        rank, W = dist.get_rank(group), dist.get_world_size(group)
        qd = H * dh
        kv = qkv[:, qd:].contiguous()                       # the shard that travels
        o = torch.zeros((B * S, qd), dtype=torch.float32, device=qkv.device)
        lse = torch.full((B, H, S), float("-inf"), dtype=torch.float32, device=qkv.device)
        blk = qkv.clone()
        for t in range(W):
            src = (rank - t) % W
            nxt = _ring_exchange(kv, group, rank, W) if t + 1 < W else None     # hop t + 1 is in flight during hop t
            if not causal or src <= rank:
                blk[:, qd:] = kv
                o_b, lse_b = att.attention_fwd(blk, B, S, H, Hkv, dh, causal=causal and src == rank)
                o, lse = _merge(o, lse, o_b, lse_b)
            kv = nxt
        out = o.to(qkv.dtype)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (B, S, H, Hkv, dh, group, causal)
        return out

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse = ctx.saved_tensors
        B, S, H, Hkv, dh, group, causal = ctx.meta
        rank, W = dist.get_rank(group), dist.get_world_size(group)
        qd = H * dh
        do = do.contiguous()
        kv = qkv[:, qd:].contiguous()
        dkv = torch.zeros_like(kv, dtype=torch.float32)     # gradient of the visiting shard, travels with it
        dq = torch.zeros((B * S, qd), dtype=torch.float32, device=qkv.device)
        blk = qkv.clone()
        for t in range(W):
            src = (rank - t) % W
            if not causal or src <= rank:
                blk[:, qd:] = kv
                g = att.attention_bwd(blk, out, lse, do, B, S, H, Hkv, dh, causal=causal and src == rank).float()
                dq += g[:, :qd]
                dkv += g[:, qd:]
            # shard and its gradient move on together; after the last hop the gradient is home
            if t + 1 < W:
                kv = _ring_exchange(kv, group, rank, W)
            dkv = _ring_exchange(dkv, group, rank, W)
        dqkv = torch.cat([dq, dkv], 1).to(qkv.dtype)
        return dqkv, None, None, None, None, None, None, None


def ring_attention(qkv: torch.Tensor, B: int, S_local: int, H: int, Hkv: int, dh: int, group=None,
                   causal: bool = True) -> torch.Tensor:
    """Attention output ``[B * S_local, H * dh]`` of this rank's queries over the WHOLE sequence (``world * S_local``
    tokens per sequence, sharded contiguously by rank). Differentiable w.r.t. ``qkv``."""
    group = group if group is not None else dist.group.WORLD
    return _RingAttention.apply(qkv, B, S_local, H, Hkv, dh, group, causal)


def shard_sequence(x: torch.Tensor, B: int, S: int, group=None) -> torch.Tensor:
    """Rows of ``x [B * S, C]`` that belong to this rank's contiguous slice of every sequence."""
    group = group if group is not None else dist.group.WORLD
    rank, W = dist.get_rank(group), dist.get_world_size(group)
    if S % W:
        raise ValueError("sequence length must be a multiple of the context-parallel size")
    sl = S // W
    return x.view(B, S, -1)[:, rank * sl:(rank + 1) * sl].reshape(B * sl, -1).contiguous()

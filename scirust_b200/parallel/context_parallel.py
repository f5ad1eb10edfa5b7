"""Context parallelism: ring attention over a sequence that is sharded across ranks.

Rank ``r`` of ``W`` holds tokens ``[r * S_l, (r + 1) * S_l)`` of every sequence as a fused ``qkv`` matrix
``[B * S_l, (H + 2 Hkv) * dh]`` (the layout of ``ops.attention``). Forward: the K/V shards travel around the ring;
at hop ``t`` a rank attends its queries to the shard of rank ``r - t`` with the ordinary flash kernel — causal on its
own shard (hop 0), unmasked on earlier shards, skipped for later ones — and folds the block's (O, LSE) into the
running result with the log-sum-exp merge, so nothing of size S x S exists anywhere and no rank ever holds the whole
sequence. Backward: the same ring; every block is differentiated with the flash backward written on the MERGED
normaliser and output (``P = exp(S - lse)``, ``delta = rowsum(dO * O)``), which yields that block's share of dQ and
the dK/dV of the visiting shard; dK/dV travel on with their shard and arrive home after W hops.

With ``layout="zigzag"`` a rank holds chunks r and 2W - 1 - r of 2W instead of one contiguous slice, which gives
every rank the same causal work (the contiguous layout gives the last rank W times the first rank's).

The blocks are visited in the same order on every run and merged in hop order, so results are repeatable bit for
bit at a fixed world size. Transfers are ``torch.distributed`` point-to-point operations (NCCL between GPUs, gloo
between CPU ranks). The K/V transfer of hop t + 1 is posted before the block's kernels of hop t are launched and
waited for after them, so it runs under that math (forward and backward); the dK/dV transfer depends on the hop's
result and is a blocking hop.
Long-context surface of the reference: its blockwise attention oracle and planner
(scirust-sciagent/src/flash_attention.rs:1-321); the reference itself is single-device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import attention as att


class _Hop:
    """One hop of the ring in flight: ``send`` goes to rank + 1 while the same shape arrives from rank - 1. The
    transfer is posted by the constructor; ``wait`` returns the received tensor. Between the two the caller may launch
    kernels that READ ``send`` (it must not be written before ``wait``)."""

    def __init__(self, send: torch.Tensor, group, rank: int, world: int):
        self.send, self.recv = send, torch.empty_like(send)
        g = (lambda r: dist.get_global_rank(group, r)) if group is not dist.group.WORLD else (lambda r: r)
        ops_ = [dist.P2POp(dist.isend, send, g((rank + 1) % world), group),
                dist.P2POp(dist.irecv, self.recv, g((rank - 1) % world), group)]
        self.work = dist.batch_isend_irecv(ops_)

    def wait(self) -> torch.Tensor:
        for w in self.work:
            w.wait()
        return self.recv


def _ring_exchange(send: torch.Tensor, group, rank: int, world: int) -> torch.Tensor:
    """Blocking form: one hop, finished on return."""
    return _Hop(send, group, rank, world).wait()


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


def _chunk_ids(rank: int, world: int, layout: str):
    """Global indices of the sequence chunks a rank holds: one chunk (``contiguous``), or chunks ``r`` and
    ``2W - 1 - r`` of ``2W`` (``zigzag``): with a causal mask every rank then has the same number of visible
    (query chunk, key chunk) pairs, where the contiguous layout gives rank W - 1 W times the work of rank 0."""
    if layout == "contiguous":
        return [rank]
    if layout == "zigzag":
        return [rank, 2 * world - 1 - rank]
    raise ValueError("layout must be 'contiguous' or 'zigzag'")


def _rows(x, B, S, n_chunks, c):
    """Rows of chunk ``c`` of a local ``[B * S, C]`` matrix whose sequences hold ``n_chunks`` equal chunks."""
    sc = S // n_chunks
    return x.view(B, n_chunks, sc, -1)[:, c].reshape(B * sc, -1)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, H, Hkv, dh, group, causal, layout):
        rank, W = dist.get_rank(group), dist.get_world_size(group)
        qd = H * dh
        mine = _chunk_ids(rank, W, layout)
        nc, sc = len(mine), S // len(mine)
        kv = qkv[:, qd:].contiguous()                       # the shard that travels
        o = [torch.zeros((B * sc, qd), dtype=torch.float32, device=qkv.device) for _ in mine]
        lse = [torch.full((B, H, sc), float("-inf"), dtype=torch.float32, device=qkv.device) for _ in mine]
        qs = [_rows(qkv, B, S, nc, i)[:, :qd] for i in range(nc)]
        for t in range(W):
            src = (rank - t) % W
            theirs = _chunk_ids(src, W, layout)
            hop = _Hop(kv, group, rank, W) if t + 1 < W else None               # hop t + 1 is in flight during hop t
            for i, a in enumerate(mine):
                for j, b in enumerate(theirs):
                    if causal and b > a:
                        continue                              # every key of that chunk lies in the future
                    blk = torch.cat([qs[i], _rows(kv, B, S, nc, j)], 1)
                    o_b, lse_b = att.attention_fwd(blk, B, sc, H, Hkv, dh, causal=causal and a == b)
                    o[i], lse[i] = _merge(o[i], lse[i], o_b, lse_b)
            kv = hop.wait() if hop is not None else None
        out = torch.stack([x.view(B, sc, qd) for x in o], 1).reshape(B * S, qd).to(qkv.dtype)
        ctx.save_for_backward(qkv, out, torch.stack(lse, 0))
        ctx.meta = (B, S, H, Hkv, dh, group, causal, layout)
        return out

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse = ctx.saved_tensors
        B, S, H, Hkv, dh, group, causal, layout = ctx.meta
        rank, W = dist.get_rank(group), dist.get_world_size(group)
        qd = H * dh
        mine = _chunk_ids(rank, W, layout)
        nc, sc = len(mine), S // len(mine)
        do = do.contiguous()
        kv = qkv[:, qd:].contiguous()
        kvd = kv.shape[1]
        dkv = torch.zeros((B, nc, sc, kvd), dtype=torch.float32, device=qkv.device)    # travels with its shard
        dq = torch.zeros((B, nc, sc, qd), dtype=torch.float32, device=qkv.device)
        qs = [_rows(qkv, B, S, nc, i)[:, :qd] for i in range(nc)]
        outs = [_rows(out, B, S, nc, i).contiguous() for i in range(nc)]
        dos = [_rows(do, B, S, nc, i).contiguous() for i in range(nc)]
        for t in range(W):
            src = (rank - t) % W
            theirs = _chunk_ids(src, W, layout)
            hop = _Hop(kv, group, rank, W) if t + 1 < W else None               # the shard moves on under this hop's math
            for i, a in enumerate(mine):
                for j, b in enumerate(theirs):
                    if causal and b > a:
                        continue
                    blk = torch.cat([qs[i], _rows(kv, B, S, nc, j)], 1)
                    g = att.attention_bwd(blk, outs[i], lse[i], dos[i], B, sc, H, Hkv, dh,
                                          causal=causal and a == b).float()
                    dq[:, i] += g[:, :qd].view(B, sc, qd)
                    dkv[:, j] += g[:, qd:].view(B, sc, kvd)
            # the gradient follows its shard once this hop's share is added; after the last hop it is home
            if hop is not None:
                kv = hop.wait()
            dkv = _ring_exchange(dkv.reshape(B * S, kvd), group, rank, W).view(B, nc, sc, kvd)
        dqkv = torch.cat([dq.reshape(B * S, qd), dkv.reshape(B * S, kvd)], 1).to(qkv.dtype)
        return dqkv, None, None, None, None, None, None, None, None


def ring_attention(qkv: torch.Tensor, B: int, S_local: int, H: int, Hkv: int, dh: int, group=None,
                   causal: bool = True, layout: str = "contiguous") -> torch.Tensor:
    """Attention output ``[B * S_local, H * dh]`` of this rank's queries over the WHOLE sequence (``world * S_local``
    tokens per sequence, sharded by ``shard_sequence`` with the same ``layout``). Differentiable w.r.t. ``qkv``."""
    group = group if group is not None else dist.group.WORLD
    if layout == "zigzag" and S_local % 2:
        raise ValueError("the zigzag layout needs an even number of local tokens")
    return _RingAttention.apply(qkv, B, S_local, H, Hkv, dh, group, causal, layout)


def shard_sequence(x: torch.Tensor, B: int, S: int, group=None, layout: str = "contiguous") -> torch.Tensor:
    """Rows of ``x [B * S, C]`` that belong to this rank: its contiguous slice of every sequence, or (``zigzag``) chunks
    ``r`` and ``2W - 1 - r`` of ``2W``, concatenated in that order."""
    group = group if group is not None else dist.group.WORLD
    rank, W = dist.get_rank(group), dist.get_world_size(group)
    ids = _chunk_ids(rank, W, layout)
    n = W * len(ids)
    if S % n:
        raise ValueError("sequence length must be a multiple of the number of chunks")
    sc = S // n
    xv = x.view(B, n, sc, -1)
    return torch.cat([xv[:, c] for c in ids], 1).reshape(B * sc * len(ids), -1).contiguous()


def visible_pairs(world: int, layout: str) -> list:
    """(query chunk, key chunk) pairs with at least one visible key under a causal mask, per rank: the work measure."""
    out = []
    for r in range(world):
        n = 0
        for src in range(world):
            for a in _chunk_ids(r, world, layout):
                for b in _chunk_ids(src, world, layout):
                    n += b <= a
        out.append(n)
    return out

#!/usr/bin/env python
"""Runs each fused compute+collective kernel once per iteration in a ONE-rank group, so that a
profiler can capture it on a single GPU (a profiler must not wrap a multi-rank command). With one
rank every "peer" pointer is the local buffer: the instruction stream, tile loop, flag protocol and
epilogues are the ones the multi-rank runs execute, only the NVLink hops are local.

    python -m scirust_b200.parallel.profile_single_rank --iters 3
    SB_TP_PAIR_SINGLE=1 python -m scirust_b200.parallel.profile_single_rank --iters 3    # the CTA-pair kernels
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.fused_allreduce import FusedAllReduce  # noqa: E402
from scirust_b200.parallel.small_collectives import SmallCollectives  # noqa: E402
from scirust_b200.parallel.symm import SymmetricRegion  # noqa: E402
from scirust_b200.parallel.tensor_parallel import TPContext  # noqa: E402

BF = torch.bfloat16


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ff", type=int, default=7168)
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29733")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device="cuda").manual_seed(0)

    def rnd(shape):
        return (torch.randn(shape, generator=g, device="cuda") * 0.05).to(BF)
    # gradient all-reduce: 64 M bf16 elements (128 MB, larger than L2)
    n = 64 << 20
    region = SymmetricRegion(dist.group.WORLD, n * 4 + (1 << 20), device=dev)
    src, dst = region.tensor((n,), BF), region.tensor((n,), BF)
    src.copy_(rnd((n,)))
    ar = FusedAllReduce(region, src, dst, n_ctas=64)
    coll = SmallCollectives(dist.group.WORLD, region)
    small = coll.source("x", (8, a.d), torch.float32)
    res = rnd((8, a.d))
    # distributed GEMMs
    T, d, ff = a.tokens, a.d, a.ff
    ctx = TPContext(dist.group.WORLD, max_rows=T, max_cols=max(d, ff), sym_bytes=T * d * 2 + (1 << 20))
    x = ctx.buffer("x", (T, d))
    x.copy_(rnd((T, d)))
    w1, h, w2 = rnd((d, ff)), rnd((T, ff)), rnd((ff, d))
    for _ in range(a.iters):
        ar.reduce(0, n, 1.0, ar.next_epoch())
        coll.all_reduce(small, residual=res)
        y1 = ctx.ag_matmul_nn(x, w1)
        y2 = ctx.matmul_nn_rs(h, w2)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    for got, ref in ((y1, x.float() @ w1.float()), (y2, h.float() @ w2.float())):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * max(1.0, ref.abs().max().item()), err
    ctx.close()
    region.close()
    dist.destroy_process_group()
    print("FUSED_SINGLE_RANK_OK")


if __name__ == "__main__":
    main()

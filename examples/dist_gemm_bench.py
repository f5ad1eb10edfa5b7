#!/usr/bin/env python
"""Fused compute+collective GEMMs against the NCCL + library-GEMM baseline, with roofline fractions.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/dist_gemm_bench.py
    ... --tokens 16384 --d 4096 --ff 14336       (Llama-3-8B-shape MLP, the default)

Per rank, W ranks, T tokens: the column-parallel product all-gather(x [T/W, d]) @ W1 [d, ff/W] and the
row-parallel product reduce-scatter(h [T, ff/W] @ W2 [ff/W, d]). Times are CUDA events on the launching
stream after warm-up (the call is queued behind a short spin kernel, so the host's launch latency is not in the
interval), maximum over ranks; every iteration's inputs are larger than L2 together with a
256 MiB scratch rewrite between iterations. The roofline time of a fused kernel is the slower of its FLOPs at
the measured bf16 GEMM rate and the bytes it must move over NVLink at the measured peer-copy rate.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

os.environ.setdefault("SB_TP_RS_MIN_GFLOP", "0")   # time the fused kernels at every size

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.tensor_parallel import TPContext  # noqa: E402

BF = torch.bfloat16
GEMM_TFLOPS = 1380.7     # measured sustained cuBLAS bf16 rate of a B200 under its power cap (TFLOP/s)
LINK_GBS = 770.0         # measured peer-copy rate per direction per GPU (GB/s)


def timed(fn, iters, warmup, scratch):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        scratch.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda._sleep(3_000_000)    # the GPU spins ~1.5 ms while the host queues the call: no launch latency in the time
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--d-model", dest="d", type=int, default=4096)
    ap.add_argument("--ff", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    W, rank = dist.get_world_size(), dist.get_rank()
    T, d, ffl = a.tokens, a.d, a.ff // W
    Tl = T // W
    g = torch.Generator(device="cuda").manual_seed(10 + rank)

    def rnd(shape):
        return (torch.randn(shape, generator=g, device="cuda") * 0.05).to(BF)
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for backend in ("fused", "nccl"):
        ctx = TPContext(dist.group.WORLD, max_rows=T, max_cols=max(d, ffl), sym_bytes=Tl * d * 2 + (1 << 20),
                        backend=backend)
        x_shard = ctx.buffer("x", (Tl, d))
        x_shard.copy_(rnd((Tl, d)))
        w1, h, w2 = rnd((d, ffl)), rnd((T, ffl)), rnd((ffl, d))
        ms_ag = timed(lambda: ctx.ag_matmul_nn(x_shard, w1), a.iters, a.warmup, scratch)
        ms_rs = timed(lambda: ctx.matmul_nn_rs(h, w2), a.iters, a.warmup, scratch)
        _lib.check_status(torch.device("cuda", local))
        fl = 2.0 * T * d * ffl
        # bytes that must cross NVLink into / out of one GPU
        ag_bytes = (W - 1) * Tl * d * 2
        rs_bytes = (W - 1) * Tl * d * 2
        roof_ag = max(fl / (GEMM_TFLOPS * 1e12), ag_bytes / (LINK_GBS * 1e9)) * 1e3
        roof_rs = max(fl / (GEMM_TFLOPS * 1e12), rs_bytes / (LINK_GBS * 1e9)) * 1e3
        rows.append({"backend": backend, "ag_gemm_ms": ms_ag, "ag_gemm_tflops": fl / ms_ag / 1e9,
                     "ag_gemm_of_roofline": roof_ag / ms_ag, "gemm_rs_ms": ms_rs,
                     "gemm_rs_tflops": fl / ms_rs / 1e9, "gemm_rs_of_roofline": roof_rs / ms_rs})
        ctx.close()
    if rank == 0:
        print(json.dumps({"bench": "dist_gemm", "world": W, "tokens": T, "d": d, "ff_local": ffl,
                          "roofline": {"gemm_tflops": GEMM_TFLOPS, "link_gbs": LINK_GBS}, "rows": rows}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Fused gradient all-reduce (csrc/comm.cu) against NCCL's all-reduce on the same buffers.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/allreduce_bench.py \
        --elems 11272192,32768000 --ctas 16,32,48

For every element count (bf16 in, bf16 out; a decoder layer's gradient bucket is 11.27 M elements, the tied
embedding 32.8 M) and every CTA count it prints the time of one call (CUDA events on the launching stream,
maximum over ranks, mean of ``--iters`` calls after warm-up; a 256 MiB buffer is rewritten between calls so
nothing is served from L2) and the bus bandwidth 2 (W-1)/W x bytes / time.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.fused_allreduce import FusedAllReduce  # noqa: E402
from scirust_b200.parallel.symm import SymmetricRegion  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", default="11272192,32768000")
    ap.add_argument("--ctas", default="16,32,48,64")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    sizes = [int(x) // 8 * 8 for x in a.elems.split(",")]
    nmax = max(sizes)
    region = SymmetricRegion(dist.group.WORLD, nmax * 4 + 8192)
    src = region.tensor((nmax,), torch.bfloat16)
    dst = region.tensor((nmax,), torch.bfloat16)
    src.copy_(torch.randn(nmax, device=dev).to(torch.bfloat16))
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def timed(fn):
        for _ in range(3):
            fn()
        tot = 0.0
        for _ in range(a.iters):
            scratch.zero_()
            dist.barrier()
            torch.cuda._sleep(3_000_000)    # the GPU spins ~1.5 ms while the host queues the call
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        t = torch.tensor([tot / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for n in sizes:
        nccl_buf = torch.empty(n, dtype=torch.bfloat16, device=dev)

        def nccl():
            nccl_buf.copy_(src[:n])
            dist.all_reduce(nccl_buf)
        copy_ms = timed(lambda: nccl_buf.copy_(src[:n]))
        ms = timed(nccl) - copy_ms
        bus = 2 * (world - 1) / world * n * 2 / (ms * 1e6)
        rows.append({"elems": n, "impl": "nccl", "ms": round(ms, 4), "busbw_gbs": round(bus, 1)})
        for ctas in [int(c) for c in a.ctas.split(",")]:
            ar = FusedAllReduce(region, src, dst, n_ctas=ctas)
            ms = timed(lambda: ar.reduce(0, n, 1.0 / world))
            _lib.check_status(dev)
            bus = 2 * (world - 1) / world * n * 2 / (ms * 1e6)
            rows.append({"elems": n, "impl": f"fused/{ctas} CTAs", "ms": round(ms, 4), "busbw_gbs": round(bus, 1)})
        ar = FusedAllReduce(region, src, dst)
        ms = timed(lambda: ar.reduce(0, n, 1.0 / world, lean=True))
        _lib.check_status(dev)
        bus = 2 * (world - 1) / world * n * 2 / (ms * 1e6)
        rows.append({"elems": n, "impl": f"fused lean/{ar.lean_ctas} CTAs x 128 threads", "ms": round(ms, 4),
                     "busbw_gbs": round(bus, 1)})
    if rank == 0:
        print(json.dumps({"world": world, "rows": rows}))
    region.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

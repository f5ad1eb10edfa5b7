#!/usr/bin/env python
"""Data-parallel vision training on synthetic data.

    # MNIST-shaped CNN, batch 512 per GPU, Adam 1e-3 (bf16 compute, fp32 master weights)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_dp_vision.py --model mnist_cnn
    # CIFAR-10-shaped ResNet-18, batch 256 per GPU, SGD momentum 0.9
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_dp_vision.py --model resnet18

Gradients are reduced by the fused all-reduce (cast to bf16 buckets, rank-ordered fp32 sum, 1/world
scale) overlapped with backward; ``--comm nccl`` selects the NCCL baseline. Prints one JSON line with
images/s (device-timed, max over ranks)."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from scirust_b200.models.cnn import MnistCNN, ResNet18  # noqa: E402
from scirust_b200.ops import _lib  # noqa: E402
from scirust_b200.parallel.ddp import FlatDataParallel  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mnist_cnn", choices=["mnist_cnn", "resnet18"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--batch", type=int, default=0)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    lr_ = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(lr_)
    dev = torch.device("cuda", lr_)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(1000 + rank)
    if a.model == "mnist_cnn":
        B = a.batch or 512
        model = MnistCNN(seed=0).to(dev)
        dp = FlatDataParallel(model, dist.group.WORLD if world > 1 else None, "adam", lr=1e-3, comm=a.comm)
        data = [(torch.rand(B, 784, generator=g).to(dev), torch.randint(0, 10, (B,), generator=g).to(dev)) for _ in range(4)]
    else:
        B = a.batch or 256
        model = ResNet18(seed=0).to(dev)
        dp = FlatDataParallel(model, dist.group.WORLD if world > 1 else None, "sgd", lr=0.05, momentum=0.9, comm=a.comm)
        data = [(torch.randn(B, 3 * 32 * 32, generator=g).to(dev), torch.randint(0, 10, (B,), generator=g).to(dev)) for _ in range(4)]

    def step(i):
        x, y = data[i % 4]
        loss = F.cross_entropy(dp(x), y)
        loss.backward()
        dp.step()
        return loss
    for i in range(a.warmup):
        step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    _lib.check_status(dev)
    if rank == 0:
        print(json.dumps({"metric": f"{a.model} train images/s", "value": B * world * a.steps / (float(ms) / 1e3),
                          "n_gpus": world, "batch_per_gpu": B, "ms_per_step": float(ms) / a.steps, "comm": a.comm,
                          "loss": float(loss.detach()), "dtype": "bf16 compute, fp32 masters", "data": "synthetic"}))
    dp.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

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


def _torch_model(name):
    import torch.nn as nn

    def block(i, o, s):
        class B(nn.Module):
            def __init__(self):
                super().__init__()
                self.c1, self.b1 = nn.Conv2d(i, o, 3, s, 1, bias=False), nn.BatchNorm2d(o)
                self.c2, self.b2 = nn.Conv2d(o, o, 3, 1, 1, bias=False), nn.BatchNorm2d(o)
                self.sh = None if (s == 1 and i == o) else nn.Sequential(nn.Conv2d(i, o, 1, s, 0, bias=False), nn.BatchNorm2d(o))

            def forward(self, x):
                y = self.b2(self.c2(torch.relu(self.b1(self.c1(x)))))
                return torch.relu(y + (x if self.sh is None else self.sh(x)))
        return B()
    if name == "mnist_cnn":
        return nn.Sequential(nn.Unflatten(1, (1, 28, 28)), nn.Conv2d(1, 32, 3), nn.ReLU(), nn.Conv2d(32, 64, 3), nn.ReLU(),
                             nn.MaxPool2d(2), nn.Flatten(), nn.Linear(12 * 12 * 64, 128), nn.ReLU(), nn.Linear(128, 10))
    layers, c = [nn.Unflatten(1, (3, 32, 32)), nn.Conv2d(3, 64, 3, 1, 1, bias=False), nn.BatchNorm2d(64), nn.ReLU()], 64
    for i, w in enumerate((64, 128, 256, 512)):
        for j in range(2):
            layers.append(block(c, w, 2 if (j == 0 and i > 0) else 1))
            c = w
    return nn.Sequential(*layers, nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(c, 10))


def torch_arm(a, rank, world, dev, g):
    """The comparison arm: none of this framework's kernels; cuDNN convolutions in channels_last, bf16 autocast,
    fused optimizers, NCCL DistributedDataParallel."""
    B = a.batch or (512 if a.model == "mnist_cnn" else 256)
    feat = 784 if a.model == "mnist_cnn" else 3 * 32 * 32
    model = _torch_model(a.model).to(dev).to(memory_format=torch.channels_last)
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index])
    opt = (torch.optim.Adam(model.parameters(), lr=1e-3, fused=True) if a.model == "mnist_cnn"
           else torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9))
    gen = (torch.rand if a.model == "mnist_cnn" else torch.randn)
    data = [(gen(B, feat, generator=g).to(dev), torch.randint(0, 10, (B,), generator=g).to(dev)) for _ in range(4)]

    def step(i):
        x, y = data[i % 4]
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(model(x).float(), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
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
    if rank == 0:
        print(json.dumps({"metric": f"{a.model} train images/s", "value": B * world * a.steps / (float(ms) / 1e3),
                          "n_gpus": world, "batch_per_gpu": B, "ms_per_step": float(ms) / a.steps, "impl": "torch",
                          "comm": "nccl ddp", "loss": float(loss.detach()), "dtype": "bf16 autocast", "data": "synthetic"}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mnist_cnn", choices=["mnist_cnn", "resnet18"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"],
                    help="torch = the same architecture on stock PyTorch (cuDNN, channels_last, bf16 autocast, DDP)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    lr_ = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(lr_)
    dev = torch.device("cuda", lr_)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator().manual_seed(1000 + rank)
    if a.impl == "torch":
        return torch_arm(a, rank, world, dev, g)
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

#!/usr/bin/env python
"""CIFAR-10 CNN in the shape of the reference's example: conv 3->32->64 (3x3, same) + ReLU + 2x2 max-pool each,
4096 -> 256 -> 10, Adam 1e-3, batch 128 (examples/cifar10_classifier/src/main.rs:19-213).

    python examples/cifar10_classifier.py --data DIR      # DIR holds data_batch_{1..5}.bin and test_batch.bin
    python examples/cifar10_classifier.py                 # no files: a learnable synthetic stand-in
    python examples/cifar10_classifier.py --device cuda   # the native NHWC path (tcgen05 GEMM convolutions)

On CPU the model is built from the framework's ``nn`` modules (NCHW flattened rows, as the reference lays images out);
with ``--device cuda`` it is a narrow ``models.cnn.ResNet18`` on the native NHWC convolution kernels, trained through
``FlatDataParallel`` (world 1), the same code that scales it over several GPUs in ``examples/train_dp_vision.py``.
"""
import argparse
import glob
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from scirust_b200 import nn  # noqa: E402
from scirust_b200.data.datasets import DataLoader, InMemoryDataset, augment, load_cifar10_bin  # noqa: E402


def synthetic(n, seed):
    g = torch.Generator().manual_seed(seed)
    protos = torch.randn(10, 3 * 32 * 32, generator=torch.Generator().manual_seed(99))
    y = torch.randint(0, 10, (n,), generator=g)
    return InMemoryDataset(protos[y] + 1.5 * torch.randn(n, 3 * 32 * 32, generator=g), y)


def build_cpu_model(rng):
    P = nn.Padding.SAME
    return nn.Sequential(
        nn.Conv2d(3, 32, 3, 1, P, 32, 32, rng=rng), nn.ReLU(), nn.MaxPool2d(2, 2, 32, 32, 32),
        nn.Conv2d(32, 64, 3, 1, P, 16, 16, rng=rng), nn.ReLU(), nn.MaxPool2d(2, 2, 64, 16, 16),
        nn.Linear(64 * 8 * 8, 256, rng=rng), nn.ReLU(), nn.Linear(256, 10, rng=rng))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="")
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--train-size", type=int, default=2048, help="synthetic stand-in only")
    ap.add_argument("--augment", action="store_true", help="random flips and 4-pixel crops")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    if a.data:
        train = load_cifar10_bin(sorted(glob.glob(os.path.join(a.data, "data_batch_*.bin"))))
        test = load_cifar10_bin([os.path.join(a.data, "test_batch.bin")])
    else:
        train, test = synthetic(a.train_size, a.seed), synthetic(512, a.seed + 1)
    loader = DataLoader(train, a.batch_size, shuffle=True, seed=a.seed, drop_last=True)
    if a.device == "cuda":
        from scirust_b200.models.cnn import ResNet18
        from scirust_b200.parallel.ddp import FlatDataParallel
        model = ResNet18(10, widths=(32, 64, 128, 256), seed=a.seed).cuda()
        dp = FlatDataParallel(model, optimizer="adam", lr=a.lr)

        def step(xb, yb):
            loss = torch.nn.functional.cross_entropy(dp(xb.cuda()), yb.cuda())
            loss.backward()
            dp.step()
            return float(loss.detach())

        def predict(x):
            return model(x.cuda()).cpu()
    else:
        model = build_cpu_model(nn.PcgEngine(a.seed))
        opt = torch.optim.Adam(model.parameters(), lr=a.lr)

        def step(xb, yb):
            loss = torch.nn.functional.cross_entropy(model(xb), yb)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return float(loss.detach())

        def predict(x):
            return model(x)
    acc = 0.0
    for epoch in range(a.epochs):
        loader.set_epoch(epoch)
        total, n = 0.0, 0
        for i, (xb, yb) in enumerate(loader):
            if a.augment:
                xb = augment(xb, 3, 32, 32, seed=a.seed * 100003 + epoch * 1009 + i, flip=True, crop_pad=4)
            total += step(xb, yb)
            n += 1
        with torch.no_grad():
            acc = float((predict(test.x).argmax(1) == test.y).float().mean())
        print(f"epoch {epoch + 1}: train loss {total / max(n, 1):.4f}  test accuracy {acc * 100:.2f} %")
    return acc


if __name__ == "__main__":
    main()

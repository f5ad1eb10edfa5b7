#!/usr/bin/env python
"""MNIST classifier in the shape of the reference's example: MLP 784 -> 256 -> 10, Adam 1e-3, batch 64, 5 epochs
(examples/mnist_classifier/src/main.rs:17-198; documented result 97.70 % test accuracy).

    python examples/mnist_classifier.py --data DIR        # DIR holds the four IDX files (optionally .gz)
    python examples/mnist_classifier.py                   # no files: a learnable synthetic stand-in of the same shape

The loader is the framework's seeded ``DataLoader`` (PCG Fisher-Yates order per epoch), the layers its ``nn`` modules,
so the run is reproducible for a given seed on CPU.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from scirust_b200 import nn  # noqa: E402
from scirust_b200.data.datasets import DataLoader, InMemoryDataset, load_mnist_idx  # noqa: E402


def synthetic(n, seed):
    """Ten fixed random prototypes plus noise: same shapes and label space as MNIST, and learnable."""
    g = torch.Generator().manual_seed(seed)
    protos = torch.rand(10, 784, generator=torch.Generator().manual_seed(1234))
    y = torch.randint(0, 10, (n,), generator=g)
    x = (protos[y] + 0.35 * torch.randn(n, 784, generator=g)).clamp(0, 1)
    return InMemoryDataset(x, y)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="")
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--train-size", type=int, default=6000, help="synthetic stand-in only")
    a = ap.parse_args()
    if a.data:
        def f(name):
            for suf in ("", ".gz"):
                p = os.path.join(a.data, name + suf)
                if os.path.exists(p):
                    return p
            raise FileNotFoundError(name)
        train = load_mnist_idx(f("train-images-idx3-ubyte"), f("train-labels-idx1-ubyte"))
        test = load_mnist_idx(f("t10k-images-idx3-ubyte"), f("t10k-labels-idx1-ubyte"))
    else:
        train, test = synthetic(a.train_size, a.seed), synthetic(1000, a.seed + 1)
    rng = nn.PcgEngine(a.seed)
    model = nn.Sequential(nn.Linear(784, 256, rng=rng), nn.ReLU(), nn.Linear(256, 10, rng=rng))
    opt = torch.optim.Adam(model.parameters(), lr=a.lr)
    loader = DataLoader(train, a.batch_size, shuffle=True, seed=a.seed)
    for epoch in range(a.epochs):
        loader.set_epoch(epoch)
        total, seen = 0.0, 0
        for xb, yb in loader:
            loss = torch.nn.functional.cross_entropy(model(xb), yb)
            opt.zero_grad()
            loss.backward()
            opt.step()
            total += float(loss.detach()) * len(yb)
            seen += len(yb)
        with torch.no_grad():
            acc = float((model(test.x).argmax(1) == test.y).float().mean())
        print(f"epoch {epoch + 1}: train loss {total / seen:.4f}  test accuracy {acc * 100:.2f} %")
    return acc


if __name__ == "__main__":
    main()

"""Vision models of the core zoo: residual blocks and ResNet-18/34 (7x7 stride-2 stem + BN + four
stages + global average pool + FC; scirust-core/src/nn/vision.rs:11-120, nn/residual.rs), a
CIFAR-style ResNet-18 variant (3x3 stem, channels 64/128/256/512), the MNIST/CIFAR tutorial CNNs
(docs/MNIST.md:27-34; examples/cifar10_classifier/src/main.rs:19-213) and a small ViT (nn/vit.rs).
These models keep NCHW 4-D tensors internally and accept flattened ``(B, C*H*W)`` input."""
from __future__ import annotations

import torch
import torch.nn as tnn
import torch.nn.functional as F

from .modules import Module


class ResidualBlock(Module):
    def __init__(self, in_c, out_c, stride=1):
        super().__init__()
        self.conv1 = tnn.Conv2d(in_c, out_c, 3, stride, 1, bias=False)
        self.bn1 = tnn.BatchNorm2d(out_c)
        self.conv2 = tnn.Conv2d(out_c, out_c, 3, 1, 1, bias=False)
        self.bn2 = tnn.BatchNorm2d(out_c)
        self.short = None
        if stride != 1 or in_c != out_c:
            self.short = tnn.Sequential(tnn.Conv2d(in_c, out_c, 1, stride, bias=False), tnn.BatchNorm2d(out_c))

    def forward(self, x):
        y = F.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return F.relu(y + (x if self.short is None else self.short(x)))


class ResNet(Module):
    def __init__(self, blocks, num_classes=10, in_c=3, in_hw=32, cifar_stem=True, widths=(64, 128, 256, 512)):
        super().__init__()
        self.in_c, self.in_hw = in_c, in_hw
        if cifar_stem:
            self.stem = tnn.Sequential(tnn.Conv2d(in_c, widths[0], 3, 1, 1, bias=False), tnn.BatchNorm2d(widths[0]),
                                       tnn.ReLU())
        else:
            self.stem = tnn.Sequential(tnn.Conv2d(in_c, widths[0], 7, 2, 3, bias=False), tnn.BatchNorm2d(widths[0]),
                                       tnn.ReLU(), tnn.MaxPool2d(3, 2, 1))
        layers, c = [], widths[0]
        for i, (w, n) in enumerate(zip(widths, blocks)):
            for j in range(n):
                layers.append(ResidualBlock(c, w, stride=2 if (j == 0 and i > 0) else 1))
                c = w
        self.stages = tnn.Sequential(*layers)
        self.fc = tnn.Linear(c, num_classes)

    def forward(self, x):
        if x.dim() == 2:
            x = x.reshape(x.shape[0], self.in_c, self.in_hw, self.in_hw)
        y = self.stages(self.stem(x))
        return self.fc(y.mean((2, 3)))


def resnet18(num_classes=10, in_c=3, in_hw=32, cifar_stem=True):
    return ResNet((2, 2, 2, 2), num_classes, in_c, in_hw, cifar_stem)


def resnet34(num_classes=10, in_c=3, in_hw=32, cifar_stem=True):
    return ResNet((3, 4, 6, 3), num_classes, in_c, in_hw, cifar_stem)


class MnistCNN(Module):
    """conv 1->32->64 3x3 + ReLU + 2x2 max-pool -> Linear 128 -> 10."""

    def __init__(self, num_classes=10):
        super().__init__()
        self.c1, self.c2 = tnn.Conv2d(1, 32, 3), tnn.Conv2d(32, 64, 3)
        self.f1, self.f2 = tnn.Linear(64 * 12 * 12, 128), tnn.Linear(128, num_classes)

    def forward(self, x):
        if x.dim() == 2:
            x = x.reshape(x.shape[0], 1, 28, 28)
        y = F.max_pool2d(F.relu(self.c2(F.relu(self.c1(x)))), 2)
        return self.f2(F.relu(self.f1(y.flatten(1))))


class CifarCNN(Module):
    """conv 3->32->64 (3x3, same) each followed by ReLU + 2x2 pool, 4096 -> 256 -> 10."""

    def __init__(self, num_classes=10):
        super().__init__()
        self.c1, self.c2 = tnn.Conv2d(3, 32, 3, padding=1), tnn.Conv2d(32, 64, 3, padding=1)
        self.f1, self.f2 = tnn.Linear(64 * 8 * 8, 256), tnn.Linear(256, num_classes)

    def forward(self, x):
        if x.dim() == 2:
            x = x.reshape(x.shape[0], 3, 32, 32)
        y = F.max_pool2d(F.relu(self.c1(x)), 2)
        y = F.max_pool2d(F.relu(self.c2(y)), 2)
        return self.f2(F.relu(self.f1(y.flatten(1))))


class ViT(Module):
    def __init__(self, image=32, patch=4, in_c=3, d_model=128, n_heads=4, n_layers=4, d_ff=256, num_classes=10):
        super().__init__()
        self.patch, self.in_c, self.image = patch, in_c, image
        n = (image // patch) ** 2
        self.proj = tnn.Conv2d(in_c, d_model, patch, patch)
        self.cls = tnn.Parameter(torch.zeros(1, 1, d_model))
        self.pos = tnn.Parameter(torch.randn(1, n + 1, d_model) * 0.02)
        layer = tnn.TransformerEncoderLayer(d_model, n_heads, d_ff, dropout=0.0, batch_first=True, norm_first=True)
        self.enc = tnn.TransformerEncoder(layer, n_layers)
        self.ln, self.head = tnn.LayerNorm(d_model), tnn.Linear(d_model, num_classes)

    def forward(self, x):
        if x.dim() == 2:
            x = x.reshape(x.shape[0], self.in_c, self.image, self.image)
        t = self.proj(x).flatten(2).transpose(1, 2)
        t = torch.cat([self.cls.expand(t.shape[0], -1, -1), t], 1) + self.pos
        return self.head(self.ln(self.enc(t)[:, 0]))

"""Convolutional classifiers on the native NHWC kernels: the MNIST-shaped CNN
(conv 1->32->64 3x3 + ReLU + 2x2 max-pool -> Linear 128 -> 10; docs/MNIST.md:27-34) and a
CIFAR-shaped ResNet-18 (3x3 stem, channels 64/128/256/512, BatchNorm, ReLU, global average pool,
FC; scirust-core/src/nn/vision.rs:65-72). Parameters are fp32 masters; compute runs in bf16 through
``ops.conv`` (im2col + tcgen05 GEMM, BatchNorm and pooling kernels) on CUDA and through
``torch.nn.functional`` on CPU. Convolution weights are kept in the packed ``[out_c, pad8(k*k*in_c)]``
layout; ``state_dict_ref`` converts back to the reference's ``(out_c, in_c*k*k)``."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..ops import conv as C

BF = torch.bfloat16


class ConvLayer(nn.Module):
    def __init__(self, in_c, out_c, k, stride=1, pad=0, bias=False, gen=None):
        super().__init__()
        self.in_c, self.out_c, self.k, self.stride, self.pad = in_c, out_c, k, stride, pad
        std = math.sqrt(2.0 / (in_c * k * k))
        w = torch.randn(out_c, in_c * k * k, generator=gen) * std
        self.weight = nn.Parameter(C.pack_conv_weight(w, in_c, k))
        self.bias = nn.Parameter(torch.zeros(out_c)) if bias else None

    def forward(self, x, geom):
        y, og = C.conv2d(x, self.weight.to(BF), geom, self.k, self.stride, self.pad)
        if self.bias is not None:
            y = y + self.bias.to(BF)
        return y, og

    def weight_ref(self):
        return C.unpack_conv_weight(self.weight.detach(), self.in_c, self.k)


class BNLayer(nn.Module):
    def __init__(self, c, relu=False):
        super().__init__()
        self.gamma, self.beta = nn.Parameter(torch.ones(c)), nn.Parameter(torch.zeros(c))
        self.register_buffer("running_mean", torch.zeros(c))
        self.register_buffer("running_var", torch.ones(c))
        self.relu = relu

    def forward(self, x):
        return C.batchnorm(x, self.gamma, self.beta, self.running_mean, self.running_var, relu=self.relu,
                           training=self.training)


class _DenseFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return ops.matmul_nn(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        return ops.matmul_nt(dy, w), ops.matmul_tn(x, dy)


class Dense(nn.Module):
    """x.W + b with W [in, out]; the out dimension is padded to a multiple of 8 internally."""

    def __init__(self, in_f, out_f, gen=None):
        super().__init__()
        self.out_f = out_f
        op = (out_f + 7) // 8 * 8
        w = torch.zeros(in_f, op)
        w[:, :out_f] = torch.randn(in_f, out_f, generator=gen) * math.sqrt(2.0 / in_f)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(op))

    def forward(self, x):
        w = self.weight.to(BF)
        y = _DenseFn.apply(x.contiguous(), w) if x.is_cuda else (x.float() @ w.float()).to(x.dtype)
        return (y + self.bias.to(y.dtype))[:, : self.out_f]


class MnistCNN(nn.Module):
    def __init__(self, num_classes=10, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.c1, self.c2 = ConvLayer(1, 32, 3, bias=True, gen=g), ConvLayer(32, 64, 3, bias=True, gen=g)
        self.f1, self.f2 = Dense(12 * 12 * 64, 128, g), Dense(128, num_classes, g)

    def forward(self, x):
        """x: [B, 784] or [B, 1, 28, 28] in any float dtype."""
        B = x.shape[0]
        rows = x.reshape(B, 28 * 28, 1).reshape(B * 784, 1).to(BF)
        g = C.ConvGeom(B, 28, 28, 1)
        y, g = self.c1(rows, g)
        y, g = self.c2(torch.relu(y), g)
        y, g = C.maxpool2d(torch.relu(y), g, 2, 2)
        y = y.reshape(B, g.H * g.W * g.C)
        return self.f2(torch.relu(self.f1(y))).float()


class BasicBlock(nn.Module):
    def __init__(self, in_c, out_c, stride, gen):
        super().__init__()
        self.conv1, self.bn1 = ConvLayer(in_c, out_c, 3, stride, 1, gen=gen), BNLayer(out_c, relu=True)
        self.conv2, self.bn2 = ConvLayer(out_c, out_c, 3, 1, 1, gen=gen), BNLayer(out_c)
        self.short = None
        if stride != 1 or in_c != out_c:
            self.short, self.short_bn = ConvLayer(in_c, out_c, 1, stride, 0, gen=gen), BNLayer(out_c)

    def forward(self, x, g):
        y, g1 = self.conv1(x, g)
        y, g2 = self.conv2(self.bn1(y), g1)
        y = self.bn2(y)
        s = x if self.short is None else self.short_bn(self.short(x, g)[0])
        return torch.relu(y + s), g2


class ResNet18(nn.Module):
    def __init__(self, num_classes=10, widths=(64, 128, 256, 512), seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.stem, self.stem_bn = ConvLayer(3, widths[0], 3, 1, 1, gen=g), BNLayer(widths[0], relu=True)
        blocks, c = [], widths[0]
        for i, w in enumerate(widths):
            for j in range(2):
                blocks.append(BasicBlock(c, w, 2 if (j == 0 and i > 0) else 1, g))
                c = w
        self.blocks = nn.ModuleList(blocks)
        self.fc = Dense(c, num_classes, g)

    def forward(self, x):
        """x: [B, 3*32*32] or [B, 3, 32, 32]."""
        B = x.shape[0]
        rows, g = C.nchw_to_rows(x.reshape(B, 3, 32, 32).to(BF))
        y, g = self.stem(rows, g)
        y = self.stem_bn(y)
        for b in self.blocks:
            y, g = b(y, g)
        pooled = y.reshape(B, g.H * g.W, g.C).float().mean(1).to(BF)
        return self.fc(pooled).float()

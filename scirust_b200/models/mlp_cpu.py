"""Deterministic CPU training of small dense classifiers in fp32 with a fixed arithmetic order.

This is the CPU path in the mould of the reference's ``scirust quickstart`` (scirust-cli/src/
quickstart.rs:36-117; examples/quickstart_v2/src/main.rs:40-167): a ``Sequential`` of ``Linear``
layers (Kaiming-normal weights from a seeded PCG stream, zero biases) with ReLU between them,
softmax cross-entropy written operation by operation as the reference loss does
(nn/loss/cross_entropy.rs:75-134), plain SGD (autodiff/optim.rs:80-110), one tape per batch.

Every floating-point operation is issued in a documented order: matrix products accumulate each
output element over ascending k in one fp32 accumulator (``fma=False``: product and sum rounded
separately; ``fma=True``: fused, the order an FMA micro-kernel produces), bias gradients add rows
top to bottom, exp/log are glibc ``expf``/``logf``. Two runs with the same seed therefore produce the
same bits, on any thread count. The reference's own GEMM is ``matrixmultiply::sgemm`` 0.3.11 whose
accumulation order depends on the CPU's micro-kernel; the reference cannot be built in this image
(no Rust toolchain), so bit equality is claimed against this restatement of its arithmetic, not
against a reference binary.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ..data.datasets import DataLoader, gaussian_clusters
from ..nn import init as I
from ..nn.rng import PcgEngine
from ..ops import _lib

_cfg = False


def _rt():
    global _cfg
    lib = _lib.rt()
    if not _cfg:
        p, i64, ci = C.c_void_p, C.c_int64, C.c_int
        lib.sbrt_gemm_f32.argtypes = [p, p, p, i64, i64, i64, ci, ci, ci]
        lib.sbrt_gemm_f32.restype = None
        lib.sbrt_softmax_ce_f32.argtypes = [p, p, p, i64, i64]
        lib.sbrt_softmax_ce_f32.restype = C.c_float
        lib.sbrt_sgd_step_f32.argtypes = [p, p, p, i64, C.c_float, C.c_float, C.c_float]
        lib.sbrt_sgd_step_f32.restype = None
        _cfg = True
    return lib


def gemm(a: np.ndarray, b: np.ndarray, trans_a=False, trans_b=False, fma=False) -> np.ndarray:
    """Fixed-order fp32 product op(a)·op(b); a, b C-contiguous fp32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    c = np.empty((M, N), dtype=np.float32)
    _rt().sbrt_gemm_f32(a.ctypes.data, b.ctypes.data, c.ctypes.data, M, K, N, int(trans_a), int(trans_b), int(fma))
    return c


def _colsum(x: np.ndarray) -> np.ndarray:
    acc = np.zeros((1, x.shape[1]), dtype=np.float32)
    for r in range(x.shape[0]):
        acc = (acc + x[r:r + 1]).astype(np.float32)
    return acc


class DeterministicMLP:
    def __init__(self, sizes, seed: int = 42, fma: bool = False):
        rng = PcgEngine(seed)
        self.fma = fma
        self.W, self.b = [], []
        for i, o in zip(sizes[:-1], sizes[1:]):
            self.W.append(I.KaimingNormal().fill((i, o), i, o, rng).numpy().copy())
            self.b.append(np.zeros((1, o), dtype=np.float32))
        self.vW = [np.zeros_like(w) for w in self.W]
        self.vb = [np.zeros_like(b) for b in self.b]

    def forward(self, x: np.ndarray):
        acts = [np.ascontiguousarray(x, dtype=np.float32)]
        for li, (w, b) in enumerate(zip(self.W, self.b)):
            z = (gemm(acts[-1], w, fma=self.fma) + b).astype(np.float32)
            acts.append(np.maximum(z, np.float32(0)) if li + 1 < len(self.W) else z)
        return acts

    def loss_and_grads(self, x, y):
        acts = self.forward(x)
        logits = acts[-1]
        B, Cn = logits.shape
        d = np.empty_like(logits)
        tgt = np.ascontiguousarray(y, dtype=np.int64)
        loss = float(_rt().sbrt_softmax_ce_f32(logits.ctypes.data, tgt.ctypes.data, d.ctypes.data, B, Cn))
        gW, gb = [None] * len(self.W), [None] * len(self.W)
        for li in range(len(self.W) - 1, -1, -1):
            gW[li] = gemm(acts[li], d, trans_a=True, fma=self.fma)
            gb[li] = _colsum(d)
            if li > 0:
                d = gemm(d, self.W[li], trans_b=True, fma=self.fma)
                d = np.where(acts[li] > 0, d, np.float32(0)).astype(np.float32)
        return loss, gW, gb

    def sgd_step(self, gW, gb, lr: float, momentum: float = 0.0, wd: float = 0.0):
        lib = _rt()
        for p, v, g in list(zip(self.W, self.vW, gW)) + list(zip(self.b, self.vb, gb)):
            g = np.ascontiguousarray(g, dtype=np.float32)
            lib.sbrt_sgd_step_f32(p.ctypes.data, v.ctypes.data, g.ctypes.data, p.size, lr, momentum, wd)

    def predict(self, x) -> np.ndarray:
        return self.forward(x)[-1].argmax(1)

    def fingerprint(self) -> int:
        from ..io.artifacts import FNV_INIT, fnv_fold_f32
        fp = FNV_INIT
        for w, b in zip(self.W, self.b):
            fp = fnv_fold_f32(fnv_fold_f32(fp, torch.from_numpy(w)), torch.from_numpy(b))
        return fp

    def state_dict_ref(self) -> dict:
        """Sequential-style keys: Linear layers sit at even indices with ReLU between them."""
        sd = {}
        for i, (w, b) in enumerate(zip(self.W, self.b)):
            sd[f"{2 * i}.weight"] = torch.from_numpy(w.copy())
            sd[f"{2 * i}.bias"] = torch.from_numpy(b.copy())
        return sd


def train_gaussian_mlp(epochs: int = 100, batch: int = 16, lr: float = 0.1, seed: int = 42, fma: bool = False,
                       hidden: int = 16, log=None):
    """4 features -> Linear 16 + ReLU -> Linear 3 on 150 points from 3 Gaussian clusters
    (sigma 0.5, seed 42), SGD lr 0.1, batch 16, 100 epochs. Returns (model, history)."""
    ds = gaussian_clusters(150, 3, 4, 0.5, seed)
    model = DeterministicMLP([4, hidden, 3], seed=seed, fma=fma)
    loader = DataLoader(ds, batch, shuffle=True, seed=seed)
    hist = []
    for ep in range(epochs):
        loader.set_epoch(ep)
        tot, nb = 0.0, 0
        for xb, yb in loader._batches():
            loss, gW, gb = model.loss_and_grads(xb.numpy(), yb.numpy())
            model.sgd_step(gW, gb, lr)
            tot += loss
            nb += 1
        acc = float((model.predict(ds.x.numpy()) == ds.y.numpy()).mean())
        hist.append((tot / nb, acc))
        if log and (ep % 10 == 0 or ep == epochs - 1):
            log(f"epoch {ep:3d}  loss {tot / nb:.6f}  acc {acc:.4f}")
    return model, hist

"""Optimizers of the tape family: ``Sgd`` (momentum, L2 decay), ``Adam`` (bias correction, L2 decay,
AMSGrad) and ``AdamW`` (decoupled decay), with state keyed by tape node index
(scirust-core/src/autodiff/optim.rs:53-117, 123-251, 272-400). ``step(params, tape)`` reads
``tape.grad(idx)`` and writes ``tape.set_value(idx, ...)`` like the reference; the element
arithmetic is the reference's formula evaluated in fp32, on CPU through the native fixed-order
kernels (csrc/rt_rng_math.cpp) so seeded runs are reproducible bit for bit.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from ..ops import _lib

_cfg = False


def _rt():
    global _cfg
    lib = _lib.rt()
    if not _cfg:
        f, p, i64 = C.c_float, C.c_void_p, C.c_int64
        lib.sbrt_sgd_step_f32.argtypes = [p, p, p, i64, f, f, f]
        lib.sbrt_sgd_step_f32.restype = None
        lib.sbrt_adam_step_f32.argtypes = [p, p, p, p, i64, f, f, f, f, f, f, f, C.c_int]
        lib.sbrt_adam_step_f32.restype = None
        _cfg = True
    return lib


def _powi(base: float, n: int) -> np.float32:
    """f32::powi: repeated fp32 multiplication by squaring (matches LLVM's powi expansion closely
    enough that bias corrections agree to the last bit for the step counts in use)."""
    r, b = np.float32(1.0), np.float32(base)
    while n > 0:
        if n & 1:
            r = np.float32(r * b)
        b = np.float32(b * b)
        n >>= 1
    return r


class Optimizer:
    lr: float

    def step(self, params, tape) -> None:
        raise NotImplementedError

    def set_lr(self, lr: float) -> None:
        self.lr = lr


class Sgd(Optimizer):
    def __init__(self, lr: float):
        self.lr, self.momentum, self.weight_decay = lr, 0.0, 0.0
        self.velocities: dict = {}

    def with_momentum(self, m: float):
        self.momentum = m
        return self

    def with_weight_decay(self, wd: float):
        self.weight_decay = wd
        return self

    def step(self, params, tape) -> None:
        for idx in params:
            var = tape.vars[idx]
            p = var.t.detach()
            g = var.t.grad if var.t.grad is not None else torch.zeros_like(p)
            if p.shape != g.shape:
                raise ValueError(f"Sgd.step: shape mismatch param/grad (idx={idx})")
            v = self.velocities.setdefault(idx, torch.zeros_like(p))
            if p.is_cuda:
                gg = g + self.weight_decay * p if self.weight_decay > 0 else g
                v.mul_(self.momentum).add_(gg)
                p.sub_(self.lr * v)
            else:
                pc, gc = p.contiguous(), g.contiguous()
                _rt().sbrt_sgd_step_f32(pc.data_ptr(), v.data_ptr(), gc.data_ptr(), pc.numel(), self.lr,
                                        self.momentum, self.weight_decay)
                if pc.data_ptr() != p.data_ptr():
                    p.copy_(pc)


class Adam(Optimizer):
    decoupled = False

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8):
        self.lr, self.beta1, self.beta2, self.epsilon = lr, beta1, beta2, epsilon
        self.weight_decay, self.amsgrad, self.t = 0.0, False, 0
        self.m, self.v, self.v_max = {}, {}, {}

    def with_weight_decay(self, wd: float):
        self.weight_decay = wd
        return self

    def with_amsgrad(self):
        self.amsgrad = True
        return self

    def step(self, params, tape) -> None:
        self.t += 1
        bc1 = float(np.float32(1.0) - _powi(self.beta1, self.t))
        bc2 = float(np.float32(1.0) - _powi(self.beta2, self.t))
        for idx in params:
            var = tape.vars[idx]
            p = var.t.detach()
            g = var.t.grad if var.t.grad is not None else torch.zeros_like(p)
            if p.shape != g.shape:
                raise ValueError(f"{type(self).__name__}.step: shape mismatch param/grad (idx={idx})")
            m = self.m.setdefault(idx, torch.zeros_like(p))
            v = self.v.setdefault(idx, torch.zeros_like(p))
            if p.is_cuda or self.amsgrad:
                gg = g + self.weight_decay * p if (self.weight_decay > 0 and not self.decoupled) else g
                m.mul_(self.beta1).add_((1 - self.beta1) * gg)
                v.mul_(self.beta2).add_((1 - self.beta2) * gg * gg)
                v_hat = v / bc2
                if self.amsgrad:
                    vm = self.v_max.setdefault(idx, torch.zeros_like(p))
                    torch.maximum(vm, v, out=vm)
                    v_hat = vm / bc2
                upd = self.lr * (m / bc1) / (v_hat.sqrt() + self.epsilon)
                if self.decoupled:
                    upd = upd + self.lr * self.weight_decay * p
                p.sub_(upd)
            else:
                pc, gc = p.contiguous(), g.contiguous()
                _rt().sbrt_adam_step_f32(pc.data_ptr(), m.data_ptr(), v.data_ptr(), gc.data_ptr(), pc.numel(),
                                         self.lr, self.beta1, self.beta2, self.epsilon, self.weight_decay, bc1, bc2,
                                         1 if self.decoupled else 0)
                if pc.data_ptr() != p.data_ptr():
                    p.copy_(pc)


class AdamW(Adam):
    """Adam with decoupled weight decay: theta <- theta - lr*m_hat/(sqrt(v_hat)+eps) - lr*wd*theta."""
    decoupled = True

    def __init__(self, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8,
                 weight_decay: float = 0.01):
        super().__init__(lr, beta1, beta2, epsilon)
        self.weight_decay = weight_decay


class MuonOptimizer(Optimizer):
    """Muon on the tape family: momentum ``m = mu m + (1 - mu) g``; a matrix parameter (both sides >= 2) steps along
    the Newton-Schulz orthogonalisation of ``m`` scaled by ``sqrt(max(1, rows / cols))``, any other parameter along
    ``m`` itself; decoupled weight decay on both (scirust-sciagent/src/train/optimizer.rs:11-103)."""

    def __init__(self, lr: float, momentum: float = 0.95, ns_steps: int = 5, weight_decay: float = 0.0):
        self.lr, self.momentum, self.ns_steps, self.weight_decay = lr, momentum, ns_steps, weight_decay
        self.mu = {}

    def step(self, params, tape) -> None:
        from .nd_optim import newton_schulz_orthogonalize
        for idx in params:
            value, grad = tape.value(idx).t.clone(), tape.grad(idx).t
            if value.shape != grad.shape:
                raise ValueError(f"Muon.step: parameter / gradient shape mismatch (idx={idx})")
            mk = self.mu.get(idx)
            if mk is None:
                mk = self.mu[idx] = torch.zeros_like(value)
            mk.mul_(self.momentum).add_(grad, alpha=1.0 - self.momentum)
            rows, cols = value.shape
            if rows >= 2 and cols >= 2:
                upd = newton_schulz_orthogonalize(mk, self.ns_steps) * (max(rows / cols, 1.0) ** 0.5)
            else:
                upd = mk
            value.sub_(self.lr * (upd + self.weight_decay * value))
            tape.set_value(idx, value)


class TrainOptimizer:
    """The SciAgent trainer's optimizer choice (Adam or Muon) behind one interface, with ``apply_schedule``
    (scirust-sciagent/src/train/optimizer.rs:105-170)."""

    def __init__(self, inner):
        self.inner = inner

    @staticmethod
    def new_adam(lr: float) -> "TrainOptimizer":
        return TrainOptimizer(Adam(lr))

    @staticmethod
    def new_muon(lr: float) -> "TrainOptimizer":
        return TrainOptimizer(MuonOptimizer(lr))

    def with_weight_decay(self, wd: float) -> "TrainOptimizer":
        self.inner.weight_decay = wd
        return self

    def step(self, params, tape) -> None:
        self.inner.step(params, tape)

    @property
    def lr(self) -> float:
        return self.inner.lr

    def set_lr(self, lr: float) -> None:
        self.inner.set_lr(lr)

    def apply_schedule(self, scheduler, step: int) -> None:
        self.set_lr(scheduler.lr_at(step))

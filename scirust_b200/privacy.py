"""Differentially private training (DP-SGD, Abadi et al. 2016) with Renyi accounting.

One step: per-SAMPLE gradients, each clipped to L2 norm ``C``, summed, Gaussian noise of standard deviation
``noise_multiplier * C`` added, divided by the batch size. ``per_sample_gradients`` obtains all of them in ONE
batched backward pass (``torch.func.vmap`` over ``grad`` of the functional model), so the step costs about one
ordinary backward on the device instead of a loop over samples; ``dp_sgd_gradient`` does clip, sum, noise, average
on flat ``[batch, params]`` matrices (norms accumulated in float64, so large finite gradients do not overflow).

``MomentsAccountant`` / ``rdp_gaussian_epsilon``: conservative accounting that charges the un-subsampled Gaussian
RDP ``alpha / (2 sigma^2)`` per step at a grid of orders (1.05 ... 1.95, then 2 ... 256) and converts with
``eps = rdp + ln(1/delta) / (alpha - 1)``, minimised over the orders: an upper bound on epsilon.

The noise generator is a parameter: ``secure_generator()`` seeds one from the operating system's entropy pool; tests
pass a fixed seed. Reference counterpart: scirust-core/src/dp.rs:58-430 (flat per-sample vectors, CSPRNG-typed noise).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch


@dataclass
class DpSgdConfig:
    l2_norm_clip: float = 1.0
    noise_multiplier: float = 1.1
    delta: float = 1e-5
    epsilon: float | None = None

    def validate(self) -> None:
        if not math.isfinite(self.l2_norm_clip) or self.l2_norm_clip <= 0:
            raise ValueError("DP l2_norm_clip must be finite and > 0")
        if not math.isfinite(self.noise_multiplier) or self.noise_multiplier <= 0:
            raise ValueError("DP noise_multiplier must be finite and > 0")
        if not math.isfinite(self.delta) or not 0 < self.delta < 1:
            raise ValueError("DP delta must be finite and in (0, 1)")
        if self.epsilon is not None and (not math.isfinite(self.epsilon) or self.epsilon <= 0):
            raise ValueError("DP epsilon must be finite and > 0 when provided")
        if not math.isfinite(self.noise_multiplier * self.l2_norm_clip):
            raise ValueError("DP noise standard deviation must be finite and > 0")


def secure_generator(device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(os.urandom(8), "little") & ((1 << 63) - 1))
    return g


def _orders():
    return [1.0 + i * 0.05 for i in range(1, 20)] + [float(a) for a in range(2, 257)]


def gaussian_rdp(alpha: float, sigma: float) -> float:
    if not (alpha > 1.0 and sigma > 0.0):
        raise ValueError("gaussian_rdp: need alpha>1, sigma>0")
    return alpha / (2.0 * sigma * sigma)


def rdp_to_dp(rdp_eps: float, alpha: float, delta: float) -> float:
    if not (alpha > 1.0 and 0.0 < delta < 1.0):
        raise ValueError("rdp_to_dp: need alpha>1, delta in (0,1)")
    return rdp_eps + math.log(1.0 / delta) / (alpha - 1.0)


def rdp_gaussian_epsilon(steps: int, sigma: float, delta: float):
    """(epsilon, best order) after ``steps`` compositions of the Gaussian mechanism."""
    best = (math.inf, 0.0)
    for a in _orders():
        eps = rdp_to_dp(steps * gaussian_rdp(a, sigma), a, delta)
        if eps < best[0]:
            best = (eps, a)
    return best


class MomentsAccountant:
    def __init__(self, delta: float, q: float, sigma: float):
        self.delta, self.q, self.sigma = delta, q, sigma
        self.orders = _orders()
        self.log_moments = [0.0] * len(self.orders)
        self.steps, self.epsilon = 0, 0.0

    def step(self) -> None:
        self.steps += 1
        if self.sigma <= 0.0:
            self.epsilon = math.inf
            return
        for i, a in enumerate(self.orders):
            self.log_moments[i] += gaussian_rdp(a, self.sigma)
        self.epsilon = max(min(rdp_to_dp(m, a, self.delta) for m, a in zip(self.log_moments, self.orders)), 0.0)


def _check_finite(g, what):
    if not bool(torch.isfinite(g).all()):
        raise ValueError(f"{what} gradients must contain only finite values")


@torch.no_grad()
def clip_gradients(grads: torch.Tensor, l2_norm_clip: float) -> torch.Tensor:
    """Scale one flat gradient (or every row of ``[batch, params]``) to L2 norm at most ``l2_norm_clip``; in place."""
    if not math.isfinite(l2_norm_clip) or l2_norm_clip <= 0:
        raise ValueError("clip_gradients: l2_norm_clip must be finite and > 0")
    _check_finite(grads, "clip_gradients")
    g2 = grads if grads.dim() == 2 else grads.view(1, -1)
    norm = g2.double().pow(2).sum(1).sqrt()
    scale = torch.where((norm > l2_norm_clip) & (norm > 1e-12), l2_norm_clip / norm.clamp_min(1e-300), torch.ones_like(norm))
    g2.mul_(scale.to(g2.dtype)[:, None])
    return grads


@torch.no_grad()
def add_noise(grads: torch.Tensor, noise_stddev: float, generator: torch.Generator) -> torch.Tensor:
    if not math.isfinite(noise_stddev) or noise_stddev <= 0:
        raise ValueError("add_noise: noise_stddev must be finite and > 0")
    grads.add_(torch.randn(grads.shape, generator=generator, device=grads.device, dtype=grads.dtype) * noise_stddev)
    return grads


@torch.no_grad()
def dp_protect(per_sample_grad: torch.Tensor, config: DpSgdConfig, generator) -> torch.Tensor:
    """Clip one sample's gradient and add the mechanism's noise to it; in place."""
    config.validate()
    _check_finite(per_sample_grad, "dp_protect")
    clip_gradients(per_sample_grad, config.l2_norm_clip)
    return add_noise(per_sample_grad, config.noise_multiplier * config.l2_norm_clip, generator)


@torch.no_grad()
def dp_sgd_gradient(per_sample_grads, config: DpSgdConfig, generator) -> torch.Tensor:
    """``[batch, params]`` (or a list of equal-length vectors) -> the privatised mean gradient ``[params]``."""
    config.validate()
    if isinstance(per_sample_grads, (list, tuple)):
        if not per_sample_grads:
            raise ValueError("dp_sgd_gradient requires at least one sample")
        if len({int(torch.as_tensor(g).numel()) for g in per_sample_grads}) != 1:
            raise ValueError("dp_sgd_gradient requires equal-size per-sample gradients")
        per_sample_grads = torch.stack([torch.as_tensor(g, dtype=torch.float32).reshape(-1) for g in per_sample_grads])
    G = per_sample_grads.clone()
    if G.dim() != 2 or G.shape[0] == 0:
        raise ValueError("dp_sgd_gradient requires at least one sample")
    _check_finite(G, "dp_sgd_gradient")
    summed = clip_gradients(G, config.l2_norm_clip).sum(0)
    add_noise(summed, config.noise_multiplier * config.l2_norm_clip, generator)
    return summed / G.shape[0]


def per_sample_gradients(model: torch.nn.Module, loss_fn, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """``[batch, params]`` gradients of ``loss_fn(model(x_i), y_i)`` for every sample, in one batched backward."""
    from torch.func import functional_call, grad, vmap
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    params = {n: p.detach() for n, p in model.named_parameters() if p.requires_grad}
    buffers = {n: b.detach() for n, b in model.named_buffers()}

    def one(p, x, y):
        return loss_fn(functional_call(model, (p, buffers), (x[None],)), y[None])

    g = vmap(grad(one), in_dims=(None, 0, 0))(params, inputs, targets)
    return torch.cat([g[n].reshape(inputs.shape[0], -1) for n in names], 1)


class DpSgd:
    """Optimiser wrapper: ``step(inputs, targets)`` computes per-sample gradients, privatises them, applies plain SGD
    and charges the accountant; ``epsilon`` is the budget spent so far at the configured delta."""

    def __init__(self, model, loss_fn, lr: float, config: DpSgdConfig, generator=None, sample_rate: float = 1.0):
        config.validate()
        self.model, self.loss_fn, self.lr, self.config = model, loss_fn, lr, config
        self.generator = generator or secure_generator()
        self.accountant = MomentsAccountant(config.delta, sample_rate, config.noise_multiplier)

    @property
    def epsilon(self) -> float:
        return self.accountant.epsilon

    def step(self, inputs, targets) -> None:
        g = dp_sgd_gradient(per_sample_gradients(self.model, self.loss_fn, inputs, targets), self.config, self.generator)
        off = 0
        with torch.no_grad():
            for p in (p for p in self.model.parameters() if p.requires_grad):
                p.sub_(self.lr * g[off:off + p.numel()].reshape(p.shape).to(p.dtype))
                off += p.numel()
        self.accountant.step()
        if self.config.epsilon is not None and self.accountant.epsilon > self.config.epsilon:
            self.budget_exceeded = True

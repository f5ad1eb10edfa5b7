"""Mixed-precision trainer for the SciAgent decoder: bf16 compute weights, fp32 master weights and
AdamW moments, device-side global-norm clipping, deferred telemetry.

Counterpart of the reference's ``CudaTrainer`` (scirust-sciagent/src/cuda_model.rs:1239-2225:
``train_step_batch_deferred`` :1393-1523, ``global_grad_sumsq`` + ``adamw_step_with_norm``
:1440-1518, deferred diagnostics :1525-1529). Differences by design: the whole model is one flat
buffer, so the gradient norm is two launches and the optimizer one launch (the reference issues
2 + 1 launches per tensor); the step never synchronises with the host unless the caller reads the
loss; data-parallel gradient reduction is a pluggable ``grad_reducer``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from .schedule import ConstantSchedule, WarmupCosineSchedule


@dataclass
class TrainerConfig:
    lr: float = 3e-4
    min_lr: float = 3e-5
    warmup_steps: int = 0
    total_steps: int = 0          # 0 = constant learning rate
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    telemetry_interval: int = 0   # 0 = never read the loss back unless asked
    optimizer: str = "adamw"
    status_interval: int = 1      # multi-GPU runs: look at the kernels' status word every N steps (0 = never)
    activation_recompute: bool = False   # keep one activation per layer, re-run each block's forward in backward


class Trainer:
    """``train_step(tokens)`` takes ``[B, S+1]`` int64 token ids (host, ideally pinned, or device) and
    returns the loss as a device scalar. ``grad_reducer(flat_grad) -> scale`` may reduce the flat
    gradient across data-parallel ranks and returns the factor still to be applied (1/world)."""

    def __init__(self, model, cfg: TrainerConfig | None = None, grad_reducer=None):
        self.model = model
        self.cfg = cfg or TrainerConfig()
        c = self.cfg
        self.schedule = (WarmupCosineSchedule(c.lr, c.min_lr, c.warmup_steps, c.total_steps)
                         if c.total_steps > 0 else ConstantSchedule(c.lr))
        flat = model.flat
        self.master = flat.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.grad_sumsq = torch.zeros(1, dtype=torch.float32, device=flat.device)
        self.step = 0
        self.grad_reducer = grad_reducer
        if c.activation_recompute:
            if not hasattr(model, "activation_recompute"):
                raise ValueError("this model has no activation-recompute path")
            model.activation_recompute = True
        self.last_loss = None
        self._dev_tokens = None
        # Kernels that wait on other ranks record a time-out in a device status word and skip their work. With
        # a reducer or a tensor-parallel model attached the word is examined (without stalling the stream, one
        # step late at most) so that a partial reduction surfaces as CollectiveTimeout instead of diverging replicas.
        self._status = None
        if flat.is_cuda and c.status_interval > 0 and (grad_reducer is not None or hasattr(model, "finish_grads")):
            from ..ops import _lib
            self._status = _lib.DeferredStatus(flat.device)

    # -- data ------------------------------------------------------------------------------
    def _to_device(self, tokens):
        dev = self.model.flat.device
        if tokens.device == dev:
            return tokens
        if self._dev_tokens is None or self._dev_tokens.shape != tokens.shape:
            self._dev_tokens = torch.empty(tokens.shape, dtype=tokens.dtype, device=dev)
        self._dev_tokens.copy_(tokens, non_blocking=True)
        return self._dev_tokens

    # -- one optimisation step ---------------------------------------------------------------
    def train_step(self, tokens):
        model, c = self.model, self.cfg
        tok = self._to_device(tokens)
        inp = tok[:, :-1].contiguous()
        tgt = tok[:, 1:].contiguous()
        model.zero_grad_flags()
        loss = model(inp, tgt)
        loss.backward()
        grad = model.flat_grad
        grad_scale = 1.0
        if hasattr(model, "finish_grads"):
            # tensor-parallel shard: sum replicated parameters' gradients, learn the remaining scale
            grad_scale = model.finish_grads()
        if self.grad_reducer is not None:
            out = self.grad_reducer(grad)
            if isinstance(out, tuple):
                grad, g2 = out
            else:
                g2 = out
            grad_scale *= g2
        if hasattr(model, "global_grad_sumsq"):
            model.global_grad_sumsq(self.grad_sumsq, grad_scale)
        else:
            ops.sumsq(grad, out=self.grad_sumsq)
        self.step += 1
        lr = self.schedule.lr_at(self.step - 1)
        ops.optim_step(self.master, self.m, self.v, grad, model.flat, lr=lr, beta1=c.beta1, beta2=c.beta2,
                       eps=c.eps, weight_decay=c.weight_decay, step=self.step, decay_end=model.decay_end,
                       grad_sumsq=self.grad_sumsq, max_grad_norm=c.max_grad_norm, grad_scale=grad_scale,
                       mode=c.optimizer)
        self.last_loss = loss.detach()
        if self._status is not None and self.step % c.status_interval == 0:
            self._status.poll()
        return self.last_loss

    def train_step_accumulated(self, micro_batches):
        """One optimizer step over several micro-batches (gradient accumulation): every micro-batch runs forward and
        backward into the SAME flat gradient (the first write overwrites, the rest accumulate), the sum is scaled by
        ``1 / n`` inside the optimizer kernel, so activations are only ever held for one micro-batch. Returns the mean of
        the micro-batch losses (device scalar). Equals one step on the concatenated batch up to summation order."""
        model, c = self.model, self.cfg
        micro_batches = list(micro_batches)
        if not micro_batches:
            raise ValueError("train_step_accumulated needs at least one micro-batch")
        if hasattr(model, "finish_grads") or self.grad_reducer is not None:
            raise ValueError("gradient accumulation is implemented for the single-process trainer")
        model.zero_grad_flags()
        total = None
        for tokens in micro_batches:
            tok = self._to_device(tokens)
            loss = model(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        scale = 1.0 / len(micro_batches)
        grad = model.flat_grad
        ops.sumsq(grad, out=self.grad_sumsq)                             # of the SUM; the optimizer applies scale^2 itself
        self.step += 1
        ops.optim_step(self.master, self.m, self.v, grad, model.flat, lr=self.schedule.lr_at(self.step - 1), beta1=c.beta1,
                       beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay, step=self.step, decay_end=model.decay_end,
                       grad_sumsq=self.grad_sumsq, max_grad_norm=c.max_grad_norm, grad_scale=scale, mode=c.optimizer)
        self.grad_sumsq.mul_(scale * scale)                              # what grad_norm() reports: the averaged gradient
        self.last_loss = total * scale
        return self.last_loss

    def check_status(self) -> None:
        """Synchronising check of the device status word (checkpoint and telemetry points call it)."""
        if self._status is not None:
            self._status.flush()

    def grad_norm(self) -> float:
        return float(self.grad_sumsq.sqrt().item())

    # -- state -------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.step, "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd: dict) -> None:
        self.step = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.model.flat.copy_(self.master.to(torch.bfloat16))

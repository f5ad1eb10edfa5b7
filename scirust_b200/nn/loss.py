"""Losses (scirust-core/src/nn/loss/{cross_entropy,mse,nll,poisson,pinn}.rs, nn/audio.rs CTC).

``CrossEntropyLoss`` takes logits and a one-hot (or soft) target matrix, shifts by the row maximum,
and averages over the batch; ``forward_with_indices`` takes class ids; on CUDA bf16 logits the
class-id path runs the fused softmax-cross-entropy kernel (loss and gradient in one pass)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from ..autodiff.tape import Var


def _u(x):
    return x.t if isinstance(x, Var) else x


def _w(y, like):
    return like._new(y) if isinstance(like, Var) else y


class _FusedCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows = logits.shape[0]
        loss_rows, d = ops.ce_fwd_bwd(logits.contiguous(), targets, 1.0 / rows, in_place=False)
        ctx.save_for_backward(d)
        return loss_rows.sum() / rows

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None


class CrossEntropyLoss:
    def forward(self, logits, target_onehot):
        lg, tg = _u(logits), _u(target_onehot)
        if lg.shape != tg.shape:
            raise ValueError(f"CrossEntropyLoss: logits {tuple(lg.shape)} vs target {tuple(tg.shape)}")
        shifted = lg - lg.detach().amax(1, keepdim=True)
        lsm = shifted - torch.log(torch.exp(shifted).sum(1, keepdim=True))
        return _w(((lsm * tg).sum() * (-1.0 / lg.shape[0])).reshape(1, 1), logits)

    __call__ = forward

    def forward_with_indices(self, logits, indices):
        lg = _u(logits)
        idx = torch.as_tensor(indices, dtype=torch.long, device=lg.device).reshape(-1)
        if lg.is_cuda and lg.dtype == torch.bfloat16 and lg.shape[1] % 8 == 0:
            return _w(_FusedCE.apply(lg, idx).reshape(1, 1), logits)
        return _w(F.cross_entropy(lg.float(), idx).reshape(1, 1), logits)


class MSELoss:
    def forward(self, pred, target):
        p, t = _u(pred), _u(target)
        return _w(((p - t) ** 2).mean().reshape(1, 1), pred)
    __call__ = forward


class NLLLoss:
    """Negative log-likelihood over log-probabilities and class ids."""

    def forward(self, log_probs, indices):
        lp = _u(log_probs)
        idx = torch.as_tensor(indices, dtype=torch.long, device=lp.device).reshape(-1)
        return _w(F.nll_loss(lp, idx).reshape(1, 1), log_probs)
    __call__ = forward


class PoissonNLLLoss:
    def __init__(self, log_input: bool = True, eps: float = 1e-8):
        self.log_input, self.eps = log_input, eps

    def forward(self, pred, target):
        p, t = _u(pred), _u(target)
        loss = torch.exp(p) - t * p if self.log_input else p - t * torch.log(p + self.eps)
        return _w(loss.mean().reshape(1, 1), pred)
    __call__ = forward


class PINNLoss:
    """data loss + weight * mean squared PDE residual."""

    def __init__(self, residual_weight: float = 1.0):
        self.residual_weight = residual_weight

    def forward(self, pred, target, residual):
        p, t, r = _u(pred), _u(target), _u(residual)
        return _w((((p - t) ** 2).mean() + self.residual_weight * (r ** 2).mean()).reshape(1, 1), pred)
    __call__ = forward


class CTCLoss:
    def __init__(self, blank: int = 0):
        self.blank = blank

    def forward(self, log_probs, targets, input_lengths, target_lengths):
        """log_probs (T, B, C) log-softmax outputs."""
        return F.ctc_loss(_u(log_probs), targets, input_lengths, target_lengths, blank=self.blank)
    __call__ = forward

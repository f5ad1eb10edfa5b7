"""Audio front end and CTC.

``ctc_loss``: exact connectionist-temporal-classification negative log-likelihood by the log-space forward
recursion over the blank-extended label ``[b, c1, b, c2, ..., b]``. The recursion is vectorised over the extended
label axis AND over a batch of padded sequences (one ``logsumexp`` of three shifted rows per time step), and it is
written in differentiable tensor operations, so the exact gradient comes from autograd on any device. The blank is
the LAST vocabulary index by default, as in the reference. Infeasible pairs (too few frames for the labels and
their repeats) give ``+inf`` loss and a zero gradient.

``AudioEncoder``: two 3x3 stride-2 SAME convolutions with ReLU (a 4x time / frequency down-sampler) on the
flattened ``(B, C*H*W)`` image convention of ``scirust_b200.nn.modules``; state-dict keys ``conv1.weight`` ...
Reference counterpart: scirust-core/src/nn/audio.rs:11-330 (``CTCLoss`` forward-backward, ``AudioEncoder``).
"""
from __future__ import annotations

import math

import torch

from .modules import Conv2d, Module, Padding
from .rng import PcgEngine


def ctc_loss(logits, targets, input_lengths=None, target_lengths=None, blank: int | None = None, reduction="none"):
    """``logits [T, V]`` with ``targets [S]``, or batched ``[B, T, V]`` with padded ``targets [B, S]`` and lengths."""
    single = logits.dim() == 2
    if single:
        logits = logits[None]
        targets = torch.as_tensor(targets, dtype=torch.int64, device=logits.device).reshape(1, -1)
    B, T, V = logits.shape
    blank = V - 1 if blank is None else blank
    targets = torch.as_tensor(targets, dtype=torch.int64, device=logits.device).clamp(0, V - 1)
    S = targets.shape[1]
    in_len = torch.full((B,), T, dtype=torch.int64, device=logits.device) if input_lengths is None else \
        torch.as_tensor(input_lengths, dtype=torch.int64, device=logits.device)
    tg_len = torch.full((B,), S, dtype=torch.int64, device=logits.device) if target_lengths is None else \
        torch.as_tensor(target_lengths, dtype=torch.int64, device=logits.device)
    logp = torch.log_softmax(logits.float(), -1)
    U = 2 * S + 1
    ext = torch.full((B, U), blank, dtype=torch.int64, device=logits.device)
    ext[:, 1::2] = targets
    # a skip s-2 -> s is allowed into a label that differs from the label two back
    skip = torch.zeros(B, U, dtype=torch.bool, device=logits.device)
    if U > 2:
        skip[:, 2:] = (ext[:, 2:] != blank) & (ext[:, 2:] != ext[:, :-2])
    neg = torch.full((B, 1), -math.inf, device=logits.device)
    emit = logp.gather(2, ext[:, None, :].expand(B, T, U))                    # [B, T, U]
    alpha = torch.full((B, U), -math.inf, device=logits.device)
    alpha[:, 0] = emit[:, 0, 0]
    if U > 1:
        alpha[:, 1] = emit[:, 0, 1]
    valid_u = torch.arange(U, device=logits.device)[None, :] < (2 * tg_len[:, None] + 1)
    alpha = torch.where(valid_u, alpha, torch.full_like(alpha, -math.inf))
    for t in range(1, T):
        a1 = torch.cat([neg, alpha[:, :-1]], 1)
        a2 = torch.cat([neg, neg, alpha[:, :-2]], 1) if U > 2 else torch.full_like(alpha, -math.inf)
        a2 = torch.where(skip, a2, torch.full_like(a2, -math.inf))
        stacked = torch.stack([alpha, a1, a2], 0)
        m = stacked.max(0).values
        safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        new = safe + torch.log(torch.exp(stacked - safe).sum(0)) + emit[:, t]
        new = torch.where(torch.isinf(m) | ~valid_u, torch.full_like(new, -math.inf), new)
        alpha = torch.where((t < in_len)[:, None], new, alpha)               # frozen past each sequence's end
    last = 2 * tg_len
    end1 = alpha.gather(1, last[:, None]).squeeze(1)
    end2 = torch.where(tg_len > 0, alpha.gather(1, (last - 1).clamp_min(0)[:, None]).squeeze(1),
                       torch.full_like(end1, -math.inf))
    m = torch.maximum(end1, end2)
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    ll = safe + torch.log(torch.exp(end1 - safe) + torch.exp(end2 - safe))
    # min frames = labels + adjacent repeats
    repeats = ((targets[:, 1:] == targets[:, :-1]) & (torch.arange(1, S, device=logits.device)[None] < tg_len[:, None])).sum(1) \
        if S > 1 else torch.zeros(B, dtype=torch.int64, device=logits.device)
    feasible = (in_len > 0) & (in_len >= tg_len + repeats) & ~torch.isinf(m)
    loss = torch.where(feasible, -ll, torch.full_like(ll, math.inf).detach())
    if single:
        return loss[0]
    if reduction == "mean":
        return (loss / tg_len.clamp_min(1)).mean()
    if reduction == "sum":
        return loss.sum()
    return loss


class CTCLossLastBlank:
    """CTC with the blank at ``vocab - 1`` on one ``(T, vocab)`` logit matrix (the reference's calling form)."""

    def forward(self, logits, targets):
        return ctc_loss(logits, targets)
    __call__ = forward


class AudioEncoder(Module):
    def __init__(self, in_channels: int, hidden_channels: int, out_channels: int, in_h: int = 0, in_w: int = 0,
                 rng: PcgEngine | None = None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.conv1 = Conv2d(in_channels, hidden_channels, 3, 2, Padding.SAME, in_h, in_w, rng)
        h2, w2 = self.conv1.out_hw(in_h, in_w) if in_h and in_w else (0, 0)
        self.conv2 = Conv2d(hidden_channels, out_channels, 3, 2, Padding.SAME, h2, w2, rng)

    def out_hw(self, h=None, w=None):
        return self.conv2.out_hw(*self.conv1.out_hw(h, w))

    def forward(self, x, h: int | None = None, w: int | None = None):
        h, w = h or self.conv1.in_h, w or self.conv1.in_w
        y = torch.relu(self.conv1(x, h, w))
        return torch.relu(self.conv2(y, *self.conv1.out_hw(h, w)))

    def state_dict_ref(self):
        sd = {"conv1.weight": self.conv1.weight.detach().float().cpu(), "conv2.weight": self.conv2.weight.detach().float().cpu()}
        for n, c in (("conv1", self.conv1), ("conv2", self.conv2)):
            if c.bias is not None:
                sd[f"{n}.bias"] = c.bias.detach().float().cpu()
        return sd

    def load_state_dict_ref(self, sd):
        for n, c in (("conv1", self.conv1), ("conv2", self.conv2)):
            if f"{n}.weight" not in sd:
                raise KeyError(f"missing key: {n}.weight")
            w = torch.as_tensor(sd[f"{n}.weight"])
            if tuple(w.shape) != tuple(c.weight.shape):
                raise ValueError(f"{n}.weight shape mismatch: expected {tuple(c.weight.shape)}, got {tuple(w.shape)}")
            with torch.no_grad():
                c.weight.copy_(w)
                if c.bias is not None:
                    if f"{n}.bias" not in sd:
                        raise KeyError(f"missing key: {n}.bias")
                    c.bias.copy_(torch.as_tensor(sd[f"{n}.bias"]).reshape(1, -1))

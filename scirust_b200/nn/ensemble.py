"""Deep ensembles (Lakshminarayanan et al., 2017): several small ReLU MLPs trained from different seeds; the
mean is the point prediction and the spread across members is an epistemic-uncertainty signal (small where the
data pins the function down, large away from it).

All members train together: their weights are stacked on a leading member axis and every step is two batched
matrix products and one Adam update over the stack, so K members cost one kernel sequence instead of K (and the
stack lives on whatever device the data is on). Member ``m`` draws its initial weights from ``PcgEngine(base_seed
+ m)`` (uniform ``+-1/sqrt(fan_in)``, zero bias) and the members never interact, so the result is the same as
training them one after another and is reproducible bit for bit on a given device.
Reference counterpart: scirust-core/src/nn/ensemble.rs:23-115 (1-D regression, sum-of-squares loss, Adam).
"""
from __future__ import annotations

import math

import torch

from .rng import PcgEngine


class DeepEnsemble:
    def __init__(self, w1, b1, w2, b2):
        self.w1, self.b1, self.w2, self.b2 = w1, b1, w2, b2           # [K,in,H] [K,1,H] [K,H,out] [K,1,out]

    def __len__(self):
        return self.w1.shape[0]

    @staticmethod
    def _init(n_members, in_f, hidden, out_f, base_seed, device):
        w1, w2 = [], []
        for m in range(n_members):
            rng = PcgEngine(base_seed + m)
            w1.append(rng.fill_uniform_signed((in_f, hidden), 1.0 / math.sqrt(in_f)))
            w2.append(rng.fill_uniform_signed((hidden, out_f), 1.0 / math.sqrt(hidden)))
        return (torch.stack(w1).to(device), torch.zeros(n_members, 1, hidden, device=device),
                torch.stack(w2).to(device), torch.zeros(n_members, 1, out_f, device=device))

    @staticmethod
    def train(xs, ys, n_members: int, hidden: int, steps: int, lr: float, base_seed: int,
              betas=(0.9, 0.999), eps: float = 1e-8) -> "DeepEnsemble":
        x = torch.as_tensor(xs, dtype=torch.float32)
        y = torch.as_tensor(ys, dtype=torch.float32)
        if x.dim() == 1:
            x = x[:, None]
        if y.dim() == 1:
            y = y[:, None]
        if x.shape[0] != y.shape[0]:
            raise ValueError("DeepEnsemble: xs/ys length mismatch")
        params = list(DeepEnsemble._init(n_members, x.shape[1], hidden, y.shape[1], base_seed, x.device))
        m_state = [torch.zeros_like(p) for p in params]
        v_state = [torch.zeros_like(p) for p in params]
        xb = x[None].expand(n_members, -1, -1)
        for t in range(1, steps + 1):
            w1, b1, w2, b2 = params
            pre = torch.baddbmm(b1, xb, w1)                       # [K, N, H]
            h = pre.clamp_min(0)
            out = torch.baddbmm(b2, h, w2)
            d_out = 2.0 * (out - y[None])                         # loss = sum of squares per member
            g_w2 = h.transpose(1, 2) @ d_out
            g_b2 = d_out.sum(1, keepdim=True)
            d_h = (d_out @ w2.transpose(1, 2)) * (pre > 0)
            g_w1 = xb.transpose(1, 2) @ d_h
            g_b1 = d_h.sum(1, keepdim=True)
            c1, c2 = 1.0 - betas[0] ** t, 1.0 - betas[1] ** t
            for p, g, m, v in zip(params, (g_w1, g_b1, g_w2, g_b2), m_state, v_state):
                m.mul_(betas[0]).add_(g, alpha=1.0 - betas[0])
                v.mul_(betas[1]).addcmul_(g, g, value=1.0 - betas[1])
                p.sub_(lr * (m / c1) / ((v / c2).sqrt() + eps))
        return DeepEnsemble(*params)

    def member_predictions(self, x) -> torch.Tensor:
        """[K, N, out] predictions of every member."""
        x = torch.as_tensor(x, dtype=torch.float32, device=self.w1.device)
        if x.dim() == 0:
            x = x.reshape(1, 1)
        elif x.dim() == 1:
            x = x[:, None]
        xb = x[None].expand(len(self), -1, -1)
        return torch.baddbmm(self.b2, torch.baddbmm(self.b1, xb, self.w1).clamp_min(0), self.w2)

    def predict(self, x):
        """(mean, standard deviation across members, population form); scalars for a scalar input."""
        p = self.member_predictions(x)
        mean = p.mean(0)
        std = ((p - mean[None]) ** 2).mean(0).sqrt()
        if not torch.is_tensor(x) and not hasattr(x, "__len__"):
            return float(mean.reshape(-1)[0]), float(std.reshape(-1)[0])
        return mean.squeeze(-1), std.squeeze(-1)

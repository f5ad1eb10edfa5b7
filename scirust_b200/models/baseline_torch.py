"""Library baseline of the same GQA decoder: every operator is a stock PyTorch call (cuBLAS GEMMs,
``scaled_dot_product_attention``, ``F.rms_norm``, ``F.cross_entropy``, fused ``torch.optim.AdamW``)
and the data-parallel reduction is NCCL through ``DistributedDataParallel``. None of this
framework's kernels run on this path; it exists to be timed against them on the same GPU
(``bench.py --impl baseline``) and to cross-check losses.

Same arithmetic contract as the native trainer: bf16 weights and activations, fp32 master weights and
AdamW moments, global-norm clipping, tied embedding / LM head, RoPE on interleaved pairs, SwiGLU.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .sciagent import SciAgentConfig

BF = torch.bfloat16


class _Block(nn.Module):
    def __init__(self, cfg: SciAgentConfig):
        super().__init__()
        d, dh = cfg.d_model, cfg.head_dim
        self.cfg = cfg
        self.rms_attn = nn.Parameter(torch.ones(d, dtype=BF))
        self.rms_ffn = nn.Parameter(torch.ones(d, dtype=BF))
        self.wqkv = nn.Parameter(torch.empty(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * dh, dtype=BF))
        self.wo = nn.Parameter(torch.empty(cfg.n_heads * dh, d, dtype=BF))
        self.wgu = nn.Parameter(torch.empty(d, 2 * cfg.d_ff, dtype=BF))
        self.wd = nn.Parameter(torch.empty(cfg.d_ff, d, dtype=BF))

    def forward(self, x, cos, sin):
        cfg = self.cfg
        B, S, d = x.shape
        H, Hkv, dh = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        h = F.rms_norm(x, (d,), self.rms_attn, cfg.eps)
        qkv = h @ self.wqkv
        q, k, v = qkv.split([H * dh, Hkv * dh, Hkv * dh], -1)
        q = _rope(q.view(B, S, H, dh), cos, sin).transpose(1, 2)
        k = _rope(k.view(B, S, Hkv, dh), cos, sin).transpose(1, 2)
        v = v.view(B, S, Hkv, dh).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + a.transpose(1, 2).reshape(B, S, H * dh) @ self.wo
        h = F.rms_norm(x, (d,), self.rms_ffn, cfg.eps)
        g, u = (h @ self.wgu).chunk(2, -1)
        return x + (F.silu(g) * u) @ self.wd


def _rope(x, cos, sin):                     # x: [B, S, H, dh]; interleaved (even, odd) pairs
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).flatten(-2)


class TorchLibraryDecoder(nn.Module):
    def __init__(self, cfg: SciAgentConfig, device="cuda", seed: int = 0, init_std: float = 0.02):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=BF))
        self.blocks = nn.ModuleList([_Block(cfg) for _ in range(cfg.n_layers)])
        self.rms_final = nn.Parameter(torch.ones(cfg.d_model, dtype=BF))
        self.to(device)
        g = torch.Generator(device=device).manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() == 2:
                    p.copy_(torch.randn(p.shape, generator=g, device=device) * init_std)
        half = cfg.head_dim // 2
        inv = torch.pow(cfg.rope_theta, -torch.arange(half, device=device, dtype=torch.float32) * 2 / cfg.head_dim)
        ang = torch.arange(cfg.max_seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos().to(BF), persistent=False)
        self.register_buffer("sin", ang.sin().to(BF), persistent=False)

    def forward(self, tokens, targets):
        S = tokens.shape[1]
        x = F.embedding(tokens, self.embed)
        cos, sin = self.cos[:S], self.sin[:S]
        for b in self.blocks:
            x = b(x, cos, sin)
        x = F.rms_norm(x, (self.cfg.d_model,), self.rms_final, self.cfg.eps)
        logits = x @ self.embed.t()
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))


class TorchLibraryTrainer:
    """fp32 masters + fused AdamW + global-norm clip around ``TorchLibraryDecoder``."""

    def __init__(self, model: TorchLibraryDecoder, lr=3e-4, weight_decay=0.1, max_grad_norm=1.0, ddp=None):
        self.model, self.wrapped = model, (ddp if ddp is not None else model)
        self.params = [p for p in model.parameters()]
        self.masters = [p.detach().float().clone().requires_grad_(True) for p in self.params]
        decay = [m for m, p in zip(self.masters, self.params) if p.dim() == 2]
        no_decay = [m for m, p in zip(self.masters, self.params) if p.dim() != 2]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": weight_decay},
                                      {"params": no_decay, "weight_decay": 0.0}], lr=lr, betas=(0.9, 0.95),
                                     eps=1e-8, fused=True)
        self.max_grad_norm = max_grad_norm

    def train_step(self, batch: torch.Tensor):
        dev = self.params[0].device
        batch = batch.to(dev, non_blocking=True)
        tokens, targets = batch[:, :-1], batch[:, 1:]
        loss = self.wrapped(tokens, targets)
        loss.backward()
        for m, p in zip(self.masters, self.params):
            m.grad = p.grad.float()
            p.grad = None
        torch.nn.utils.clip_grad_norm_(self.masters, self.max_grad_norm, foreach=True)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        with torch.no_grad():
            torch._foreach_copy_(self.params, self.masters)
        return loss.detach()

"""Transformer building blocks of the core library (scirust-core/src/nn/transformer/{attention,
flash_attention,moe,mini_llm}.rs): multi-head attention with an ``infer_step`` KV cache, pre-norm
encoder/decoder blocks, a blockwise (online-softmax) attention reference, top-k gated
mixture-of-experts and a character-level MiniLLM. Inputs are ``(B*S, d)`` matrices."""
from __future__ import annotations

import math

import torch
import torch.nn as tnn
import torch.nn.functional as F

from .modules import LayerNorm, Linear, Module
from .rng import PcgEngine


def flash_attention_blockwise(q, k, v, block: int = 64, causal: bool = False, scale: float | None = None):
    """Tiled attention with online softmax over KV blocks for one head: numerically the dense result
    without materialising the score matrix (nn/transformer/flash_attention.rs:25-531). Returns
    (output, row max, row sum) - the statistics a blockwise backward needs."""
    n, d = q.shape
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    o = torch.zeros_like(q, dtype=torch.float32)
    m = torch.full((n,), float("-inf"))
    l = torch.zeros(n)
    qf = q.float()
    for j0 in range(0, k.shape[0], block):
        kj, vj = k[j0:j0 + block].float(), v[j0:j0 + block].float()
        s = qf @ kj.t() * scale
        if causal:
            cols = torch.arange(j0, j0 + kj.shape[0])[None, :]
            s = s.masked_fill(cols > torch.arange(n)[:, None], float("-inf"))
        m_new = torch.maximum(m, s.amax(1))
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        p = torch.exp(s - safe[:, None])
        alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - safe))
        l = l * alpha + p.sum(1)
        o = o * alpha[:, None] + p @ vj
        m = m_new
    return o / l[:, None], m, l


class MultiHeadAttention(Module):
    def __init__(self, d_model: int, n_heads: int, rng: PcgEngine | None = None, causal: bool = False):
        super().__init__()
        rng = rng or PcgEngine(0)
        if d_model % n_heads:
            raise ValueError("d_model must divide by n_heads")
        self.d_model, self.n_heads, self.dh, self.causal = d_model, n_heads, d_model // n_heads, causal
        self.w_q, self.w_k = Linear(d_model, d_model, rng=rng), Linear(d_model, d_model, rng=rng)
        self.w_v, self.w_o = Linear(d_model, d_model, rng=rng), Linear(d_model, d_model, rng=rng)
        self._cache = None

    def _split(self, x, B, S):
        return x.reshape(B, S, self.n_heads, self.dh).transpose(1, 2)

    def forward(self, x, seq_len: int | None = None, context=None):
        S = seq_len or x.shape[0]
        B = x.shape[0] // S
        src = x if context is None else context
        Sk = src.shape[0] // B
        q, k, v = self._split(self.w_q(x), B, S), self._split(self.w_k(src), B, Sk), self._split(self.w_v(src), B, Sk)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=self.causal and context is None)
        return self.w_o(o.transpose(1, 2).reshape(B * S, self.d_model))

    def reset_cache(self):
        self._cache = None

    def infer_step(self, x_t):
        """One new position per sequence, attending over everything cached so far."""
        B = x_t.shape[0]
        q = self.w_q(x_t).reshape(B, self.n_heads, 1, self.dh)
        k = self.w_k(x_t).reshape(B, self.n_heads, 1, self.dh)
        v = self.w_v(x_t).reshape(B, self.n_heads, 1, self.dh)
        if self._cache is not None:
            k, v = torch.cat([self._cache[0], k], 2), torch.cat([self._cache[1], v], 2)
        self._cache = (k.detach(), v.detach())
        o = F.scaled_dot_product_attention(q, k, v)
        return self.w_o(o.reshape(B, self.d_model))


class FeedForward(Module):
    def __init__(self, d_model, d_ff, rng=None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.fc1, self.fc2 = Linear(d_model, d_ff, rng=rng), Linear(d_ff, d_model, rng=rng)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


class TransformerBlock(Module):
    """Pre-norm block: x + MHA(LN(x)); x + FFN(LN(x))."""

    def __init__(self, d_model, n_heads, d_ff, rng=None, causal=False):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.ln1, self.ln2 = LayerNorm(d_model), LayerNorm(d_model)
        self.attn = MultiHeadAttention(d_model, n_heads, rng, causal)
        self.ffn = FeedForward(d_model, d_ff, rng)

    def forward(self, x, seq_len=None):
        x = x + self.attn(self.ln1(x), seq_len)
        return x + self.ffn(self.ln2(x))


class TransformerEncoder(Module):
    def __init__(self, n_layers, d_model, n_heads, d_ff, rng=None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.blocks = tnn.ModuleList([TransformerBlock(d_model, n_heads, d_ff, rng) for _ in range(n_layers)])
        self.ln = LayerNorm(d_model)

    def forward(self, x, seq_len=None):
        for b in self.blocks:
            x = b(x, seq_len)
        return self.ln(x)


class TransformerDecoder(TransformerEncoder):
    def __init__(self, n_layers, d_model, n_heads, d_ff, rng=None):
        Module.__init__(self)
        rng = rng or PcgEngine(0)
        self.blocks = tnn.ModuleList([TransformerBlock(d_model, n_heads, d_ff, rng, causal=True) for _ in range(n_layers)])
        self.ln = LayerNorm(d_model)


class MoE(Module):
    """Top-k gated mixture of experts: softmax gate, keep the k largest, renormalise, weighted sum
    of the selected experts' outputs (nn/transformer/moe.rs:10-201)."""

    def __init__(self, d_model, d_ff, n_experts, top_k=2, rng=None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.top_k = top_k
        self.gate = Linear(d_model, n_experts, rng=rng)
        self.experts = tnn.ModuleList([FeedForward(d_model, d_ff, rng) for _ in range(n_experts)])

    def forward(self, x):
        probs = torch.softmax(self.gate(x), -1)
        w, idx = probs.topk(self.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(x)
        for e, expert in enumerate(self.experts):
            mask = idx == e
            rows = mask.any(-1)
            if rows.any():
                out[rows] = out[rows] + expert(x[rows]) * (w * mask)[rows].sum(-1, keepdim=True)
        return out

    def load_balance_loss(self, x):
        probs = torch.softmax(self.gate(x), -1)
        frac = F.one_hot(probs.argmax(-1), probs.shape[-1]).float().mean(0)
        return probs.shape[-1] * (frac * probs.mean(0)).sum()


class MiniLLM(Module):
    """Small character-level decoder LM (embedding + learned positions + causal blocks + head)."""

    def __init__(self, vocab, d_model=64, n_heads=4, n_layers=2, d_ff=128, max_len=128, seed=0):
        super().__init__()
        rng = PcgEngine(seed)
        self.tok = tnn.Parameter(rng.fill_normal((vocab, d_model), 0.0, 0.02))
        self.pos = tnn.Parameter(rng.fill_normal((max_len, d_model), 0.0, 0.02))
        self.dec = TransformerDecoder(n_layers, d_model, n_heads, d_ff, rng)
        self.head = Linear(d_model, vocab, rng=rng)

    def forward(self, tokens):
        B, S = tokens.shape
        x = self.tok[tokens.reshape(-1)] + self.pos[:S].repeat(B, 1)
        return self.head(self.dec(x, S))

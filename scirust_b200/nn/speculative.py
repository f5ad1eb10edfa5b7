"""Multi-token drafting for decoder LMs with exact greedy output: Medusa heads and the EAGLE feature head.

Both draft a block of tokens from ONE base forward and verify it with ONE more forward over ``sequence + block``:
the longest prefix that matches the base model's own arg-max is committed, the first mismatch is replaced by the
base model's token, and a fully accepted block earns a bonus token. Whatever the heads propose, the result equals
``generate_greedy``; good heads only reduce the number of base forwards.

* ``MedusaHeads``: ``num_heads`` linear heads over the last hidden state; head ``j`` predicts the token ``j + 2``
  positions ahead. All heads are one stacked weight ``[heads, d, vocab]`` so a proposal is a single batched product.
* ``EagleHead``: a linear map ``(feature_t, embedding(token_{t+1})) -> feature_{t+1}``; chained ``k - 1`` times and
  decoded through the frozen LM head.
* Training freezes the base model: hidden states are computed once, then the heads are fitted with Adam.

Works with any model exposing ``hidden(tokens) -> [B, L, d]`` and a tied head ``embed.weight`` (``zoo.NdDecoderLM``).
Draft / target speculative decoding with two models is ``zoo.speculative_generate``.
Reference counterpart: scirust-core/src/nn/nd_decoder.rs:250-700 (``generate_greedy``, ``MedusaHeads``,
``generate_medusa``, ``EagleHead``, ``generate_eagle``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .rng import PcgEngine


def _logits(model, h):
    return h @ model.embed.weight.t()


@torch.no_grad()
def generate_greedy(model, prompt, n_new: int):
    seq = list(prompt)
    for _ in range(n_new):
        t = torch.tensor([seq], device=model.embed.weight.device)
        seq.append(int(_logits(model, model.hidden(t)[0, -1]).argmax()))
    return seq[len(prompt):]


def _verify_and_commit(model, seq, block, prompt_len, n_new):
    """One verification forward over seq + block; returns the extended sequence."""
    t = torch.tensor([seq + block], device=model.embed.weight.device)
    preds = _logits(model, model.hidden(t)[0]).argmax(-1).tolist()
    base = len(seq) - 1
    accepted = 0
    for i, b in enumerate(block):
        if preds[base + i] == b:
            seq.append(b)
            accepted += 1
        else:
            seq.append(preds[base + i])
            break
    if accepted == len(block) and len(seq) - prompt_len < n_new:
        seq.append(preds[base + len(block)])
    return seq


class MedusaHeads(torch.nn.Module):
    def __init__(self, num_heads: int, d_model: int, vocab: int, rng: PcgEngine | None = None):
        super().__init__()
        if num_heads < 1:
            raise ValueError("Medusa needs at least one head")
        rng = rng or PcgEngine(0)
        w = torch.stack([rng.fill_uniform_signed((d_model, vocab), 1.0 / math.sqrt(d_model)) for _ in range(num_heads)])
        self.weight = torch.nn.Parameter(w)                              # [heads, d, vocab]
        self.bias = torch.nn.Parameter(torch.zeros(num_heads, 1, vocab))
        self.d_model = d_model

    def num_heads(self) -> int:
        return self.weight.shape[0]

    def head_logits(self, hidden):
        """hidden [L, d] -> [heads, L, vocab]."""
        return torch.baddbmm(self.bias, hidden[None].expand(self.num_heads(), -1, -1), self.weight)

    @torch.no_grad()
    def propose(self, hidden_last) -> list:
        if hidden_last.numel() != self.d_model:
            raise ValueError("Medusa: hidden width")
        return self.head_logits(hidden_last.reshape(1, -1))[:, 0].argmax(-1).tolist()

    def fit(self, model, seq, steps: int, lr: float):
        """Head j learns token j + 2 ahead of every position of ``seq`` (base model frozen)."""
        toks = torch.tensor([list(seq)], device=self.weight.device)
        with torch.no_grad():
            hidden = model.hidden(toks)[0].float()
        L = hidden.shape[0]
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        tgt = toks[0]
        for _ in range(steps):
            logits = self.head_logits(hidden)
            loss = None
            for j in range(self.num_heads()):
                o = j + 2
                if L <= o:
                    continue
                ce = F.cross_entropy(logits[j, : L - o], tgt[o:])
                loss = ce if loss is None else loss + ce
            if loss is None:
                return
            opt.zero_grad()
            loss.backward()
            opt.step()


@torch.no_grad()
def generate_medusa(model, heads: MedusaHeads, prompt, n_new: int):
    """(new tokens, number of base forwards)."""
    if not len(prompt):
        raise ValueError("empty prompt")
    seq, forwards = list(prompt), 0
    while len(seq) - len(prompt) < n_new:
        remaining = n_new - (len(seq) - len(prompt))
        h = model.hidden(torch.tensor([seq], device=model.embed.weight.device))[0]
        forwards += 1
        block = [int(_logits(model, h[-1]).argmax())] + heads.propose(h[-1].float())
        seq = _verify_and_commit(model, seq, block[:remaining], len(prompt), n_new)
        forwards += 1
    return seq[len(prompt): len(prompt) + n_new], forwards


class EagleHead(torch.nn.Module):
    def __init__(self, d_model: int, rng: PcgEngine | None = None):
        super().__init__()
        rng = rng or PcgEngine(0)
        self.weight = torch.nn.Parameter(rng.fill_uniform_signed((2 * d_model, d_model), 1.0 / math.sqrt(2 * d_model)))
        self.bias = torch.nn.Parameter(torch.zeros(1, d_model))
        self.d_model = d_model

    def predict_feature(self, feature, embed):
        if feature.shape[-1] != self.d_model or embed.shape[-1] != self.d_model:
            raise ValueError("EAGLE: feature / embed width")
        return torch.cat([feature, embed], -1) @ self.weight + self.bias

    def fit(self, model, seq, steps: int, lr: float):
        if len(seq) < 2:
            return
        toks = torch.tensor([list(seq)], device=self.weight.device)
        with torch.no_grad():
            h = model.hidden(toks)[0].float()
            x = torch.cat([h[:-1], model.embed.weight[toks[0, 1:]].float()], 1)
            y = h[1:]
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        for _ in range(steps):
            loss = ((x @ self.weight + self.bias - y) ** 2).sum()
            opt.zero_grad()
            loss.backward()
            opt.step()


@torch.no_grad()
def generate_eagle(model, eagle: EagleHead, prompt, n_new: int, k: int):
    if k < 1:
        raise ValueError("k must be >= 1")
    if not len(prompt):
        raise ValueError("empty prompt")
    seq, forwards = list(prompt), 0
    while len(seq) - len(prompt) < n_new:
        remaining = n_new - (len(seq) - len(prompt))
        h = model.hidden(torch.tensor([seq], device=model.embed.weight.device))[0]
        forwards += 1
        feature = h[-1].float()
        tok = int(_logits(model, h[-1]).argmax())
        block = [tok]
        for _ in range(1, k):
            feature = eagle.predict_feature(feature[None], model.embed.weight[tok].float()[None])[0]
            tok = int(_logits(model, feature.to(h.dtype)).argmax())
            block.append(tok)
        seq = _verify_and_commit(model, seq, block[:remaining], len(prompt), n_new)
        forwards += 1
    return seq[len(prompt): len(prompt) + n_new], forwards

"""Text embeddings from the local character-level transformer: tokenise, run the decoder stack, mean-pool the hidden
states over the sequence (non-finite values skipped) and L2-normalise. ``embed_batch`` pads a whole batch to one
length and runs it as ONE forward pass with a masked mean, so many texts cost one kernel sequence; an empty string
maps to the zero vector. Reference counterpart: scirust-core/src/embed.rs:10-110 (``EmbeddingEngine`` over MiniLLM,
one text at a time).
"""
from __future__ import annotations

import torch

from .nn.transformer import MiniLLM


class CharTokenizer:
    """Sorted set of the characters seen in the vocabulary texts; unknown characters map to id 0."""

    def __init__(self, vocab_texts):
        chars = sorted({c for t in vocab_texts for c in t})
        self.itos = ["\0"] + chars
        self.stoi = {c: i for i, c in enumerate(self.itos)}

    @property
    def vocab_size(self) -> int:
        return len(self.itos)

    def encode(self, text: str):
        return [self.stoi.get(c, 0) for c in text]

    def decode(self, ids) -> str:
        return "".join(self.itos[i] for i in ids if 0 < i < len(self.itos))


class EmbeddingEngine:
    def __init__(self, vocab_texts, d_model: int = 128, n_heads: int = 4, n_layers: int = 2, d_ff: int = 256,
                 max_seq_len: int = 128, seed: int = 0, device="cpu"):
        self.tokenizer = CharTokenizer(vocab_texts)
        self.max_seq_len = max_seq_len
        self.llm = MiniLLM(self.tokenizer.vocab_size, d_model, n_heads, n_layers, d_ff, max_seq_len, seed).to(device)
        self.llm.eval()
        self._dim = d_model

    def dim(self) -> int:
        return self._dim

    @torch.no_grad()
    def _hidden(self, tokens: torch.Tensor) -> torch.Tensor:
        B, S = tokens.shape
        x = self.llm.tok[tokens.reshape(-1)] + self.llm.pos[:S].repeat(B, 1)
        return self.llm.dec(x, S).reshape(B, S, -1)

    def embed(self, text: str) -> torch.Tensor:
        return self.embed_batch([text])[0]

    @torch.no_grad()
    def embed_batch(self, texts) -> torch.Tensor:
        ids = [self.tokenizer.encode(t)[: self.max_seq_len] for t in texts]
        out = torch.zeros(len(ids), self._dim)
        lengths = sorted({len(i) for i in ids if i})
        dev = self.llm.tok.device
        # causal decoder: right padding does not change the states of the real positions, so one padded batch per
        # call is exact; texts are grouped only to bound the padding work
        if lengths:
            S = lengths[-1]
            rows = [k for k, i in enumerate(ids) if i]
            tok = torch.zeros(len(rows), S, dtype=torch.int64)
            mask = torch.zeros(len(rows), S)
            for r, k in enumerate(rows):
                tok[r, : len(ids[k])] = torch.tensor(ids[k])
                mask[r, : len(ids[k])] = 1.0
            h = self._hidden(tok.to(dev)).float().cpu()
            h = torch.where(torch.isfinite(h), h, torch.zeros_like(h))
            mean = (h * mask[:, :, None]).sum(1) / mask.sum(1, keepdim=True)
            out[rows] = mean / mean.norm(dim=1, keepdim=True).clamp_min(1e-12)
        return out

    @staticmethod
    def cosine_similarity(a, b) -> float:
        a, b = torch.as_tensor(a, dtype=torch.float32), torch.as_tensor(b, dtype=torch.float32)
        eps = torch.finfo(torch.float32).eps
        return float((a * b).sum() / (a.norm().clamp_min(eps) * b.norm().clamp_min(eps)))

"""Device-side token sampling (csrc/sampler.cu: ``sb_sample_rows``) with a host fallback.

``DeviceSampler`` owns the per-row xorshift64 states (seeded like the host ``SamplerRng``), the token
history used by the repetition penalty and the scratch row; ``sample(logits)`` picks one token per
row without leaving the device, so a sampled decode step can be captured in a CUDA graph. On CPU
tensors it calls the host ``sample_row`` (scirust_b200/generate.py), the reference's policy
(scirust-sciagent/src/generate.rs:202-337).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..generate import SamplerRng, SamplingParams, sample_row, seed_to_state
from . import _lib
from . import gemm as _g

_lib.register("sb_sample_rows", [_lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.f32, _lib.i32, _lib.f32, _lib.f32,
                                 _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                 _lib.vp, _lib.vp])


def _i64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


class DeviceSampler:
    def __init__(self, params: SamplingParams, rows: int, vocab: int, seeds, device, history_len: int = 0):
        self.params, self.rows, self.vocab = params, rows, vocab
        self.device = torch.device(device)
        seeds = list(seeds)
        if len(seeds) != rows:
            raise ValueError("one seed per row")
        self._host_rng = [SamplerRng(s) for s in seeds]
        # xorshift64 states as int64 bit patterns
        self.state = torch.tensor([_i64(seed_to_state(s)) for s in seeds], dtype=torch.int64, device=self.device)
        self.history = torch.zeros((rows, max(history_len, 1)), dtype=torch.int64, device=self.device)
        self.n_hist = torch.zeros(rows, dtype=torch.int32, device=self.device)
        self.work = (_lib.empty((rows, vocab), torch.int32, self.device)
                     if self.device.type == "cuda" else None)
        self.tokens = torch.zeros(rows, dtype=torch.int64, device=self.device)

    def set_history(self, tokens: torch.Tensor):
        """tokens [rows, n]: the prompt (and anything generated so far), oldest first."""
        n = tokens.shape[1]
        if n > self.history.shape[1]:
            raise ValueError("history buffer too small")
        self.history[:, :n] = tokens.to(self.device)
        self.n_hist.fill_(n)

    def push(self, tokens: torch.Tensor):
        """Append one token per row to the history (device-side, graph-capturable)."""
        idx = self.n_hist.to(torch.int64).clamp_(max=self.history.shape[1] - 1)
        self.history.scatter_(1, idx[:, None], tokens[:, None])
        self.n_hist.add_(1).clamp_(max=self.history.shape[1])

    def sample(self, logits: torch.Tensor, out_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """logits fp32 [rows, vocab] -> int64 [rows]; advances each row's RNG by one draw when
        temperature > 0."""
        p = self.params
        out = self.tokens if out_tokens is None else out_tokens
        B = logits.shape[0]
        if not logits.is_cuda:
            hist = self.history.tolist()
            nh = self.n_hist.tolist()
            for b in range(B):
                out[b] = sample_row(logits[b], p, hist[b][:nh[b]], self._host_rng[b])
            return out
        if logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise ValueError("sample: fp32 logits with unit inner stride expected")
        if p.repetition_window > 256 and p.repetition_penalty > 1.0:
            raise ValueError("the device sampler supports repetition windows up to 256 tokens")
        _lib.call("sb_sample_rows", logits.data_ptr(), logits.stride(0), B, self.vocab, float(p.temperature),
                  int(p.top_k), float(p.top_p), float(p.repetition_penalty), int(p.repetition_window),
                  self.history.data_ptr(), self.history.stride(0), self.n_hist.data_ptr(), self.state.data_ptr(),
                  out.data_ptr(), None, 0, 0, self.work.data_ptr(), _lib.stream())
        _g.launch_count += 1
        return out

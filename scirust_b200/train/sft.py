"""Supervised fine-tuning on instruction / response pairs.

A JSON-lines file holds one example per line: ``{"instruction": ..., "output": ..., "tool_calls": [{"name": ...,
"params": {...}}]}``. An example becomes ``<bos> "user: " instruction <eos> <bos> "assistant: " output <eos>``.
Batches are padded to ONE fixed length (``max_seq_len``): the shapes never change from step to step, which is what
the persistent kernels and any captured graph want. Padding positions, and with ``mask_prompt`` also the
prompt positions, carry the target ``-1``, which the fused cross-entropy kernel skips (zero loss, zero gradient), so
only response tokens teach. The optimisation step is the framework's ``Trainer`` (warm-up + cosine to a tenth of the
peak rate, global-norm clipping at 1).
Reference counterpart: scirust-sciagent/src/train/sft.rs:12-190 (same prompt format; no padding, no prompt mask).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

import torch

from .trainer import Trainer, TrainerConfig


@dataclass
class ToolCallExample:
    name: str
    params: list = field(default_factory=list)          # (key, value) pairs


@dataclass
class SftExample:
    instruction: str
    output: str
    tool_calls: list | None = None


class SftDataset:
    def __init__(self, examples):
        self.examples = list(examples)

    @staticmethod
    def from_jsonl(path) -> "SftDataset":
        examples = []
        with open(path, "r", encoding="utf-8") as f:
            for n, line in enumerate(f, 1):
                if not line.strip():
                    continue
                try:
                    j = json.loads(line)
                except json.JSONDecodeError as e:
                    raise ValueError(f"{path}:{n}: {e}") from e
                calls = None
                if isinstance(j.get("tool_calls"), list):
                    calls = [ToolCallExample(tc["name"], [(k, v if isinstance(v, str) else "") for k, v in tc["params"].items()])
                             for tc in j["tool_calls"]
                             if isinstance(tc, dict) and isinstance(tc.get("name"), str) and isinstance(tc.get("params"), dict)]
                ins, out = j.get("instruction"), j.get("output")
                examples.append(SftExample(ins if isinstance(ins, str) else "", out if isinstance(out, str) else "", calls))
        return SftDataset(examples)

    def __len__(self):
        return len(self.examples)

    def is_empty(self) -> bool:
        return not self.examples


def format_sft_prompt(example: SftExample, tokenizer, with_boundary: bool = False):
    """Token ids of one example; with ``with_boundary`` also the index of the first RESPONSE token."""
    bos, eos = tokenizer.special_id("<bos>"), tokenizer.special_id("<eos>")
    prompt = [bos] + tokenizer.encode("user: ") + tokenizer.encode(example.instruction) + [eos, bos] + tokenizer.encode("assistant: ")
    tokens = prompt + tokenizer.encode(example.output) + [eos]
    return (tokens, len(prompt)) if with_boundary else tokens


def sft_batch(examples, tokenizer, max_seq_len: int, mask_prompt: bool = True, pad_id: int = 0):
    """``(inputs [B, max_seq_len], targets [B, max_seq_len])``; ignored target positions hold -1."""
    B = len(examples)
    inp = torch.full((B, max_seq_len), pad_id, dtype=torch.int64)
    tgt = torch.full((B, max_seq_len), -1, dtype=torch.int64)
    for b, ex in enumerate(examples):
        tokens, start = format_sft_prompt(ex, tokenizer, True)
        tokens = tokens[: max_seq_len + 1]
        n = len(tokens) - 1
        if n < 1:
            continue
        t = torch.tensor(tokens, dtype=torch.int64)
        inp[b, :n] = t[:-1]
        tgt[b, :n] = t[1:]
        if mask_prompt:
            tgt[b, : max(min(start - 1, n), 0)] = -1         # target j is token j + 1: the first response token is target start - 1
    return inp, tgt


def sft_train(model, dataset: SftDataset, tokenizer, lr: float, epochs: int, batch_size: int, max_seq_len: int,
              mask_prompt: bool = True, log=None, trainer: Trainer | None = None):
    """Returns the per-epoch mean losses. ``model`` is a ``GQADecoder`` (any device)."""
    total = max(len(dataset) * epochs // max(batch_size, 1), 1)
    trainer = trainer or Trainer(model, TrainerConfig(lr=lr, min_lr=lr * 0.1, warmup_steps=total // 20, total_steps=total,
                                                      max_grad_norm=1.0, weight_decay=0.0))
    history, step = [], 0
    for epoch in range(epochs):
        losses = []
        for i in range(0, len(dataset), batch_size):
            chunk = dataset.examples[i:i + batch_size]
            if len(chunk) < batch_size:
                chunk = chunk + dataset.examples[: batch_size - len(chunk)]       # keep the batch shape fixed
            inp, tgt = sft_batch(chunk, tokenizer, max_seq_len, mask_prompt)
            live = int((tgt >= 0).sum())
            if live == 0:
                continue
            # Trainer.train_step takes [B, S+1] tokens and derives targets by shifting; SFT needs its own targets,
            # so the step is issued through the same pieces with explicit targets.
            loss = _step_with_targets(trainer, inp, tgt)
            losses.append(float(loss) * tgt.numel() / live)                        # mean over the live targets
            step += 1
            if log and step % 10 == 0:
                log(f"[SFT epoch {epoch} step {step}] loss: {losses[-1]:.4f} | lr: {trainer.schedule.lr_at(step - 1):.8f}")
        history.append(sum(losses) / max(len(losses), 1))
        if log:
            log(f"[SFT epoch {epoch}] avg loss: {history[-1]:.4f}")
    return history


def _step_with_targets(trainer: Trainer, inp: torch.Tensor, tgt: torch.Tensor):
    from .. import ops
    model, c = trainer.model, trainer.cfg
    dev = model.flat.device
    inp, tgt = inp.to(dev, non_blocking=True), tgt.to(dev, non_blocking=True)
    model.zero_grad_flags()
    loss = model(inp, tgt)
    loss.backward()
    ops.sumsq(model.flat_grad, out=trainer.grad_sumsq)
    trainer.step += 1
    ops.optim_step(trainer.master, trainer.m, trainer.v, model.flat_grad, model.flat, lr=trainer.schedule.lr_at(trainer.step - 1),
                   beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay, step=trainer.step,
                   decay_end=model.decay_end, grad_sumsq=trainer.grad_sumsq, max_grad_norm=c.max_grad_norm, grad_scale=1.0,
                   mode=c.optimizer)
    trainer.last_loss = loss.detach()
    return trainer.last_loss

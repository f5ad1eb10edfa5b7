#!/usr/bin/env python
"""Transformer demo: a tiny decoder-only language model learns a character sequence and continues it.

    python examples/transformer_demo.py [--steps 300] [--mixer llama|mamba|retnet|rwkv|...]

Counterpart of the reference's ``transformer_demo`` example: builds the model from the layer zoo
(``nn.zoo.NdDecoderLM`` over any of its sequence mixers), trains next-character prediction with AdamW and a
warm-up-cosine schedule, then generates greedily and with nucleus sampling through the shared sampling policy
(``generate.sample_row``), so the sampled continuation is reproducible for a seed.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from scirust_b200.generate import SamplerRng, SamplingParams, sample_row  # noqa: E402
from scirust_b200.nn.zoo import NdDecoderLM  # noqa: E402
from scirust_b200.train.schedule import WarmupCosineSchedule  # noqa: E402

TEXT = ("the quick brown fox jumps over the lazy dog. " * 8).strip()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--mixer", default="llama")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    torch.manual_seed(a.seed)
    chars = sorted(set(TEXT))
    stoi = {c: i for i, c in enumerate(chars)}
    ids = torch.tensor([stoi[c] for c in TEXT])
    model = NdDecoderLM(len(chars), d_model=48, n_layers=2, mixer=a.mixer, n_heads=4, n_kv_heads=2, d_ff=96)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, weight_decay=0.01)
    sched = WarmupCosineSchedule(3e-3, 3e-4, 20, a.steps)
    S = 64
    for step in range(a.steps):
        off = (step * 17) % (len(ids) - S - 1)
        x, y = ids[off:off + S][None], ids[off + 1:off + S + 1]
        for gparam in opt.param_groups:
            gparam["lr"] = sched.lr_at(step)
        loss = torch.nn.functional.cross_entropy(model(x)[0], y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        if step % 50 == 0 or step + 1 == a.steps:
            print(f"step {step:4d}  loss {float(loss.detach()):.4f}  lr {sched.lr_at(step):.2e}")

    def generate(prompt, n, params, seed):
        toks = [stoi[c] for c in prompt]
        rng = SamplerRng(seed)
        with torch.no_grad():
            for _ in range(n):
                logits = model(torch.tensor([toks[-S:]]))[0, -1]
                toks.append(sample_row(logits, params, toks, rng))
        return "".join(chars[t] for t in toks)
    print("greedy :", generate("the quick ", 40, SamplingParams(), 0))
    print("sampled:", generate("the quick ", 40, SamplingParams(temperature=0.8, top_k=8, top_p=0.95), 7))
    return float(loss.detach())


if __name__ == "__main__":
    main()

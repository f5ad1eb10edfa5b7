"""Tone sequences -> log-mel features (scirust_b200.dsp) -> convolutional encoder + linear head -> CTC loss.

Each synthetic clip plays a short sequence of "notes" (one of four tones each); the model must name the notes in order
without being told where they start. Runs on CPU in well under a minute; pass --device cuda to run the same code on a GPU.

    python examples/audio_ctc_demo.py --steps 150
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from scirust_b200 import dsp  # noqa: E402
from scirust_b200.nn import AudioEncoder, ctc_loss  # noqa: E402

RATE, NOTE, TONES = 8000, 1600, (440.0, 660.0, 880.0, 1320.0)


def make_clips(n, notes, gen):
    labels = torch.randint(0, len(TONES), (n, notes), generator=gen)
    t = torch.arange(NOTE) / RATE
    env = torch.hann_window(NOTE, periodic=False)
    waves = torch.stack([torch.cat([torch.sin(2 * math.pi * TONES[int(k)] * t) * env for k in row]) for row in labels])
    return waves + 0.05 * torch.randn(waves.shape, generator=gen), labels


def greedy_decode(logits, blank):
    out = []
    for row in logits.argmax(-1).tolist():
        seq, prev = [], blank
        for k in row:
            if k != prev and k != blank:
                seq.append(k)
            prev = k
        out.append(seq)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=150)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    gen = torch.Generator().manual_seed(0)
    notes, mels = 4, 24
    waves, labels = make_clips(64, notes, gen)
    feats = dsp.log_mel_features(waves, RATE, frame=256, hop=128, n_mels=mels)          # [clips, frames, mels]
    feats = ((feats - feats.mean()) / feats.std()).to(a.device)
    frames = feats.shape[1]
    enc = AudioEncoder(1, 8, 8, in_h=frames, in_w=mels).to(a.device)
    oh, ow = enc.out_hw(frames, mels)
    head = torch.nn.Linear(8 * ow, len(TONES) + 1).to(a.device)                          # last class = blank
    opt = torch.optim.Adam(list(enc.parameters()) + list(head.parameters()), lr=3e-3)

    def logits_of(x):
        y = enc(x.reshape(x.shape[0], -1))                                              # [clips, 8 * oh * ow]
        y = y.reshape(x.shape[0], 8, oh, ow).permute(0, 2, 1, 3).reshape(x.shape[0], oh, 8 * ow)
        return head(y)                                                                  # [clips, time, classes]
    tgt = labels.to(a.device)
    for step in range(a.steps):
        opt.zero_grad()
        loss = ctc_loss(logits_of(feats), tgt, reduction="none").mean()
        loss.backward()
        opt.step()
        if step % 25 == 0 or step == a.steps - 1:
            print(f"step {step:4d}  ctc loss {float(loss.detach()):.4f}")
    with torch.no_grad():
        test_w, test_l = make_clips(32, notes, gen)
        tf = dsp.log_mel_features(test_w, RATE, frame=256, hop=128, n_mels=mels)
        tf = ((tf - tf.mean()) / tf.std()).to(a.device)
        decoded = greedy_decode(logits_of(tf).cpu(), len(TONES))
    exact = sum(d == row for d, row in zip(decoded, test_l.tolist())) / len(decoded)
    print(f"held-out clips decoded exactly: {exact:.2%}")
    return exact


if __name__ == "__main__":
    main()

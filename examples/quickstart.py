#!/usr/bin/env python
"""XOR with the tape API, in the shape of the reference's quickstart (2 -> 8 -> 2, Adam 0.05):
one fresh tape per step, ``Linear`` weights registered on the tape, softmax cross-entropy, backward,
optimizer step by node index."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from scirust_b200 import nn  # noqa: E402
from scirust_b200.autodiff import Adam, Tape  # noqa: E402

rng = nn.PcgEngine(42)
w1 = nn.KaimingNormal().fill((2, 8), 2, 8, rng)
b1 = torch.zeros(1, 8)
w2 = nn.KaimingNormal().fill((8, 2), 8, 2, rng)
b2 = torch.zeros(1, 2)
x = torch.tensor([[0., 0.], [0., 1.], [1., 0.], [1., 1.]])
y = torch.tensor([[1., 0.], [0., 1.], [0., 1.], [1., 0.]])
opt = Adam(0.05)
params = [w1, b1, w2, b2]
for epoch in range(1000):
    tape = Tape()
    vs = [tape.input(p) for p in params]
    h = tape.constant(x).linear(vs[0], vs[1]).relu()
    logits = h.linear(vs[2], vs[3])
    loss = nn.CrossEntropyLoss()(logits, tape.constant(y))
    tape.backward(loss)
    # optimizer state is keyed by node index; parameters are registered first, so indices are stable
    opt.step([v.idx for v in vs], tape)
    params = [tape.value(v.idx).t for v in vs]
    if epoch % 250 == 0 or epoch == 999:
        print(f"epoch {epoch:4d} loss {loss.item():.6f}")
pred = (torch.relu(x @ params[0] + params[1]) @ params[2] + params[3]).argmax(1)
print("predictions", pred.tolist(), "expected", y.argmax(1).tolist())

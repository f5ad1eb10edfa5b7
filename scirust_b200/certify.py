"""Certified output bounds and the statistical response guard.

* ``Interval`` / ``IbpLinear`` / ``IbpMlp``: interval bound propagation through affine + ReLU layers: an
  axis-aligned box around an input is pushed through the network, every output is bracketed, and
  ``certified_robust`` says whether the predicted class can change anywhere in the box.
* ``crown_bounds``: the CROWN linear relaxation of a one-hidden-layer ReLU network (chord upper bound, area-minimising
  lower slope per unstable neuron, back-substituted to the input and intervalised once), never looser than IBP.
* ``ConformalClassifier`` / ``StatisticalGuard``: split-conformal prediction sets at risk ``alpha`` and the
  accept / abstain / reject verdict built on them (one class in the set: accept; several: abstain; none: reject).

Counterparts in the reference: scirust-core/src/nn/ibp.rs (``Interval``, ``IbpLinear``, ``IbpMlp``,
``certified_robust`` :838, ``crown_bounds`` :857), nn/conformal.rs:93 and nn/guard.rs:34-70; `scirust certify` and
`scirust guard` (scirust-cli/src/learning.rs:46, synergy.rs:90) print their results.
"""
from __future__ import annotations

import torch

from .conformal import ConformalClassifier  # noqa: F401  (the guard's calibrated threshold rule)


class Interval:
    def __init__(self, lo: torch.Tensor, hi: torch.Tensor):
        self.lo, self.hi = lo.float(), hi.float()
        if bool((self.lo > self.hi).any()):
            raise ValueError("Interval: lo must not exceed hi")

    @staticmethod
    def around(centre, eps: float) -> "Interval":
        c = torch.as_tensor(centre, dtype=torch.float32)
        return Interval(c - eps, c + eps)

    def width(self) -> torch.Tensor:
        return self.hi - self.lo


class IbpLinear:
    """``y = x W + b`` with ``W [in, out]`` (the x.W layout of the framework's Linear)."""

    def __init__(self, w: torch.Tensor, b: torch.Tensor):
        self.w, self.b = w.float(), b.float().reshape(-1)
        self.in_f, self.out_f = self.w.shape

    @staticmethod
    def from_linear(lin) -> "IbpLinear":
        w = lin.weight.detach()
        if w.shape[0] == getattr(lin, "out_features", -1) and w.shape[1] == getattr(lin, "in_features", -2):
            w = w.t()                      # torch.nn.Linear stores [out, in]
        b = lin.bias.detach() if getattr(lin, "bias", None) is not None else torch.zeros(w.shape[1])
        return IbpLinear(w, b)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() @ self.w + self.b

    def forward_interval(self, box: Interval) -> Interval:
        c, r = 0.5 * (box.lo + box.hi), 0.5 * (box.hi - box.lo)
        mid = c @ self.w + self.b
        rad = r @ self.w.abs()
        return Interval(mid - rad, mid + rad)


class IbpMlp:
    """Affine layers with ReLU between them (none after the last)."""

    def __init__(self, layers):
        self.layers = list(layers)

    def forward(self, x) -> torch.Tensor:
        h = torch.as_tensor(x, dtype=torch.float32)
        for i, l in enumerate(self.layers):
            h = l.forward(h)
            if i + 1 < len(self.layers):
                h = h.clamp_min(0)
        return h

    def certify(self, box: Interval) -> Interval:
        b = box
        for i, l in enumerate(self.layers):
            b = l.forward_interval(b)
            if i + 1 < len(self.layers):
                b = Interval(b.lo.clamp_min(0), b.hi.clamp_min(0))
        return b


def certified_robust(out: Interval, target: int) -> bool:
    """The target's lower bound exceeds every other class's upper bound."""
    others = torch.cat([out.hi[:target], out.hi[target + 1:]])
    return bool((out.lo[target] > others).all())


def crown_bounds(l1: IbpLinear, l2: IbpLinear, box: Interval) -> Interval:
    if l1.out_f != l2.in_f or box.lo.numel() != l1.in_f:
        raise ValueError("crown_bounds: layer sizes must chain")
    pre = l1.forward_interval(box)
    zlo, zhi = pre.lo, pre.hi
    hid = l1.out_f
    sl, su, iu = torch.zeros(hid), torch.zeros(hid), torch.zeros(hid)
    pos, neg = zlo >= 0, zhi <= 0
    unstable = ~(pos | neg)
    sl[pos] = 1.0
    su[pos] = 1.0
    s = zhi[unstable] / (zhi[unstable] - zlo[unstable])
    su[unstable] = s
    iu[unstable] = -s * zlo[unstable]
    sl[unstable] = (zhi[unstable] >= -zlo[unstable]).float()
    c, r = 0.5 * (box.lo + box.hi), 0.5 * (box.hi - box.lo)
    lo, hi = torch.zeros(l2.out_f), torch.zeros(l2.out_f)
    for o in range(l2.out_f):
        w2 = l2.w[:, o]
        for upper in (False, True):
            pick_lower = (w2 >= 0) ^ upper
            slope = torch.where(pick_lower, sl, su)
            icpt = torch.where(pick_lower, torch.zeros(hid), iu)
            cz = w2 * slope
            konst = l2.b[o] + (w2 * icpt).sum() + (cz * l1.b).sum()
            coef = l1.w @ cz
            centre = konst + (coef * c).sum()
            rad = (coef.abs() * r).sum()
            if upper:
                hi[o] = centre + rad
            else:
                lo[o] = centre - rad
    return Interval(torch.minimum(lo, hi), torch.maximum(lo, hi))


class StatisticalGuard:
    ACCEPT, ABSTAIN, REJECT = "accept", "abstain", "reject"

    def __init__(self, clf: ConformalClassifier):
        self.clf = clf

    @staticmethod
    def calibrate(cal_probs, cal_labels, alpha: float) -> "StatisticalGuard":
        return StatisticalGuard(ConformalClassifier.calibrate(cal_probs, cal_labels, alpha))

    def prediction_set(self, probs):
        return self.clf.predict_set(probs)

    def decide(self, probs):
        """``("accept", class)``, ``("abstain", None)`` or ``("reject", None)``."""
        s = self.clf.predict_set(probs)
        if len(s) == 0:
            return self.REJECT, None
        if len(s) == 1:
            return self.ACCEPT, s[0]
        return self.ABSTAIN, None

    def covers(self, probs, y_true: int) -> bool:
        return self.clf.covers(probs, y_true)

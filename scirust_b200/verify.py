"""Abstract domains and complete verifiers for ReLU networks (``IbpLinear`` stacks, ReLU between layers).

* ``Zonotope`` / ``relu_zonotope`` / ``certify_zonotope``: DeepZ. Affine layers map a zonotope exactly; an unstable
  ReLU becomes ``lambda x + mu`` (``lambda = u/(u-l)``, ``mu = -lambda l / 2``) plus one fresh generator of magnitude
  ``mu``. Generators are one ``[m, n]`` matrix, so a layer is one matrix product.
* ``deeppoly_certify`` / ``deeppoly_bounds``: DeepPoly with eager back-substitution: every neuron keeps a lower and
  an upper bound that is AFFINE in the network inputs. Stored as ``[boxes, d_in + 1, n]`` coefficient tensors, so an
  affine layer is two batched matrix products (positive and negative weight parts) and MANY input boxes are bounded
  in one pass.
* ``verify_robustness``: input-space branch and bound on the margin network (``logit_t - logit_j``). The whole
  frontier of open boxes is bounded per round in one batched DeepPoly pass; boxes whose margins are all positive
  are closed, box centres are probed for concrete counterexamples, the rest are split along their widest axis.
  ``Robust`` / ``Unsafe(x)`` / ``Unknown`` (tolerance or box budget reached).
* ``milp_min_margin`` / ``milp_verify_robustness``: exact worst-case margin of a 2-input, one-hidden-layer network
  by enumerating ReLU activation patterns and solving each 2-D linear program at its vertices.
* ``reluplex_verify``: the same search, but only UNSTABLE neurons (pre-activation interval straddling 0) are
  case-split: ``2^unstable`` leaves instead of ``2^hidden``.

Reference counterpart: scirust-core/src/nn/ibp.rs:190-835 (scalar loops, one box at a time, depth-first stack) and
nn/ibp_checked.rs (validated variants: the checks live in ``Interval`` and in the argument checks here).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .certify import IbpLinear, IbpMlp, Interval


# ------------------------------------------------------------------ zonotopes

class Zonotope:
    """``{ c + sum_i e_i g_i : e_i in [-1, 1] }`` with ``generators [m, n]``."""

    def __init__(self, center: torch.Tensor, generators: torch.Tensor):
        self.center = center.float()
        self.generators = generators.float().reshape(-1, self.center.numel())

    @staticmethod
    def from_interval(box: Interval) -> "Zonotope":
        c = 0.5 * (box.lo + box.hi)
        r = 0.5 * (box.hi - box.lo)
        keep = torch.nonzero(r != 0).reshape(-1)
        g = torch.zeros(keep.numel(), c.numel())
        g[torch.arange(keep.numel()), keep] = r[keep]
        return Zonotope(c, g)

    def radii(self) -> torch.Tensor:
        return self.generators.abs().sum(0)

    def interval(self) -> Interval:
        r = self.radii()
        return Interval(self.center - r, self.center + r)


def forward_zonotope(layer: IbpLinear, z: Zonotope) -> Zonotope:
    if z.center.numel() != layer.in_f:
        raise ValueError("forward_zonotope: input size")
    return Zonotope(z.center @ layer.w + layer.b, z.generators @ layer.w)


def relu_zonotope(z: Zonotope) -> Zonotope:
    box = z.interval()
    l, u = box.lo, box.hi
    unstable = (l < 0) & (u > 0)
    lam = torch.where(l >= 0, torch.ones_like(l), torch.zeros_like(l))
    lam = torch.where(unstable, u / torch.where(unstable, u - l, torch.ones_like(u)), lam)
    mu = torch.where(unstable, -lam * l * 0.5, torch.zeros_like(l))
    center = lam * z.center + mu
    gens = z.generators * lam[None, :]
    fresh_idx = torch.nonzero(mu != 0).reshape(-1)
    fresh = torch.zeros(fresh_idx.numel(), l.numel())
    fresh[torch.arange(fresh_idx.numel()), fresh_idx] = mu[fresh_idx]
    return Zonotope(center, torch.cat([gens, fresh], 0))


def certify_zonotope(layers, box: Interval) -> Interval:
    z = Zonotope.from_interval(box)
    for i, layer in enumerate(layers):
        z = forward_zonotope(layer, z)
        if i + 1 < len(layers):
            z = relu_zonotope(z)
    return z.interval()


# ------------------------------------------------------------------ DeepPoly (batched over boxes)

def _concretize(aff: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, maximize: bool) -> torch.Tensor:
    """``aff [nb, d+1, n]`` (last row = constant) over boxes ``lo, hi [nb, d]`` -> ``[nb, n]``."""
    coef, cst = aff[:, :-1, :], aff[:, -1, :]
    pos, neg = coef.clamp_min(0), coef.clamp_max(0)
    a, b = (hi, lo) if maximize else (lo, hi)
    return cst + torch.einsum("bd,bdn->bn", a, pos) + torch.einsum("bd,bdn->bn", b, neg)


def deeppoly_bounds(layers, lo: torch.Tensor, hi: torch.Tensor):
    """Output bounds ``(lo [nb, out], hi [nb, out])`` for a batch of input boxes ``lo, hi [nb, d]``."""
    if not layers:
        raise ValueError("deeppoly: empty network")
    lo, hi = lo.float(), hi.float()
    nb, d = lo.shape
    eye = torch.cat([torch.eye(d), torch.zeros(1, d)], 0)
    lower = eye[None].repeat(nb, 1, 1)
    upper = lower.clone()
    for li, layer in enumerate(layers):
        wp, wn = layer.w.clamp_min(0), layer.w.clamp_max(0)
        new_upper = upper @ wp + lower @ wn
        new_lower = lower @ wp + upper @ wn
        new_upper[:, -1, :] += layer.b
        new_lower[:, -1, :] += layer.b
        lower, upper = new_lower, new_upper
        if li + 1 < len(layers):
            l = _concretize(lower, lo, hi, False)
            u = _concretize(upper, lo, hi, True)
            dead = u <= 0
            unstable = (l < 0) & (u > 0)
            slope = torch.where(unstable, u / torch.where(unstable, u - l, torch.ones_like(u)), torch.ones_like(u))
            slope = torch.where(dead, torch.zeros_like(slope), slope)
            upper = upper * slope[:, None, :]
            upper[:, -1, :] = upper[:, -1, :] - torch.where(unstable, slope * l, torch.zeros_like(l))
            lam = torch.where(unstable, (u > -l).float(), torch.ones_like(u))
            lam = torch.where(dead, torch.zeros_like(lam), lam)
            lower = lower * lam[:, None, :]
    return _concretize(lower, lo, hi, False), _concretize(upper, lo, hi, True)


def deeppoly_certify(layers, box: Interval) -> Interval:
    l, u = deeppoly_bounds(layers, box.lo[None], box.hi[None])
    return Interval(torch.minimum(l[0], u[0]), u[0])


IbpMlp.certify_zonotope = lambda self, box: certify_zonotope(self.layers, box)
IbpMlp.certify_deeppoly = lambda self, box: deeppoly_certify(self.layers, box)


# ------------------------------------------------------------------ branch and bound

@dataclass
class BabResult:
    status: str                      # "robust" | "unsafe" | "unknown"
    counterexample: torch.Tensor | None = None
    boxes: int = 0

    ROBUST, UNSAFE, UNKNOWN = "robust", "unsafe", "unknown"

    def __eq__(self, other):
        return self.status == (other.status if isinstance(other, BabResult) else other)


def _forward(layers, x):
    h = x
    for i, l in enumerate(layers):
        h = h @ l.w + l.b
        if i + 1 < len(layers):
            h = h.clamp_min(0)
    return h


def build_margin_net(layers, t: int):
    """Replace the logit layer by ``logit_t - logit_j`` for every ``j != t``: all outputs positive <=> t wins."""
    last = layers[-1]
    others = [j for j in range(last.out_f) if j != t]
    wm = last.w[:, [t]] - last.w[:, others]
    bm = last.b[t] - last.b[others]
    return list(layers[:-1]) + [IbpLinear(wm, bm)]


def verify_robustness(layers, box: Interval, true_class: int, tol: float = 1e-4, max_boxes: int = 10000,
                      frontier: int = 256) -> BabResult:
    mnet = build_margin_net(layers, true_class)
    lo, hi = box.lo[None].clone(), box.hi[None].clone()
    count = 0
    while lo.shape[0]:
        take = min(frontier, lo.shape[0])
        blo, bhi = lo[-take:], hi[-take:]                  # newest boxes first (depth-first flavour, batched)
        lo, hi = lo[:-take], hi[:-take]
        count += take
        if count > max_boxes:
            return BabResult(BabResult.UNKNOWN, None, count)
        out_lo, _ = deeppoly_bounds(mnet, blo, bhi)
        open_ = ~(out_lo > 0).all(1)
        if not bool(open_.any()):
            continue
        blo, bhi = blo[open_], bhi[open_]
        centre = 0.5 * (blo + bhi)
        bad = (_forward(mnet, centre) <= 0).any(1)
        if bool(bad.any()):
            return BabResult(BabResult.UNSAFE, centre[torch.nonzero(bad)[0, 0]].clone(), count)
        width = bhi - blo
        if bool((0.5 * width.max(1).values < tol).any()):
            return BabResult(BabResult.UNKNOWN, None, count)
        axis = width.argmax(1)
        mid = centre.gather(1, axis[:, None])
        left_hi = bhi.scatter(1, axis[:, None], mid)
        right_lo = blo.scatter(1, axis[:, None], mid)
        lo = torch.cat([lo, blo, right_lo], 0)
        hi = torch.cat([hi, left_hi, bhi], 0)
    return BabResult(BabResult.ROBUST, None, count)


# ------------------------------------------------------------------ exact 2-input verifiers

def _lp_min_2d(cons: torch.Tensor, obj: torch.Tensor):
    """min obj.x over {x : cons[:, :2] x <= cons[:, 2]} by vertex enumeration (bounded region). None if empty."""
    n = cons.shape[0]
    i, j = torch.triu_indices(n, n, 1)
    a, b = cons[i], cons[j]
    det = a[:, 0] * b[:, 1] - a[:, 1] * b[:, 0]
    ok = det.abs() >= 1e-9
    if not bool(ok.any()):
        return None
    a, b, det = a[ok], b[ok], det[ok]
    x0 = (a[:, 2] * b[:, 1] - a[:, 1] * b[:, 2]) / det
    x1 = (a[:, 0] * b[:, 2] - a[:, 2] * b[:, 0]) / det
    pts = torch.stack([x0, x1], 1)
    feas = ((pts @ cons[:, :2].t()) <= cons[:, 2][None] + 1e-4).all(1)
    if not bool(feas.any()):
        return None
    pts = pts[feas]
    vals = pts @ obj
    k = int(vals.argmin())
    return float(vals[k]), pts[k]


def _box_constraints(box: Interval) -> torch.Tensor:
    return torch.tensor([[1.0, 0.0, float(box.hi[0])], [-1.0, 0.0, -float(box.lo[0])],
                         [0.0, 1.0, float(box.hi[1])], [0.0, -1.0, -float(box.lo[1])]])


def _pattern_min_margin(l1, l2, base, active, t):
    """Smallest margin over one activation pattern (region = box and the pattern's half-spaces)."""
    w0, w1, b1 = l1.w[0], l1.w[1], l1.b
    sign = torch.where(active, -torch.ones_like(b1), torch.ones_like(b1))
    region = torch.cat([base, torch.stack([sign * w0, sign * w1, -sign * b1], 1)], 0)
    best = None
    for j in range(l2.out_f):
        if j == t:
            continue
        coef = (l2.w[:, t] - l2.w[:, j]) * active.float()
        obj = torch.stack([(coef * w0).sum(), (coef * w1).sum()])
        d = float(l2.b[t] - l2.b[j] + (coef * b1).sum())
        r = _lp_min_2d(region, obj)
        if r is not None and (best is None or r[0] + d < best[0]):
            best = (r[0] + d, r[1])
    return best


def milp_min_margin(l1: IbpLinear, l2: IbpLinear, box: Interval, true_class: int):
    if l1.in_f != 2:
        raise ValueError("milp_min_margin: exactly 2 inputs")
    if l1.out_f != l2.in_f:
        raise ValueError("milp_min_margin: layer mismatch")
    h = l1.out_f
    base = _box_constraints(box)
    best, witness = float("inf"), 0.5 * (box.lo + box.hi)
    for pat in range(1 << h):
        active = torch.tensor([(pat >> i) & 1 == 1 for i in range(h)])
        r = _pattern_min_margin(l1, l2, base, active, true_class)
        if r is not None and r[0] < best:
            best, witness = r
    return best, witness


def milp_verify_robustness(l1, l2, box, true_class) -> BabResult:
    m, witness = milp_min_margin(l1, l2, box, true_class)
    return BabResult(BabResult.ROBUST) if m > 0 else BabResult(BabResult.UNSAFE, witness)


def reluplex_unstable_count(l1: IbpLinear, box: Interval) -> int:
    z = l1.forward_interval(box)
    return int(((z.lo < 0) & (z.hi > 0)).sum())


def reluplex_verify(l1: IbpLinear, l2: IbpLinear, box: Interval, true_class: int) -> BabResult:
    if l1.in_f != 2:
        raise ValueError("reluplex_verify: exactly 2 inputs")
    z = l1.forward_interval(box)
    forced_on = z.lo >= 0
    unstable = torch.nonzero((z.lo < 0) & (z.hi > 0)).reshape(-1).tolist()
    base = _box_constraints(box)
    for pat in range(1 << len(unstable)):
        active = forced_on.clone()
        for bit, nu in enumerate(unstable):
            if (pat >> bit) & 1:
                active[nu] = True
        r = _pattern_min_margin(l1, l2, base, active, true_class)
        if r is not None and r[0] <= 0:
            return BabResult(BabResult.UNSAFE, r[1], pat + 1)
    return BabResult(BabResult.ROBUST, None, 1 << len(unstable))

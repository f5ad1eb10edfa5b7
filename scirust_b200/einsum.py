"""Einstein summation lowered to batched matrix products, with a planned contraction order.

``einsum(pattern, *tensors)`` accepts explicit (``"ij,jk->ik"``) and implicit (``"ij,jk"``: output = labels that occur once,
in alphabetical order) patterns, repeated labels inside one operand (diagonals), labels summed inside one operand, and
any number of operands. ``ContractionPlan`` fixes the pairwise order ahead of time: exhaustive dynamic programming over
subsets for up to ``OPTIMAL_MAX`` operands, a greedy smallest-intermediate rule beyond; both minimise multiply-adds with
the size of the largest intermediate as the tie-break. Every pairwise step is ONE ``torch.bmm`` after a permute / reshape
into ``[batch, M, K] x [batch, K, N]`` (labels shared and kept -> batch, shared and dropped -> K, the rest -> M and N): on
a GPU each step is a tensor-core GEMM, never an index loop. The plan records FLOPs and peak intermediate elements so
a caller can compare orders without running them.
Reference counterpart: scirust-tensor-einsum/src/lib.rs:12-205 (``einsum`` by nested index iteration) and
scirust-tensor-contraction/src/lib.rs:14-186 (``ContractionPlan``, left-to-right pairwise).
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field

import torch

OPTIMAL_MAX = 6


class EinsumError(ValueError):
    pass


def parse_pattern(pattern: str, n_operands: int):
    p = "".join(pattern.split())
    if "->" in p:
        lhs, rhs = p.split("->", 1)
        explicit = True
    else:
        lhs, rhs, explicit = p, "", False
    specs = lhs.split(",")
    if len(specs) != n_operands:
        raise EinsumError(f"pattern names {len(specs)} operands, {n_operands} given")
    for s in specs + [rhs]:
        if not all(c.isalpha() for c in s):
            raise EinsumError("labels are letters")
    if not explicit:
        cnt = {}
        for s in specs:
            for c in s:
                cnt[c] = cnt.get(c, 0) + 1
        rhs = "".join(sorted(c for c, k in cnt.items() if k == 1))
    if len(set(rhs)) != len(rhs):
        raise EinsumError("an output label is repeated")
    seen = set("".join(specs))
    for c in rhs:
        if c not in seen:
            raise EinsumError(f"output index '{c}' does not appear in any input")
    return [list(s) for s in specs], list(rhs)


def _sizes(specs, shapes):
    sizes = {}
    for spec, shp in zip(specs, shapes):
        if len(spec) != len(shp):
            raise EinsumError(f"operand '{''.join(spec)}' has rank {len(spec)} but the tensor has rank {len(shp)}")
        for lab, d in zip(spec, shp):
            if sizes.setdefault(lab, d) != d:
                raise EinsumError(f"index '{lab}' has inconsistent sizes {sizes[lab]} and {d}")
    return sizes


@dataclass
class Step:
    left: int
    right: int
    left_labels: list
    right_labels: list
    out_labels: list
    flops: int


@dataclass
class ContractionPlan:
    pattern: str
    specs: list
    output: list
    steps: list = field(default_factory=list)
    flops: int = 0
    peak_elements: int = 0
    method: str = ""

    # ---- planning
    @staticmethod
    def new(pattern: str, shapes, method: str = "auto") -> "ContractionPlan":
        shapes = [tuple(s) for s in shapes]
        specs, out = parse_pattern(pattern, len(shapes))
        sizes = _sizes(specs, shapes)
        plan = ContractionPlan(pattern, specs, out)
        # operands after the unary clean-up (diagonals taken, private labels summed): label sets without repeats
        others = lambda i: set(out) | {c for j, s in enumerate(specs) if j != i for c in s}
        cur = [[c for c in dict.fromkeys(s) if c in others(i) or len(specs) == 1 and c in out] for i, s in enumerate(specs)]
        if method == "auto":
            method = "optimal" if len(cur) <= OPTIMAL_MAX else "greedy"
        plan.method = method
        order = _optimal(cur, out, sizes) if method == "optimal" else _greedy(cur, out, sizes) if method == "greedy" else \
            [(0, 1)] * (len(cur) - 1) if method == "left" else None
        if order is None:
            raise EinsumError(f"unknown planning method {method!r}")
        work = [list(c) for c in cur]
        for a, b in order:
            la, lb = work[a], work[b]
            rest = set(out) | {c for k, w in enumerate(work) if k not in (a, b) for c in w}
            keep = [c for c in dict.fromkeys(la + lb) if c in rest]
            fl = math.prod(sizes[c] for c in set(la) | set(lb))
            plan.steps.append(Step(a, b, la, lb, keep, fl))
            plan.flops += fl
            plan.peak_elements = max(plan.peak_elements, math.prod(sizes[c] for c in keep))
            work = [w for k, w in enumerate(work) if k not in (a, b)] + [keep]
        plan._cur = cur
        return plan

    # ---- execution
    def execute(self, *tensors) -> torch.Tensor:
        if len(tensors) != len(self.specs):
            raise EinsumError(f"plan expects {len(self.specs)} operands, got {len(tensors)}")
        _sizes(self.specs, [t.shape for t in tensors])
        work = [_unary(t, s, keep) for t, s, keep in zip(tensors, self.specs, self._cur)]
        labels = [list(c) for c in self._cur]
        for st in self.steps:
            res = _pair(work[st.left], labels[st.left], work[st.right], labels[st.right], st.out_labels)
            work = [w for k, w in enumerate(work) if k not in (st.left, st.right)] + [res]
            labels = [l for k, l in enumerate(labels) if k not in (st.left, st.right)] + [st.out_labels]
        res, lab = work[0], labels[0]
        drop = [i for i, c in enumerate(lab) if c not in self.output]
        if drop:
            res = res.sum(drop)
            lab = [c for c in lab if c in self.output]
        return res.permute([lab.index(c) for c in self.output]) if lab != self.output else res


def _unary(t, spec, keep):
    """Take diagonals of repeated labels and sum the labels nobody else needs."""
    lab = list(spec)
    while len(set(lab)) != len(lab):
        c = next(x for x in lab if lab.count(x) > 1)
        i, j = [k for k, x in enumerate(lab) if x == c][:2]
        t = torch.diagonal(t, dim1=i, dim2=j)                                 # the diagonal becomes the last axis
        lab = [x for k, x in enumerate(lab) if k not in (i, j)] + [c]
    drop = [k for k, c in enumerate(lab) if c not in keep]
    if drop:
        t = t.sum(drop)
        lab = [c for c in lab if c in keep]
    return t.permute([lab.index(c) for c in keep]) if lab != list(keep) else t


def _pair(a, la, b, lb, out):
    sa, sb, so = set(la), set(lb), set(out)
    batch = [c for c in la if c in sb and c in so]
    con = [c for c in la if c in sb and c not in so]
    m = [c for c in la if c not in sb]
    n = [c for c in lb if c not in sa]
    size = lambda t, l, cs: [t.shape[l.index(c)] for c in cs]
    bs, ks, ms, ns = size(a, la, batch), size(a, la, con), size(a, la, m), size(b, lb, n)
    a2 = a.permute([la.index(c) for c in batch + m + con]).reshape(math.prod(bs), math.prod(ms), math.prod(ks))
    b2 = b.permute([lb.index(c) for c in batch + con + n]).reshape(math.prod(bs), math.prod(ks), math.prod(ns))
    res = torch.bmm(a2, b2).reshape(bs + ms + ns)
    lab = batch + m + n
    drop = [i for i, c in enumerate(lab) if c not in so]                       # private labels of one side that are summed
    if drop:
        res = res.sum(drop)
        lab = [c for c in lab if c in so]
    return res.permute([lab.index(c) for c in out]) if lab != list(out) else res


def _pair_cost(la, lb, rest, sizes):
    keep = [c for c in dict.fromkeys(list(la) + list(lb)) if c in rest]
    return math.prod(sizes[c] for c in set(la) | set(lb)), math.prod(sizes[c] for c in keep), keep


def _greedy(cur, out, sizes):
    work, order = [list(c) for c in cur], []
    while len(work) > 1:
        best = None
        for a, b in itertools.combinations(range(len(work)), 2):
            rest = set(out) | {c for k, w in enumerate(work) if k not in (a, b) for c in w}
            fl, sz, keep = _pair_cost(work[a], work[b], rest, sizes)
            shared = bool(set(work[a]) & set(work[b]))
            key = (not shared, sz, fl)                                        # outer products last, then small results
            if best is None or key < best[0]:
                best = (key, a, b, keep)
        _, a, b, keep = best
        order.append((a, b))
        work = [w for k, w in enumerate(work) if k not in (a, b)] + [keep]
    return order


def _optimal(cur, out, sizes):
    n = len(cur)
    if n == 1:
        return []
    full = (1 << n) - 1
    labels_of = {1 << i: frozenset(cur[i]) for i in range(n)}
    outside = lambda mask: set(out) | {c for i in range(n) if not mask >> i & 1 for c in cur[i]}
    best = {1 << i: (0, 0, None) for i in range(n)}                           # mask -> (flops, peak, split)
    for size in range(2, n + 1):
        for combo in itertools.combinations(range(n), size):
            mask = sum(1 << i for i in combo)
            keep = frozenset(c for i in combo for c in cur[i]) & frozenset(outside(mask))
            labels_of[mask] = keep
            sub = (mask - 1) & mask
            while sub:
                other = mask ^ sub
                if sub < other and sub in best and other in best:
                    fl = math.prod(sizes[c] for c in labels_of[sub] | labels_of[other])
                    cost = (best[sub][0] + best[other][0] + fl, max(best[sub][1], best[other][1], math.prod(sizes[c] for c in keep)))
                    if mask not in best or cost < best[mask][:2]:
                        best[mask] = (cost[0], cost[1], (sub, other))
                sub = (sub - 1) & mask
    # unroll the split tree into positional (a, b) pairs over a shrinking work list
    order, work = [], [1 << i for i in range(n)]

    def build(mask):
        if best[mask][2] is None:
            return
        l, r = best[mask][2]
        build(l)
        build(r)
        a, b = work.index(l), work.index(r)
        order.append((min(a, b), max(a, b)))
        for m_ in (l, r):
            work.remove(m_)
        work.append(mask)
    build(full)
    return order


def einsum(pattern: str, *tensors, method: str = "auto") -> torch.Tensor:
    tensors = [torch.as_tensor(t) for t in tensors]
    return ContractionPlan.new(pattern, [t.shape for t in tensors], method).execute(*tensors)

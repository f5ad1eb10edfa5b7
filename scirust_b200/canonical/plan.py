"""Planning pipeline of the canonical facade: ``Graph`` -> ``ExecutionPlan`` -> ``MemoryPlan`` -> ``LoweredPlan``.

* ``plan_execution``: the nodes the outputs depend on, in definition order (a valid topological order of an append-only
  graph), with each value's last use; values behind a ``Checkpoint`` are marked recomputable.
* ``plan_memory``: one arena for all intermediates; a value's slot is released after its last use and reused by later
  values (first fit over a free list kept in address order, 256-byte granularity), so the arena is the peak of the
  live set rather than the sum of all values. Views (``Reshape``, ``StopGradient``, ``Checkpoint``) alias their input.
* ``lower``: one kernel record per executed node, of one of the kernel kinds the adapters implement: ``elementwise``
  (relu / scale / add / sub / mul / div / relu_grad / fill), ``transcendental`` (exp / log: executed by the CPU
  reference only, refused by the bit-exact device adapter), ``permute``, ``matmul`` / ``batch_matmul`` (fixed k
  order), ``broadcast`` and ``reduce`` (ascending index order), ``alias`` (no kernel).

Counterparts: scirust-tensor-compile (execution / memory planning), scirust-tensor-reference (lowered artefacts),
scirust-gpu/src/cuda_reference.rs:498-520 (kernel kinds and arities).
"""
from __future__ import annotations

from dataclasses import dataclass

from .ir import Graph, GraphError, _numel

ALIGN = 256
_ALIAS = {"Reshape", "StopGradient", "Checkpoint"}
_KIND = {"Add": "elementwise", "Sub": "elementwise", "Mul": "elementwise", "Div": "elementwise", "Scale": "elementwise",
         "Relu": "elementwise", "ReluGrad": "elementwise", "ZerosLike": "elementwise", "OnesLike": "elementwise",
         "Exp": "transcendental", "Log": "transcendental", "MatMul": "matmul", "BatchMatMul": "batch_matmul",
         "Transpose": "permute", "BroadcastTo": "broadcast", "ReduceSumTo": "reduce"}


@dataclass
class ExecutionPlan:
    graph: Graph
    order: list            # node ids to execute, ascending
    last_use: dict         # value id -> index in `order` of its last consumer (len(order) for outputs)
    recomputable: set


@dataclass
class MemoryPlan:
    offsets: dict          # value id -> byte offset in the arena (inputs and constants included)
    arena_bytes: int
    naive_bytes: int       # what one buffer per value would take


@dataclass
class Kernel:
    kind: str
    op: str
    out: int
    inputs: tuple
    attrs: dict


@dataclass
class LoweredPlan:
    exec_plan: ExecutionPlan
    memory: MemoryPlan
    kernels: list


def plan_execution(g: Graph) -> ExecutionPlan:
    if not g.outputs:
        raise GraphError("graph has no outputs")
    needed = set()
    stack = list(g.outputs)
    while stack:
        v = stack.pop()
        if v in needed:
            continue
        needed.add(v)
        stack.extend(g.nodes[v].inputs)
    order = sorted(needed)
    pos = {v: i for i, v in enumerate(order)}
    last = {v: pos[v] for v in order}
    for v in order:
        for i in g.nodes[v].inputs:
            last[i] = max(last[i], pos[v])
    for o in g.outputs:
        last[o] = len(order)
    recomputable = set()
    for v in order:
        if g.nodes[v].op == "Checkpoint":
            stack = list(g.nodes[v].inputs)
            while stack:
                x = stack.pop()
                if g.nodes[x].op in ("Input", "Constant") or x in recomputable:
                    continue
                recomputable.add(x)
                stack.extend(g.nodes[x].inputs)
    return ExecutionPlan(g, order, last, recomputable)


def _root(g: Graph, v: int) -> int:
    while g.nodes[v].op in _ALIAS:
        v = g.nodes[v].inputs[0]
    return v


def plan_memory(ep: ExecutionPlan) -> MemoryPlan:
    g = ep.graph
    size = {v: (_numel(g.nodes[v].shape) * 4 + ALIGN - 1) // ALIGN * ALIGN or ALIGN for v in ep.order}
    # an aliased value keeps its storage alive until its own last use
    last = dict(ep.last_use)
    for v in ep.order:
        r = _root(g, v)
        if r != v:
            last[r] = max(last[r], last[v])
    free: list = []          # (offset, bytes), address order
    top = 0
    offsets: dict = {}
    release_at: dict = {}
    # inputs and constants are written before the first kernel runs, whatever their position in the graph: they get
    # their storage up front (and give it back after their last use like every other value)
    feeds = [v for v in ep.order if g.nodes[v].op in ("Input", "Constant")]
    for v in feeds:
        offsets[v] = top
        top += size[v]
        release_at.setdefault(last[v], []).append(v)
    for i, v in enumerate(ep.order):
        r = _root(g, v)
        if r != v:
            offsets[v] = offsets[r]
        elif v in offsets:
            pass                     # a feed, placed above
        else:
            need = size[v]
            for k, (off, nb) in enumerate(free):
                if nb >= need:
                    offsets[v] = off
                    if nb > need:
                        free[k] = (off + need, nb - need)
                    else:
                        free.pop(k)
                    break
            else:
                offsets[v] = top
                top += need
            release_at.setdefault(last[v], []).append(v)
        for dead in release_at.pop(i, []):
            free.append((offsets[dead], size[dead]))
            free.sort()
            merged = []
            for off, nb in free:
                if merged and merged[-1][0] + merged[-1][1] == off:
                    merged[-1] = (merged[-1][0], merged[-1][1] + nb)
                else:
                    merged.append((off, nb))
            free = merged
    naive = sum(size[v] for v in ep.order if _root(g, v) == v)
    return MemoryPlan(offsets, top, naive)


def lower(g: Graph) -> LoweredPlan:
    ep = plan_execution(g)
    mp = plan_memory(ep)
    kernels = []
    for v in ep.order:
        n = g.nodes[v]
        if n.op in ("Input", "Constant"):
            continue
        if n.op in _ALIAS:
            kernels.append(Kernel("alias", n.op, v, n.inputs, {"shape": n.shape}))
            continue
        kernels.append(Kernel(_KIND[n.op], n.op, v, n.inputs, dict(n.attrs, shape=n.shape)))
    return LoweredPlan(ep, mp, kernels)

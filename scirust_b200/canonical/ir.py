"""Canonical tensor IR: a typed, append-only graph of fp32 tensor operations with shape inference.

Operations (scirust-tensor-ir/src/operation.rs:49-97): ``Input``, ``Constant``; ``Add Sub Mul Div`` (equal shapes),
``Scale{factor}``; ``Relu``, ``Exp``, ``Log``, ``ReluGrad`` (cotangent * 1(primal > 0)), ``ZerosLike``, ``OnesLike``;
``MatMul`` (rank 2), ``BatchMatMul`` (identical batch prefix, product over the last two axes: the lowering target of
``vmap(MatMul)``); ``Reshape{shape}``, ``Transpose{permutation}``, ``BroadcastTo{shape}`` (NumPy right-aligned),
``ReduceSumTo{shape}`` (sums the broadcast axes back); ``StopGradient`` (identity, barrier to differentiation) and
``Checkpoint`` (identity, marks intermediates as recomputable).

Transforms build new graphs: ``grad`` appends the reverse-mode program (the vector-Jacobian rules use only
operations of the same set, so a gradient graph can be differentiated again), ``vmap`` lifts a graph over a leading
batch axis (MatMul becomes BatchMatMul, broadcasts gain the axis).
"""
from __future__ import annotations

from dataclasses import dataclass, field


class GraphError(ValueError):
    pass


@dataclass(frozen=True)
class Value:
    id: int
    shape: tuple
    owner: int = 0          # identity of the graph that produced it: values of two graphs never mix


@dataclass
class Node:
    op: str
    inputs: tuple
    shape: tuple
    attrs: dict = field(default_factory=dict)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def _broadcastable(src, dst) -> bool:
    if len(src) > len(dst):
        return False
    for a, b in zip(reversed(src), reversed(dst)):
        if a != b and a != 1:
            return False
    return True


class Graph:
    def __init__(self):
        self.nodes: list = []
        self.inputs: dict = {}          # name -> value id
        self.constants: dict = {}       # value id -> nested list / tensor-like
        self.outputs: list = []

    # ---- construction
    def _push(self, op, inputs, shape, **attrs) -> Value:
        for v in inputs:
            if (not isinstance(v, Value) or v.owner != id(self) or v.id >= len(self.nodes)
                    or tuple(self.nodes[v.id].shape) != tuple(v.shape)):
                raise GraphError(f"{op}: operand does not belong to this graph")
        self.nodes.append(Node(op, tuple(v.id for v in inputs), tuple(int(s) for s in shape), attrs))
        return Value(len(self.nodes) - 1, tuple(int(s) for s in shape), id(self))

    def input(self, name: str, shape) -> Value:
        if name in self.inputs:
            raise GraphError(f"duplicate input {name!r}")
        if any(int(s) < 0 for s in shape):
            raise GraphError("negative dimension")
        v = self._push("Input", (), shape, name=name)
        self.inputs[name] = v.id
        return v

    def constant(self, data, shape) -> Value:
        v = self._push("Constant", (), shape)
        self.constants[v.id] = data
        return v

    def _same(self, op, a, b):
        if a.shape != b.shape:
            raise GraphError(f"{op}: shapes {a.shape} and {b.shape} differ (broadcast explicitly with BroadcastTo)")

    def add(self, a, b):
        self._same("Add", a, b)
        return self._push("Add", (a, b), a.shape)

    def sub(self, a, b):
        self._same("Sub", a, b)
        return self._push("Sub", (a, b), a.shape)

    def mul(self, a, b):
        self._same("Mul", a, b)
        return self._push("Mul", (a, b), a.shape)

    def div(self, a, b):
        self._same("Div", a, b)
        return self._push("Div", (a, b), a.shape)

    def scale(self, a, factor: float):
        return self._push("Scale", (a,), a.shape, factor=float(factor))

    def relu(self, a):
        return self._push("Relu", (a,), a.shape)

    def exp(self, a):
        return self._push("Exp", (a,), a.shape)

    def log(self, a):
        return self._push("Log", (a,), a.shape)

    def relu_grad(self, primal, cotangent):
        self._same("ReluGrad", primal, cotangent)
        return self._push("ReluGrad", (primal, cotangent), primal.shape)

    def zeros_like(self, a):
        return self._push("ZerosLike", (a,), a.shape)

    def ones_like(self, a):
        return self._push("OnesLike", (a,), a.shape)

    def matmul(self, a, b):
        if len(a.shape) != 2 or len(b.shape) != 2 or a.shape[1] != b.shape[0]:
            raise GraphError(f"MatMul: incompatible shapes {a.shape} x {b.shape}")
        return self._push("MatMul", (a, b), (a.shape[0], b.shape[1]))

    def batch_matmul(self, a, b):
        if len(a.shape) < 3 or len(a.shape) != len(b.shape) or a.shape[:-2] != b.shape[:-2] or a.shape[-1] != b.shape[-2]:
            raise GraphError(f"BatchMatMul: incompatible shapes {a.shape} x {b.shape}")
        return self._push("BatchMatMul", (a, b), a.shape[:-1] + (b.shape[-1],))

    def reshape(self, a, shape):
        if _numel(shape) != _numel(a.shape):
            raise GraphError(f"Reshape: {a.shape} -> {tuple(shape)} changes the element count")
        return self._push("Reshape", (a,), shape)

    def transpose(self, a, permutation):
        if sorted(permutation) != list(range(len(a.shape))):
            raise GraphError("Transpose: not a permutation of the axes")
        return self._push("Transpose", (a,), tuple(a.shape[p] for p in permutation), permutation=tuple(permutation))

    def broadcast_to(self, a, shape):
        if not _broadcastable(a.shape, tuple(shape)):
            raise GraphError(f"BroadcastTo: {a.shape} does not broadcast to {tuple(shape)}")
        return self._push("BroadcastTo", (a,), shape)

    def reduce_sum_to(self, a, shape):
        if not _broadcastable(tuple(shape), a.shape):
            raise GraphError(f"ReduceSumTo: {tuple(shape)} is not a broadcast source of {a.shape}")
        return self._push("ReduceSumTo", (a,), shape)

    def stop_gradient(self, a):
        return self._push("StopGradient", (a,), a.shape)

    def checkpoint(self, a):
        return self._push("Checkpoint", (a,), a.shape)

    def set_outputs(self, *values) -> None:
        self.outputs = [v.id for v in values]

    def value(self, vid: int) -> Value:
        return Value(vid, self.nodes[vid].shape, id(self))

    def signature(self) -> tuple:
        """Structural identity (used as the compilation-cache key)."""
        return (tuple((n.op, n.inputs, n.shape, tuple(sorted((k, v) for k, v in n.attrs.items()))) for n in self.nodes),
                tuple(self.outputs))


# ------------------------------------------------------------------------------------------- grad
def grad(g: Graph, output: Value, wrt) -> list:
    """Append the reverse-mode program of the scalar-or-tensor ``output`` (seeded with ones) to ``g`` and return the
    gradient values for ``wrt`` (zeros where there is no dependence)."""
    cot: dict = {output.id: g.ones_like(output)}

    def acc(vid, c):
        cot[vid] = c if vid not in cot else g.add(cot[vid], c)
    for vid in range(output.id, -1, -1):
        if vid not in cot:
            continue
        n, c = g.nodes[vid], cot[vid]
        ins = [g.value(i) for i in n.inputs]
        if n.op in ("Input", "Constant", "StopGradient", "ZerosLike", "OnesLike"):
            continue
        if n.op == "Add":
            acc(ins[0].id, c); acc(ins[1].id, c)
        elif n.op == "Sub":
            acc(ins[0].id, c); acc(ins[1].id, g.scale(c, -1.0))
        elif n.op == "Mul":
            acc(ins[0].id, g.mul(c, ins[1])); acc(ins[1].id, g.mul(c, ins[0]))
        elif n.op == "Div":
            acc(ins[0].id, g.div(c, ins[1]))
            acc(ins[1].id, g.scale(g.div(g.mul(c, g.value(vid)), ins[1]), -1.0))
        elif n.op == "Scale":
            acc(ins[0].id, g.scale(c, n.attrs["factor"]))
        elif n.op == "Relu":
            acc(ins[0].id, g.relu_grad(ins[0], c))
        elif n.op == "ReluGrad":
            acc(ins[1].id, g.relu_grad(ins[0], c))
        elif n.op == "Exp":
            acc(ins[0].id, g.mul(c, g.value(vid)))
        elif n.op == "Log":
            acc(ins[0].id, g.div(c, ins[0]))
        elif n.op == "MatMul":
            acc(ins[0].id, g.matmul(c, g.transpose(ins[1], (1, 0))))
            acc(ins[1].id, g.matmul(g.transpose(ins[0], (1, 0)), c))
        elif n.op == "BatchMatMul":
            r = len(ins[0].shape)
            sw = tuple(range(r - 2)) + (r - 1, r - 2)
            acc(ins[0].id, g.batch_matmul(c, g.transpose(ins[1], sw)))
            acc(ins[1].id, g.batch_matmul(g.transpose(ins[0], sw), c))
        elif n.op == "Reshape":
            acc(ins[0].id, g.reshape(c, ins[0].shape))
        elif n.op == "Transpose":
            p = n.attrs["permutation"]
            inv = tuple(p.index(i) for i in range(len(p)))
            acc(ins[0].id, g.transpose(c, inv))
        elif n.op == "BroadcastTo":
            acc(ins[0].id, g.reduce_sum_to(c, ins[0].shape))
        elif n.op == "ReduceSumTo":
            acc(ins[0].id, g.broadcast_to(c, ins[0].shape))
        elif n.op == "Checkpoint":
            acc(ins[0].id, c)
        else:
            raise GraphError(f"grad: no rule for {n.op}")
    return [cot[w.id] if w.id in cot else g.zeros_like(w) for w in wrt]


# ------------------------------------------------------------------------------------------- vmap
def vmap(g: Graph, batch: int, batched_inputs) -> Graph:
    """A new graph computing ``g`` independently for ``batch`` values of the inputs named in ``batched_inputs`` (they
    gain a leading axis of that size; every other input is shared)."""
    out = Graph()
    m: dict = {}
    is_b: dict = {}

    def lift(v_old):
        """The batched form of an old value (broadcast in if it is not batched)."""
        v = m[v_old]
        if is_b[v_old]:
            return v
        return out.broadcast_to(out.reshape(v, (1,) + v.shape), (batch,) + v.shape)
    for vid, n in enumerate(g.nodes):
        ins = list(n.inputs)
        anyb = any(is_b[i] for i in ins)
        if n.op == "Input":
            name = n.attrs["name"]
            b = name in batched_inputs
            m[vid] = out.input(name, ((batch,) if b else ()) + n.shape)
            is_b[vid] = b
            continue
        if n.op == "Constant":
            m[vid] = out.constant(g.constants[vid], n.shape)
            is_b[vid] = False
            continue
        if not anyb:
            args = [m[i] for i in ins]
            m[vid] = getattr(out, _METHOD[n.op])(*args, **_kwargs(n))
            is_b[vid] = False
            continue
        is_b[vid] = True
        if n.op == "MatMul":
            a, b = lift(ins[0]), lift(ins[1])
            m[vid] = out.batch_matmul(a, b)
        elif n.op == "BatchMatMul":
            m[vid] = out.batch_matmul(lift(ins[0]), lift(ins[1]))
        elif n.op == "Reshape":
            m[vid] = out.reshape(lift(ins[0]), (batch,) + n.shape)
        elif n.op == "Transpose":
            p = n.attrs["permutation"]
            m[vid] = out.transpose(lift(ins[0]), (0,) + tuple(x + 1 for x in p))
        elif n.op == "BroadcastTo":
            src = lift(ins[0])
            pad = len(n.shape) - (len(src.shape) - 1)
            src = out.reshape(src, (batch,) + (1,) * pad + src.shape[1:])
            m[vid] = out.broadcast_to(src, (batch,) + n.shape)
        elif n.op == "ReduceSumTo":
            src = lift(ins[0])
            pad = (len(src.shape) - 1) - len(n.shape)
            red = out.reduce_sum_to(src, (batch,) + (1,) * pad + n.shape)
            m[vid] = out.reshape(red, (batch,) + n.shape)
        else:
            args = [lift(i) for i in ins]
            m[vid] = getattr(out, _METHOD[n.op])(*args, **_kwargs(n))
    out.set_outputs(*[lift(o) if is_b[o] else m[o] for o in g.outputs])
    out.batched_outputs = [is_b[o] for o in g.outputs]
    return out


_METHOD = {"Add": "add", "Sub": "sub", "Mul": "mul", "Div": "div", "Scale": "scale", "Relu": "relu", "Exp": "exp",
           "Log": "log", "ReluGrad": "relu_grad", "ZerosLike": "zeros_like", "OnesLike": "ones_like",
           "MatMul": "matmul", "BatchMatMul": "batch_matmul", "Reshape": "reshape", "Transpose": "transpose",
           "BroadcastTo": "broadcast_to", "ReduceSumTo": "reduce_sum_to", "StopGradient": "stop_gradient",
           "Checkpoint": "checkpoint"}


def _kwargs(n: Node) -> dict:
    if n.op == "Scale":
        return {"factor": n.attrs["factor"]}
    if n.op == "Transpose":
        return {"permutation": n.attrs["permutation"]}
    if n.op in ("Reshape", "BroadcastTo", "ReduceSumTo"):
        return {"shape": n.shape}
    return {}

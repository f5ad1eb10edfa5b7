"""Operator-graph fusion pass of the canonical facade.

``fuse_elementwise`` rewrites an execution plan so that every maximal tree of element-wise operations whose inner
values have exactly one consumer (and are not graph outputs) becomes ONE ``fused_elementwise`` kernel: the inner
values never get storage (the memory plan is laid out over the fused order, so the arena shrinks), and the device
adapter runs the group as one generated CUDA kernel instead of one launch per operation.

The fused kernel is a straight-line program over registers, one element per thread. Bit-exactness is kept by
construction: every step is the same individually rounded IEEE operation as the unfused kernel (the generated source
uses ``__fadd_rn`` / ``__fsub_rn`` / ``__fmul_rn`` / ``__fdiv_rn``, which the compiler may neither contract into FMAs
nor reassociate), ``Relu`` passes NaN and positive words through untouched and turns everything else into +0, and
``ReluGrad`` gates the cotangent on ``primal > 0``. The CPU adapter interprets the same program with the canonical
CPU statements, so both adapters still agree word for word, fused or not.

Counterpart: the fusion stage of the reference's arena executor (scirust-compute: op graph -> fused groups -> arena),
rebuilt on the canonical kernels' rules (scirust-gpu/src/cuda_reference.rs:684-890).
"""
from __future__ import annotations

import ctypes as C
import struct

import torch

from ..ops import canonical as K
from .ir import Graph, _numel
from .plan import _ALIAS, _KIND, ExecutionPlan, Kernel, LoweredPlan, plan_execution, plan_memory

_FUSABLE = {"Add", "Sub", "Mul", "Div", "Scale", "Relu", "ReluGrad", "ZerosLike", "OnesLike"}


def find_groups(ep: ExecutionPlan) -> dict:
    """root value id -> member ids in execution order (root last). A producer joins its consumer's group when it is
    element-wise, has the consumer's shape, feeds nothing else and is not a graph output."""
    g = ep.graph
    uses: dict = {}
    for v in ep.order:
        for i in g.nodes[v].inputs:
            uses.setdefault(i, []).append(v)
    outputs = set(g.outputs)
    owner: dict = {}
    for v in reversed(ep.order):                     # consumers before producers
        n = g.nodes[v]
        if n.op not in _FUSABLE:
            continue
        root = owner.get(v, v)
        owner[v] = root
        for i in set(n.inputs):
            p = g.nodes[i]
            if (p.op in _FUSABLE and p.shape == n.shape and i not in outputs and i not in owner
                    and all(owner.get(u) == root for u in uses.get(i, []))):
                owner[i] = root
    groups: dict = {}
    for v in ep.order:
        if v in owner:
            groups.setdefault(owner[v], []).append(v)
    return {r: m for r, m in groups.items() if len(m) > 1}


def _program(g: Graph, members: list):
    """(external input ids, steps): step = (op, attrs, operands), operand = ('in', k) or ('tmp', j)."""
    ext: list = []
    slot = {}
    steps = []
    for v in members:
        n = g.nodes[v]
        ops_ = []
        for i in n.inputs:
            if i in slot:
                ops_.append(("tmp", slot[i]))
            else:
                if i not in ext:
                    ext.append(i)
                ops_.append(("in", ext.index(i)))
        slot[v] = len(steps)
        steps.append((n.op, {k: val for k, val in n.attrs.items()}, tuple(ops_)))
    return tuple(ext), tuple(steps)


def lower_fused(g: Graph) -> LoweredPlan:
    """``lower`` with the fusion pass: same outputs, fewer kernels, a smaller arena."""
    ep = plan_execution(g)
    groups = find_groups(ep)
    root_of = {m: r for r, ms in groups.items() for m in ms}
    inner = {m for r, ms in groups.items() for m in ms if m != r}
    progs = {r: _program(g, ms) for r, ms in groups.items()}
    order = [v for v in ep.order if v not in inner]
    pos = {v: i for i, v in enumerate(order)}
    last = {v: pos[v] for v in order}
    for v in order:
        ins = progs[v][0] if v in progs else g.nodes[v].inputs
        for i in ins:
            last[i] = max(last[i], pos[v])
    for o in g.outputs:
        last[o] = len(order)
    ep2 = ExecutionPlan(g, order, last, ep.recomputable)
    mp = plan_memory(ep2)
    kernels = []
    for v in order:
        n = g.nodes[v]
        if n.op in ("Input", "Constant"):
            continue
        if v in progs:
            ext, steps = progs[v]
            kernels.append(Kernel("fused_elementwise", "Fused", v, ext, {"program": steps, "shape": n.shape}))
        elif n.op in _ALIAS:
            kernels.append(Kernel("alias", n.op, v, n.inputs, {"shape": n.shape}))
        else:
            kernels.append(Kernel(_KIND[n.op], n.op, v, n.inputs, dict(n.attrs, shape=n.shape)))
    assert all(root_of.get(m, m) in pos for m in root_of)
    return LoweredPlan(ep2, mp, kernels)


# ------------------------------------------------------------------------------------------------ execution
def run_program_cpu(steps, ins):
    """Interpret a fused program with the canonical statements (one rounded operation per step)."""
    tmp = []

    def val(o):
        return ins[o[1]] if o[0] == "in" else tmp[o[1]]
    for op, attrs, operands in steps:
        a = val(operands[0]).contiguous()
        if op in ("Add", "Sub", "Mul", "Div"):
            r = K.run(op.lower(), a, val(operands[1]).contiguous())
        elif op == "Scale":
            r = K.run("scale", a, factor=attrs["factor"])
        elif op == "Relu":
            r = K.run("relu", a)
        elif op == "ReluGrad":
            r = torch.where(a > 0, val(operands[1]), torch.zeros_like(a))
        elif op == "ZerosLike":
            r = torch.zeros_like(a)
        else:
            r = torch.ones_like(a)
        tmp.append(r)
    return tmp[-1]


def cuda_source(steps, n_inputs: int, entry: str = "fused_elementwise") -> str:
    """CUDA C of one fused program: ``entry(out, in0, ..., n)``, one element per thread."""
    lines = [f'extern "C" __global__ void {entry}(float* __restrict__ out, '
             + "".join(f"const float* __restrict__ in{k}, " for k in range(n_inputs)) + "long long n) {",
             "  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;",
             "  if (i >= n) return;"]
    lines += [f"  const float x{k} = in{k}[i];" for k in range(n_inputs)]

    def val(o):
        return f"x{o[1]}" if o[0] == "in" else f"t{o[1]}"
    for j, (op, attrs, operands) in enumerate(steps):
        a = val(operands[0])
        b = val(operands[1]) if len(operands) > 1 else None
        if op == "Add":
            e = f"__fadd_rn({a}, {b})"
        elif op == "Sub":
            e = f"__fsub_rn({a}, {b})"
        elif op == "Mul":
            e = f"__fmul_rn({a}, {b})"
        elif op == "Div":
            e = f"__fdiv_rn({a}, {b})"
        elif op == "Scale":
            bits = struct.unpack("<I", struct.pack("<f", float(attrs["factor"])))[0]
            e = f"__fmul_rn({a}, __uint_as_float(0x{bits:08x}u))"
        elif op == "Relu":
            e = f"(({a} != {a}) || ({a} > 0.0f)) ? {a} : 0.0f"
        elif op == "ReluGrad":
            e = f"({a} > 0.0f) ? {b} : 0.0f"
        elif op == "ZerosLike":
            e = "0.0f"
        else:
            e = "1.0f"
        lines.append(f"  const float t{j} = {e};")
    lines += [f"  out[i] = t{len(steps) - 1};", "}"]
    return "\n".join(lines) + "\n"


class FusedKernelCache:
    """Compiles each distinct fused program once per device (NVRTC through the raw runtime, strict-IEEE options) and
    launches it on views of the plan's arena through the validated-binding path."""

    def __init__(self, device):
        from ..runtime import RawRuntime
        self.rt = RawRuntime(device.index or 0)
        self.kernels: dict = {}
        self.compiled = 0

    def launch(self, steps, arena: torch.Tensor, out_off: int, in_offs: list, n: int) -> None:
        from ..runtime import RawAccess, RawBinding, RawBuffer, RawLaunchConfig
        key = (repr(steps), len(in_offs))
        k = self.kernels.get(key)
        if k is None:
            k = self.kernels[key] = self.rt.compile(cuda_source(steps, len(in_offs)), "fused_elementwise")
            self.compiled += 1
        buf = RawBuffer(arena.numel() * 4, arena.view(torch.uint8))
        # bindings: the output span (write) and one read span per program input; the validator refuses the launch if
        # the memory plan ever let the output overlap an input
        binds = [RawBinding(buf, RawAccess.WRITE, out_off, n * 4)]
        binds += [RawBinding(buf, RawAccess.READ, off, n * 4) for off in in_offs]
        self.rt.launch(k, RawLaunchConfig(((n + 255) // 256, 1, 1), (256, 1, 1)), binds, scalars=[C.c_longlong(n)])

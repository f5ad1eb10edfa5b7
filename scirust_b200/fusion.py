"""Operator-graph fusion: find producer -> consumer chains whose intermediate never needs to reach memory and
run each as one fused kernel.

A graph is a list of nodes (``OpKind`` + input node ids + optional constant). ``FusionPipeline.fuse`` walks it in
topological order and grows a chain from each unvisited node along edges that (a) belong to a known pattern and
(b) are SAFE: the intermediate has exactly one consumer and is not a requested output, so dropping it changes
nothing observable. Chains of two or more nodes become ``FusedKernel`` records (kernel type, member nodes,
external inputs); ``execute`` evaluates a whole graph with or without the fused kernels, and the two must agree
(the test of the pass). Patterns: matmul -> {SiLU, ReLU, GELU}, matmul -> LayerNorm, matmul -> SiLU -> LayerNorm,
matmul -> scale, matmul -> matmul -> add (two-layer MLP with residual), LayerNorm -> activation, and the
sequential state-space scan (kept as one kernel, no memory saving claimed).

The fused bodies are ``scirust_b200.nn.fused_ops``: on a B200 the product is the tcgen05 GEMM and the tail is applied
to its output tile rows. Reference counterpart: scirust-fusion/src/{graph,patterns,fusion,kernel}.rs (``OpGraph``,
``FusionPatterns``, ``FusionPipeline::fuse``, ``FusedKernel::execute``), which fuses along every pattern edge
without the single-consumer check.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .nn import fused_ops as FO


class OpKind(enum.Enum):
    INPUT = "input"
    MATMUL = "matmul"
    LINEAR = "linear"          # inputs: x, w, bias
    RELU = "relu"
    SILU = "silu"
    GELU = "gelu"
    SIGMOID = "sigmoid"
    TANH = "tanh"
    LAYERNORM = "layernorm"    # inputs: x, gamma, beta; constant: eps
    RMSNORM = "rmsnorm"        # inputs: x, weight; constant: eps
    ADD = "add"
    SUB = "sub"
    MUL = "mul"
    DIV = "div"
    SCALE = "scale"            # constant: factor
    SSM_STEP = "ssm_step"      # inputs: x, a, b, c (diagonal scan over the whole sequence)
    SOFTMAX = "softmax"
    TRANSPOSE = "transpose"


_MM = (OpKind.MATMUL, OpKind.LINEAR)
_ACT = (OpKind.RELU, OpKind.SILU, OpKind.GELU, OpKind.SIGMOID, OpKind.TANH)


class KernelType(enum.Enum):
    MATMUL_SILU = "matmul_silu"
    MATMUL_RELU = "matmul_relu"
    MATMUL_GELU = "matmul_gelu"
    MATMUL_LAYERNORM = "matmul_layernorm"
    MATMUL_SILU_LAYERNORM = "matmul_silu_layernorm"
    MATMUL_SCALE = "matmul_scale"
    TWO_LAYER_MLP = "two_layer_mlp"
    LAYERNORM_ACTIVATION = "layernorm_activation"
    SSM_SCAN = "ssm_scan"


@dataclass(frozen=True)
class FusionPattern:
    name: str
    kernel: KernelType
    ops: tuple                 # tuple of tuples of OpKind (alternatives per position)
    memory_savings: float      # percent of intermediate traffic removed


PATTERNS = (
    FusionPattern("matmul_silu_layernorm", KernelType.MATMUL_SILU_LAYERNORM, (_MM, (OpKind.SILU,), (OpKind.LAYERNORM,)), 66.0),
    FusionPattern("two_layer_mlp", KernelType.TWO_LAYER_MLP, (_MM, _MM, (OpKind.ADD,)), 66.0),
    FusionPattern("matmul_silu", KernelType.MATMUL_SILU, (_MM, (OpKind.SILU,)), 50.0),
    FusionPattern("matmul_relu", KernelType.MATMUL_RELU, (_MM, (OpKind.RELU,)), 50.0),
    FusionPattern("matmul_gelu", KernelType.MATMUL_GELU, (_MM, (OpKind.GELU,)), 50.0),
    FusionPattern("matmul_layernorm", KernelType.MATMUL_LAYERNORM, (_MM, (OpKind.LAYERNORM,)), 50.0),
    FusionPattern("matmul_scale", KernelType.MATMUL_SCALE, (_MM, (OpKind.SCALE,)), 50.0),
    FusionPattern("layernorm_activation", KernelType.LAYERNORM_ACTIVATION, ((OpKind.LAYERNORM,), _ACT), 50.0),
    FusionPattern("ssm_scan", KernelType.SSM_SCAN, ((OpKind.SSM_STEP,), (OpKind.SSM_STEP,)), 0.0),
)


def match_sequence(kinds) -> FusionPattern | None:
    """The pattern whose positions match ``kinds`` exactly (longest patterns are listed first)."""
    for p in PATTERNS:
        if len(p.ops) == len(kinds) and all(k in alt for k, alt in zip(kinds, p.ops)):
            return p
    return None


def is_prefix(kinds) -> bool:
    """Whether ``kinds`` starts some pattern (so the chain may still grow into a full match)."""
    return any(len(p.ops) >= len(kinds) and all(k in alt for k, alt in zip(kinds, p.ops)) for p in PATTERNS)


def high_gain_patterns(threshold: float):
    return [p.name for p in PATTERNS if p.memory_savings >= threshold]


@dataclass
class Node:
    kind: OpKind
    inputs: tuple = ()
    constant: object = None


@dataclass
class FusedKernel:
    kernel_type: KernelType
    group: list                 # member node ids, producer first
    inputs: list                # external node ids, in first-use order
    output: int                 # node id whose value the kernel produces
    constants: dict = field(default_factory=dict)

    def op_count(self) -> int:
        return len(self.group)


class OpGraph:
    def __init__(self):
        self.nodes: list[Node] = []
        self.outputs: set[int] = set()

    def add_input(self) -> int:
        self.nodes.append(Node(OpKind.INPUT))
        return len(self.nodes) - 1

    def add(self, kind: OpKind, *inputs: int, constant=None) -> int:
        for i in inputs:
            if not 0 <= i < len(self.nodes):
                raise ValueError(f"OpGraph.add: input {i} does not exist yet")
        self.nodes.append(Node(kind, tuple(inputs), constant))
        return len(self.nodes) - 1

    def mark_output(self, idx: int) -> None:
        self.outputs.add(idx)

    def __len__(self):
        return len(self.nodes)

    def topo_order(self) -> list[int]:
        """Nodes are appended after their inputs, so insertion order is topological; verified here."""
        for i, n in enumerate(self.nodes):
            if any(j >= i for j in n.inputs):
                raise ValueError("OpGraph: cycle or forward reference")
        return list(range(len(self.nodes)))

    def consumers(self, idx: int) -> list[int]:
        return [i for i, n in enumerate(self.nodes) if idx in n.inputs]

    def sinks(self) -> set[int]:
        used = {j for n in self.nodes for j in n.inputs}
        return {i for i in range(len(self.nodes)) if i not in used} | self.outputs


class FusionPipeline:
    def fuse(self, graph: OpGraph) -> list[FusedKernel]:
        graph.topo_order()
        keep = graph.sinks()
        visited = [False] * len(graph)
        kernels = []
        for root in range(len(graph)):
            if visited[root] or graph.nodes[root].kind == OpKind.INPUT:
                continue
            chain = [root]
            while True:
                last = chain[-1]
                cons = graph.consumers(last)
                if len(cons) != 1 or last in keep:
                    break                                  # the intermediate is observable: do not swallow it
                nxt = cons[0]
                kinds = [graph.nodes[i].kind for i in chain] + [graph.nodes[nxt].kind]
                feeds_first = graph.nodes[nxt].inputs[0] == last or graph.nodes[nxt].kind == OpKind.ADD
                if visited[nxt] or not is_prefix(kinds) or not feeds_first:
                    break
                chain.append(nxt)
            # shrink to the longest prefix that is a complete pattern
            while len(chain) >= 2 and match_sequence([graph.nodes[i].kind for i in chain]) is None:
                chain.pop()
            if len(chain) >= 2:
                pat = match_sequence([graph.nodes[i].kind for i in chain])
                for i in chain:
                    visited[i] = True
                ext = []
                for i in chain:
                    for j in graph.nodes[i].inputs:
                        if j not in chain and j not in ext:
                            ext.append(j)
                consts = {i: graph.nodes[i].constant for i in chain if graph.nodes[i].constant is not None}
                kernels.append(FusedKernel(pat.kernel, chain, ext, chain[-1], consts))
        return kernels


# ---------------------------------------------------------------- evaluation

def _ssm_scan(x, a, b, c):
    """h <- a*h + b*x[t]; y[t] = sum(c*h): ascending-state reduction, sequential in t."""
    h = torch.zeros_like(a, dtype=torch.float32)
    y = torch.empty_like(x, dtype=torch.float32)
    for t in range(x.numel()):
        h = a * h + b * x[t]
        y[t] = (c * h).sum()
    return y


def _eval_node(n: Node, vals):
    a = [vals[i] for i in n.inputs]
    k = n.kind
    if k == OpKind.MATMUL:
        return a[0].float() @ a[1].float()
    if k == OpKind.LINEAR:
        return a[0].float() @ a[1].float() + (a[2].float().reshape(1, -1) if len(a) > 2 else 0.0)
    if k == OpKind.RELU:
        return a[0].clamp_min(0)
    if k == OpKind.SILU:
        return F.silu(a[0])
    if k == OpKind.GELU:
        return FO.gelu_tanh(a[0])
    if k == OpKind.SIGMOID:
        return torch.sigmoid(a[0])
    if k == OpKind.TANH:
        return torch.tanh(a[0])
    if k == OpKind.LAYERNORM:
        return FO._layernorm(a[0].float(), a[1], a[2], 1e-5 if n.constant is None else float(n.constant))
    if k == OpKind.RMSNORM:
        eps = 1e-5 if n.constant is None else float(n.constant)
        return a[0] * torch.rsqrt((a[0] ** 2).mean(-1, keepdim=True) + eps) * a[1]
    if k == OpKind.ADD:
        return a[0] + a[1]
    if k == OpKind.SUB:
        return a[0] - a[1]
    if k == OpKind.MUL:
        return a[0] * a[1]
    if k == OpKind.DIV:
        return a[0] / a[1]
    if k == OpKind.SCALE:
        return a[0] * float(n.constant if n.constant is not None else 1.0)
    if k == OpKind.SSM_STEP:
        return _ssm_scan(*a) if len(a) == 4 else a[0]
    if k == OpKind.SOFTMAX:
        return torch.softmax(a[0], -1)
    if k == OpKind.TRANSPOSE:
        return a[0].t()
    raise ValueError(f"cannot evaluate {k}")


def _act(kind: OpKind, y):
    return {OpKind.RELU: lambda v: v.clamp_min(0), OpKind.SILU: F.silu, OpKind.SIGMOID: torch.sigmoid,
            OpKind.TANH: torch.tanh,
            OpKind.GELU: FO.gelu_tanh}[kind](y)


def run_kernel(kernel: FusedKernel, graph: OpGraph, vals):
    """Value of ``kernel.output`` from the external inputs in ``vals``."""
    nodes = [graph.nodes[i] for i in kernel.group]
    head = nodes[0]
    hv = [vals[i] for i in head.inputs]
    bias = hv[2] if head.kind == OpKind.LINEAR and len(hv) > 2 else None
    kt = kernel.kernel_type
    if kt == KernelType.MATMUL_SILU:
        return FO.matmul_silu(hv[0], hv[1], bias)
    if kt == KernelType.MATMUL_RELU:
        return FO.matmul_relu(hv[0], hv[1], bias)
    if kt == KernelType.MATMUL_GELU:
        return FO.matmul_gelu(hv[0], hv[1], bias)
    if kt == KernelType.MATMUL_SCALE:
        return FO.matmul_scale(hv[0], hv[1], float(nodes[1].constant if nodes[1].constant is not None else 1.0)) \
            if bias is None else (FO._affine(hv[0], hv[1], bias) * float(nodes[1].constant or 1.0))
    if kt in (KernelType.MATMUL_LAYERNORM, KernelType.MATMUL_SILU_LAYERNORM):
        ln = nodes[-1]
        gamma, beta = vals[ln.inputs[1]], vals[ln.inputs[2]]
        eps = 1e-5 if ln.constant is None else float(ln.constant)
        y = FO._affine(hv[0], hv[1], bias)
        if kt == KernelType.MATMUL_SILU_LAYERNORM:
            y = F.silu(y)
        return FO._layernorm(y, gamma, beta, eps)
    if kt == KernelType.TWO_LAYER_MLP:
        second, add = nodes[1], nodes[2]
        sv = [vals[i] if i != kernel.group[0] else None for i in second.inputs]
        h = FO._affine(hv[0], hv[1], bias)
        b2 = sv[2] if second.kind == OpKind.LINEAR and len(sv) > 2 else None
        y = FO._affine(h, sv[1], b2)
        other = [i for i in add.inputs if i != kernel.group[1]]
        return y + (vals[other[0]] if other else y)
    if kt == KernelType.LAYERNORM_ACTIVATION:
        ln = nodes[0]
        eps = 1e-5 if ln.constant is None else float(ln.constant)
        return _act(nodes[1].kind, FO._layernorm(hv[0].float(), hv[1], hv[2], eps))
    if kt == KernelType.SSM_SCAN:
        y = _eval_node(nodes[0], vals)
        for n in nodes[1:]:
            ins = [y] + [vals[i] for i in n.inputs[1:]]
            y = _ssm_scan(*ins) if len(ins) == 4 else y
        return y
    raise ValueError(f"no body for {kt}")


def execute(graph: OpGraph, feeds: dict, fuse: bool = True) -> dict:
    """Evaluate every sink of ``graph``. ``feeds`` maps input node ids to tensors. With ``fuse`` the chains found
    by ``FusionPipeline`` run as single kernels and their interior values are never produced."""
    kernels = FusionPipeline().fuse(graph) if fuse else []
    by_output = {k.output: k for k in kernels}
    interior = {i for k in kernels for i in k.group[:-1]}
    vals = dict(feeds)
    for i, n in enumerate(graph.nodes):
        if n.kind == OpKind.INPUT:
            if i not in vals:
                raise KeyError(f"execute: input node {i} has no feed")
            continue
        if i in interior:
            continue
        vals[i] = run_kernel(by_output[i], graph, vals) if i in by_output else _eval_node(n, vals)
    return {i: vals[i] for i in sorted(graph.sinks())}

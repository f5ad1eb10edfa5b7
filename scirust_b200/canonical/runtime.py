"""Sessions that execute lowered canonical plans, and the adapter conformance suite.

* ``ReferencePlanRuntime``: runs a ``LoweredPlan`` kernel by kernel inside ONE arena laid out by the memory plan
  (so buffer reuse is exercised, not just computed). On CPU every kernel is the plain fp32 statement; on a CUDA device
  the element-wise and permute kernels are the bit-exact canonical kernels (``ops/canonical.py``), matmul runs with
  a fixed k order, and ``Exp`` / ``Log`` are refused, as the device adapter of the reference refuses them.
* ``ReferenceJitSession``: lowers a graph once per structural signature and caches the plan.
* ``ReferenceSpmdSession``: runs a graph once per logical rank of a ``DeviceMesh`` on the rank's shards of the inputs
  (``PartitionSpec`` per input), reassembles sharded outputs and checks that outputs declared replicated are
  bit-identical on every rank; communication-free, like the reference's logical SPMD layer.
* ``conformance_cases`` / ``run_conformance``: graphs with known answers that every adapter must reproduce bit for
  bit; the device test runs them on the GPU against the CPU results.

Counterparts: scirust-tensor-runtime/src/lib.rs:21-46 (the three sessions), spmd.rs:59-110,
scirust-gpu/src/compute_conformance.rs (suite), scirust-gpu/src/cuda_reference.rs (device adapter rules).
"""
from __future__ import annotations

import torch

from ..ops import canonical as K
from ..parallel.mesh import DeviceMesh, PartitionSpec, plan_sharding
from .ir import Graph, GraphError, _numel
from .plan import LoweredPlan, lower


class ReferencePlanRuntime:
    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self._fused = None          # compiled fused element-wise kernels of this device

    def _view(self, arena, plan: LoweredPlan, vid: int):
        shape = plan.exec_plan.graph.nodes[vid].shape
        off = plan.memory.offsets[vid] // 4
        return arena[off:off + _numel(shape)].view(shape)

    def run(self, plan: LoweredPlan, feeds: dict) -> list:
        g = plan.exec_plan.graph
        arena = torch.zeros(max(plan.memory.arena_bytes // 4, 1), dtype=torch.float32, device=self.device)
        for name, vid in g.inputs.items():
            if vid not in plan.memory.offsets:
                continue
            if name not in feeds:
                raise GraphError(f"missing input {name!r}")
            t = torch.as_tensor(feeds[name], dtype=torch.float32)
            if tuple(t.shape) != tuple(g.nodes[vid].shape):
                raise GraphError(f"input {name!r}: shape {tuple(t.shape)} != {g.nodes[vid].shape}")
            self._view(arena, plan, vid).copy_(t)
        for vid, data in g.constants.items():
            if vid in plan.memory.offsets:
                self._view(arena, plan, vid).copy_(torch.as_tensor(data, dtype=torch.float32).reshape(g.nodes[vid].shape))
        for k in plan.kernels:
            if k.kind == "alias":
                continue
            if k.kind == "fused_elementwise" and self.device.type == "cuda":
                from .fusion import FusedKernelCache
                if self._fused is None:
                    self._fused = FusedKernelCache(self.device)
                self._fused.launch(k.attrs["program"], arena, plan.memory.offsets[k.out],
                                   [plan.memory.offsets[i] for i in k.inputs], _numel(k.attrs["shape"]))
                continue
            ins = [self._view(arena, plan, i) for i in k.inputs]
            out = self._view(arena, plan, k.out)
            out.copy_(self._kernel(k, ins))
        return [self._view(arena, plan, o).clone() for o in g.outputs]

    def _kernel(self, k, ins):
        dev = self.device.type == "cuda"
        op = k.op
        if k.kind == "fused_elementwise":
            from .fusion import run_program_cpu
            return run_program_cpu(k.attrs["program"], ins)
        if k.kind == "elementwise":
            if op in ("Add", "Sub", "Mul", "Div"):
                return K.run(op.lower(), ins[0].contiguous(), ins[1].contiguous())
            if op == "Scale":
                return K.run("scale", ins[0].contiguous(), factor=k.attrs["factor"])
            if op == "Relu":
                return K.run("relu", ins[0].contiguous())
            if op == "ReluGrad":
                # cotangent where the primal is strictly positive, +0 elsewhere (NaN primal: +0)
                return torch.where(ins[0] > 0, ins[1], torch.zeros_like(ins[1]))      # a select, never inf * 0
            if op == "ZerosLike":
                return torch.zeros_like(ins[0])
            return torch.ones_like(ins[0])
        if k.kind == "transcendental":
            if dev:
                raise K.Unsupported(f"{op} has no bit-reproducible device implementation and is not executed")
            return torch.exp(ins[0]) if op == "Exp" else torch.log(ins[0])
        if k.kind == "permute":
            return K.run("permute", ins[0].contiguous(), perm=list(k.attrs["permutation"]))
        if k.kind in ("matmul", "batch_matmul"):
            return _matmul_fixed_order(ins[0], ins[1])
        if k.kind == "broadcast":
            return ins[0].broadcast_to(k.attrs["shape"]).contiguous()
        if k.kind == "reduce":
            return _reduce_sum_to(ins[0], k.attrs["shape"])
        raise GraphError(f"no kernel for {k.kind}")


def _matmul_fixed_order(a, b):
    """Product over the last two axes with the contraction index walked in ascending order, one rounded fp32
    multiply-add per step (no split, no reassociation): the same bits on every adapter."""
    out = torch.zeros(a.shape[:-1] + (b.shape[-1],), dtype=torch.float32, device=a.device)
    for kk in range(a.shape[-1]):
        out = out + a[..., :, kk:kk + 1] * b[..., kk:kk + 1, :]
    return out


def _reduce_sum_to(x, shape):
    """Sum the broadcast axes in ascending index order (slice by slice, never a tree)."""
    shape = tuple(shape)
    lead = x.dim() - len(shape)
    for _ in range(lead):
        acc = x[0].clone()
        for i in range(1, x.shape[0]):
            acc = acc + x[i]
        x = acc
    for ax, s in enumerate(shape):
        if s == 1 and x.shape[ax] != 1:
            acc = x.select(ax, 0).clone()
            for i in range(1, x.shape[ax]):
                acc = acc + x.select(ax, i)
            x = acc.unsqueeze(ax)
    return x


class ReferenceJitSession:
    def __init__(self, device="cpu", fuse: bool = False):
        self.runtime = ReferencePlanRuntime(device)
        self.cache: dict = {}
        self.compilations = 0
        self.fuse = fuse            # run the element-wise fusion pass (canonical/fusion.py) when lowering

    def run(self, g: Graph, feeds: dict) -> list:
        key = g.signature()
        plan = self.cache.get(key)
        if plan is None:
            if self.fuse:
                from .fusion import lower_fused
                plan = lower_fused(g)
            else:
                plan = lower(g)
            self.cache[key] = plan
            self.compilations += 1
        return self.runtime.run(plan, feeds)


class ReferenceSpmdSession:
    def __init__(self, mesh: DeviceMesh, device="cpu"):
        self.mesh = mesh
        self.jit = ReferenceJitSession(device)

    def run(self, build_local, feeds: dict, in_specs: dict, out_specs: list) -> list:
        """``build_local(local_shapes) -> Graph`` builds the per-rank graph from the local input shapes;
        ``in_specs[name]`` / ``out_specs[i]`` are ``PartitionSpec``s (``None`` dims = replicated)."""
        plans = {n: plan_sharding(tuple(torch.as_tensor(feeds[n]).shape), in_specs[n], self.mesh) for n in feeds}
        per_rank = []
        for r in self.mesh.ranks():
            local = {}
            for n, t in feeds.items():
                sl = plans[n][r]
                local[n] = torch.as_tensor(t, dtype=torch.float32)[tuple(sl)]
            g = build_local({n: tuple(v.shape) for n, v in local.items()})
            per_rank.append(self.jit.run(g, local))
        outs = []
        for i, spec in enumerate(out_specs):
            parts = [res[i] for res in per_rank]
            if all(d is None for d in spec.dims):
                for p in parts[1:]:
                    if not torch.equal(p.view(torch.int32), parts[0].view(torch.int32)):
                        raise GraphError(f"output {i} is declared replicated but differs between ranks")
                outs.append(parts[0])
                continue
            full_shape = list(parts[0].shape)
            for ax, name in enumerate(spec.dims):
                if name is not None:
                    full_shape[ax] *= self.mesh.axis_size(name)
            full = torch.zeros(full_shape)
            for r, slices in enumerate(plan_sharding(tuple(full_shape), spec, self.mesh)):
                full[tuple(slices)] = parts[r]
            outs.append(full)
        return outs


# ---------------------------------------------------------------------------------------- conformance
def conformance_cases():
    """(name, graph, feeds) triples covering every kernel kind the device adapter executes."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 7, generator=g)
    y = torch.randn(5, 7, generator=g)
    x[0, 0], x[0, 1], y[0, 2] = float("nan"), -0.0, float("inf")
    w = torch.randn(7, 3, generator=g)
    cases = []
    g1 = Graph()
    a, b = g1.input("x", (5, 7)), g1.input("y", (5, 7))
    t = g1.div(g1.mul(g1.add(a, b), g1.sub(a, b)), g1.scale(b, 0.3))
    g1.set_outputs(g1.relu(t), g1.relu_grad(a, b))
    cases.append(("elementwise", g1, {"x": x, "y": y}))
    g2 = Graph()
    a, ww = g2.input("x", (5, 7)), g2.input("w", (7, 3))
    mm = g2.matmul(g2.relu(a), ww)
    g2.set_outputs(g2.transpose(mm, (1, 0)), g2.reshape(mm, (3, 5)))
    cases.append(("matmul_permute_reshape", g2, {"x": torch.nan_to_num(x), "w": w}))
    g3 = Graph()
    bias = g3.input("b", (7,))
    a = g3.input("x", (5, 7))
    s = g3.add(a, g3.broadcast_to(bias, (5, 7)))
    g3.set_outputs(g3.reduce_sum_to(s, (7,)), g3.reduce_sum_to(s, (5, 1)))
    cases.append(("broadcast_reduce", g3, {"x": torch.nan_to_num(x), "b": torch.randn(7, generator=g)}))
    g4 = Graph()
    a = g4.input("x", (2, 5, 7))
    bb = g4.input("y", (2, 7, 4))
    g4.set_outputs(g4.batch_matmul(a, bb))
    cases.append(("batch_matmul", g4, {"x": torch.randn(2, 5, 7, generator=g), "y": torch.randn(2, 7, 4, generator=g)}))
    return cases


def run_conformance(device="cpu", fuse: bool = False) -> dict:
    """name -> list of output tensors (on the host) for every conformance case on ``device``."""
    sess = ReferenceJitSession(device, fuse=fuse)
    return {name: [o.cpu() for o in sess.run(g, feeds)] for name, g, feeds in conformance_cases()}

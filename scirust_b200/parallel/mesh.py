"""Logical device meshes and SPMD sharding (scirust-tensor-ir/src/shard.rs:38-470,
scirust-tensor-runtime/src/spmd.rs:59-110): ``DeviceMesh`` names the axes of a grid of ranks,
``PartitionSpec`` says which tensor dimension is split over which mesh axis, ``plan_sharding``
computes each rank's slice, and ``shard_map`` runs a function once per logical rank on its local
shards, reassembling sharded outputs and checking that replicated outputs agree on every rank.
Like the reference's, this layer is communication-free and runs on host tensors; the same
``DeviceMesh`` also names the axes used by the GPU process groups (``"dp"``, ``"tp"``)."""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import torch


class ShardingError(ValueError):
    pass


@dataclass(frozen=True)
class DeviceMesh:
    axis_names: tuple
    shape: tuple

    def __post_init__(self):
        if len(self.axis_names) != len(self.shape) or any(s < 1 for s in self.shape):
            raise ShardingError("mesh axis names and shape must match and be positive")
        if len(set(self.axis_names)) != len(self.axis_names):
            raise ShardingError("duplicate mesh axis name")

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def axis_size(self, name: str) -> int:
        return self.shape[self.axis_names.index(name)]

    def coords(self, rank: int) -> dict:
        out, r = {}, rank
        for name, s in zip(reversed(self.axis_names), reversed(self.shape)):
            out[name] = r % s
            r //= s
        return out

    def ranks(self):
        return range(self.size)

    def group_ranks(self, axis: str, rank: int) -> list:
        """Ranks that differ from ``rank`` only along ``axis`` (a process group of that axis)."""
        me = self.coords(rank)
        return [r for r in self.ranks() if all(v == me[k] for k, v in self.coords(r).items() if k != axis)]

    def process_groups(self, rank: int | None = None) -> dict:
        """``torch.distributed`` groups of the calling rank, one per mesh axis (``{"dp": group, "tp": group}``). Every
        rank of the job must call this, in the same order: all groups of all axes are created collectively, each rank
        keeps the ones it belongs to. The last axis varies fastest, so with ``("dp", "tp")`` a tensor-parallel group is
        a run of consecutive ranks: the GPUs that share an NVSwitch domain on one node."""
        import torch.distributed as dist
        if dist.get_world_size() != self.size:
            raise ShardingError(f"mesh of {self.size} ranks on a job of {dist.get_world_size()}")
        rank = dist.get_rank() if rank is None else rank
        mine = {}
        for axis in self.axis_names:
            seen = set()
            for r in self.ranks():
                members = tuple(self.group_ranks(axis, r))
                if members in seen:
                    continue
                seen.add(members)
                g = dist.new_group(list(members))
                if rank in members:
                    mine[axis] = g
        return mine


@dataclass(frozen=True)
class PartitionSpec:
    """One entry per tensor dimension: a mesh axis name or None (replicated along that dimension)."""
    dims: tuple

    def __init__(self, *dims):
        object.__setattr__(self, "dims", tuple(dims))


def plan_sharding(shape, spec: PartitionSpec, mesh: DeviceMesh) -> list:
    """For every rank, the tuple of slices of its local shard."""
    if len(spec.dims) != len(shape):
        raise ShardingError(f"spec has {len(spec.dims)} entries for a rank-{len(shape)} tensor")
    used = [d for d in spec.dims if d is not None]
    if len(set(used)) != len(used):
        raise ShardingError("a mesh axis may shard at most one tensor dimension")
    for d, axis in zip(shape, spec.dims):
        if axis is not None:
            if axis not in mesh.axis_names:
                raise ShardingError(f"unknown mesh axis {axis!r}")
            if d % mesh.axis_size(axis):
                raise ShardingError(f"dimension {d} does not divide by mesh axis {axis!r} ({mesh.axis_size(axis)})")
    plans = []
    for r in mesh.ranks():
        c = mesh.coords(r)
        sl = []
        for d, axis in zip(shape, spec.dims):
            if axis is None:
                sl.append(slice(0, d))
            else:
                per = d // mesh.axis_size(axis)
                sl.append(slice(c[axis] * per, (c[axis] + 1) * per))
        plans.append(tuple(sl))
    return plans


def shard(t: torch.Tensor, spec: PartitionSpec, mesh: DeviceMesh) -> list:
    return [t[p].clone() for p in plan_sharding(tuple(t.shape), spec, mesh)]


def unshard(shards, global_shape, spec: PartitionSpec, mesh: DeviceMesh) -> torch.Tensor:
    out = torch.zeros(tuple(global_shape), dtype=shards[0].dtype)
    for s, p in zip(shards, plan_sharding(tuple(global_shape), spec, mesh)):
        out[p] = s
    return out


def shard_map(fn, mesh: DeviceMesh, in_specs, out_specs, *args):
    """Run ``fn(*local_args)`` once per logical rank. ``out_specs`` entries that are fully replicated
    must produce identical tensors on every rank (checked); sharded outputs are reassembled."""
    if len(in_specs) != len(args):
        raise ShardingError("one input spec per argument is required")
    locals_per_rank = [[] for _ in mesh.ranks()]
    for a, sp in zip(args, in_specs):
        for r, s in enumerate(shard(a, sp, mesh)):
            locals_per_rank[r].append(s)
    outs = [fn(*la) for la in locals_per_rank]
    single = not isinstance(outs[0], (tuple, list))
    if single:
        outs = [(o,) for o in outs]
        out_specs = (out_specs,)
    results = []
    for i, sp in enumerate(out_specs):
        per_rank = [o[i] for o in outs]
        if all(d is None for d in sp.dims):
            for r, t in enumerate(per_rank[1:], 1):
                if not torch.equal(t, per_rank[0]):
                    raise ShardingError(f"replicated output {i} diverges on rank {r}")
            results.append(per_rank[0])
        else:
            gshape = list(per_rank[0].shape)
            for d, axis in enumerate(sp.dims):
                if axis is not None:
                    gshape[d] *= mesh.axis_size(axis)
            results.append(unshard(per_rank, gshape, sp, mesh))
    return results[0] if single else tuple(results)

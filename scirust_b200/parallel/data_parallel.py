"""Data-parallel gradient reduction over the model's flat bf16 gradient buffer.

Two reducers with the same contract ``reduce(flat_grad) -> (grad_tensor, scale)``:

* ``nccl``  - the baseline: one NCCL all-reduce (sum) of the bf16 buffer; the 1/world mean is
  folded into the optimizer's gradient scale.
* ``fused`` - the product path (parallel/fused_allreduce.py): peers' bf16 buckets are pulled over
  NVLink by a hand-written kernel that sums them in fixed rank order in fp32, applies 1/world and
  writes the fp32 gradient the optimizer consumes - cast, scale and reduction in one pass,
  bitwise-stable at a fixed world size like the reference's rank-ordered host all-reduce
  (scirust-core/src/distributed.rs:96-167).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def make_grad_reducer(model, group, kind: str = "fused"):
    world = dist.get_world_size(group)
    if world == 1:
        return None
    if kind == "fused":
        from .fused_allreduce import FusedGradAllReduce
        return FusedGradAllReduce(model, group)

    def nccl_reduce(flat_grad):
        dist.all_reduce(flat_grad, op=dist.ReduceOp.SUM, group=group)
        return flat_grad, 1.0 / world
    return nccl_reduce

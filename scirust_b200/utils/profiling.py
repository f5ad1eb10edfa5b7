"""Tracing and timing helpers: NVTX ranges per layer / phase (visible to Nsight tools), CUDA-event
timers that return the maximum over ranks, and a per-step launch counter. The reference has no
tracing framework - only wall-clock throughput lines and advice to run an external profiler
(scirust-sciagent/THOR_PRODUCTION_BENCH.md:67-84); these helpers make the same information
available in-process."""
from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class DeviceTimer:
    """``with DeviceTimer() as t: ...`` then ``t.ms`` (max over the ranks of ``group`` if given)."""

    def __init__(self, group=None, sync_ranks: bool = True):
        self.group, self.sync_ranks, self.ms = group, sync_ranks, None

    def __enter__(self):
        import torch.distributed as dist
        if self.sync_ranks and dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.group)
        torch.cuda.synchronize()
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.e0.record()
        return self

    def __exit__(self, *exc):
        import torch.distributed as dist
        self.e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([self.e0.elapsed_time(self.e1)], device="cuda")
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=self.group)
        self.ms = float(ms)
        return False


def launch_counter():
    from ..ops import gemm
    return gemm.launch_count


def annotate_model(model):
    """Wrap each decoder layer's forward in an NVTX range named after its index."""
    for i, layer in enumerate(getattr(model, "layers", [])):
        fwd = layer.forward

        def wrapped(*a, _f=fwd, _i=i, **kw):
            with nvtx_range(f"layer{_i}"):
                return _f(*a, **kw)
        layer.forward = wrapped
    return model

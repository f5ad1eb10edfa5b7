"""Data parallelism for any ``torch.nn.Module`` on the fused gradient all-reduce.

``FlatDataParallel`` flattens the module's fp32 parameters into one master buffer (parameters become
views), mirrors the gradient as a flat bf16 buffer in symmetric (peer-mapped) memory, and registers
post-accumulate hooks: as each parameter's gradient appears during backward it is cast into its
slice of the bf16 buffer (one multi-tensor launch per bucket), and when the last gradient of a bucket has arrived the bucket's fused
all-reduce (rank-ordered fp32 sum x 1/world, fp32 output; csrc/comm.cu) is launched on a
communication stream, overlapping the rest of backward. ``step()`` joins the streams and applies
one fused optimizer launch (Adam / AdamW / SGD-momentum; csrc/kernels_basic.cu) over the flat
buffers. ``comm="nccl"`` performs the same reduction with NCCL (the baseline configuration).

Semantics kept from the reference's data-parallel trainer
(scirust-core/src/autodiff/data_parallel.rs:109-177, distributed.rs:96-167): gradients are summed in
rank order and multiplied once by 1/world, so every replica applies identical bits.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from .fused_allreduce import FusedAllReduce
from .symm import SymmetricRegion

BF = torch.bfloat16


class FlatDataParallel:
    """Gradient bookkeeping, per step:

    * a parameter whose hook did not fire (unused branch, frozen head) contributes a ZERO gradient: its
      slice of the bf16 buffer is cleared in ``step()`` before the bucket is reduced;
    * a second ``backward()`` before ``step()`` (gradient accumulation) ADDS to the slice (fp32 add, one
      rounding); a bucket that had already been reduced is reduced again in ``step()``. Wrap all but the
      last micro-batch in ``no_sync()`` to avoid the wasted early reductions;
    * a bucket's gradients are cast into the flat buffer by one multi-tensor launch when the bucket is
      complete, not by one copy per parameter.
    """

    def __init__(self, module: torch.nn.Module, group=None, optimizer: str = "adam", lr: float = 1e-3,
                 momentum: float = 0.9, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 comm: str = "fused", bucket_elems: int = 4 << 20, overlap: bool = True, n_ctas: int = 48,
                 max_buckets: int = 192):
        self.module, self.group = module, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.mode = {"adam": "adam", "adamw": "adamw", "sgd": "sgd"}[optimizer]
        self.lr, self.momentum, self.betas, self.eps, self.wd = lr, momentum, betas, eps, weight_decay
        self.comm = comm if self.world > 1 else "none"
        self.step_count = 0
        params = [p for p in module.parameters() if p.requires_grad]
        dev = params[0].device
        self.dev = dev
        offs, off = [], 0
        for p in params:
            offs.append(off)
            off += (p.numel() + 7) // 8 * 8
        self.n = off
        # every bucket takes a flag slot and a counter word of the fused reducer: grow the buckets of a large model
        bucket_elems = max(bucket_elems, -(-off // max_buckets))
        self.master = torch.zeros(off, dtype=torch.float32, device=dev)
        for p, o in zip(params, offs):
            self.master[o:o + p.numel()].copy_(p.detach().reshape(-1))
            p.data = self.master[o:o + p.numel()].view(p.shape)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master) if self.mode != "sgd" else None
        self.params, self.offs = params, offs
        if self.comm == "fused":
            self.region = SymmetricRegion(group, off * 2 + off * 4 + 8192, device=dev)
            self.grad16 = self.region.tensor((off,), BF)
            self.reduced = self.region.tensor((off,), torch.float32)
            self.ar = FusedAllReduce(self.region, self.grad16, self.reduced, n_ctas=n_ctas)
        else:
            self.region = None
            self.grad16 = torch.zeros(off, dtype=BF, device=dev)
            self.reduced = torch.zeros(off, dtype=torch.float32, device=dev)
        self.grad16.zero_()
        # buckets in reverse parameter order (the order gradients appear in backward)
        self.buckets, cur, cur_n = [], [], 0
        for i in reversed(range(len(params))):
            cur.append(i)
            cur_n += params[i].numel()
            if cur_n >= bucket_elems:
                self.buckets.append(cur)
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(cur)
        self.bucket_of = {i: b for b, idxs in enumerate(self.buckets) for i in idxs}
        self.bucket_range = []
        for idxs in self.buckets:
            lo = min(offs[i] for i in idxs)
            hi = max(offs[i] + (params[i].numel() + 7) // 8 * 8 for i in idxs)
            self.bucket_range.append((lo, hi - lo))
        self.overlap = overlap and self.world > 1
        self.comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self._sync = True
        # a peer-flag time-out inside the reducer leaves a partial sum: surface it one step late at most
        self._status = _lib.DeferredStatus(dev) if (self.comm == "fused" and dev.type == "cuda") else None
        for i, p in enumerate(params):
            p.register_post_accumulate_grad_hook(self._make_hook(i))
        self._reset()

    def _reset(self):
        self.pending = [len(b) for b in self.buckets]
        self._launched = set()
        self._fired = [False] * len(self.params)      # hook fired since the last step()
        self._held = [[] for _ in self.buckets]       # (param index, fp32 gradient) waiting for the bucket's cast
        self._dirty = [False] * len(self.buckets)     # slice holds gradients of an earlier backward of this step

    class _NoSync:
        def __init__(self, dp):
            self.dp = dp

        def __enter__(self):
            self.prev, self.dp._sync = self.dp._sync, False

        def __exit__(self, *exc):
            self.dp._sync = self.prev

    def no_sync(self):
        """Context manager: backward passes inside it only accumulate; nothing is reduced until ``step()``
        (or until a later backward outside the context completes a bucket)."""
        return FlatDataParallel._NoSync(self)

    def _cast_bucket(self, b):
        held = self._held[b]
        if not held:
            return
        if self._dirty[b] and b in self._launched and self.comm_stream is not None:
            # an earlier reduction of this bucket may still be reading the slice
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        fresh = [(i, g) for i, g, acc in held if not acc]
        again = [(i, g) for i, g, acc in held if acc]
        for items, acc in ((fresh, False), (again, True)):
            if items:
                ops.multi_cast_to_bf16([g.reshape(-1) for _, g in items], self.grad16,
                                       [self.offs[i] for i, _ in items], accumulate=acc)
        self._held[b] = []

    def _make_hook(self, i):
        def hook(p):
            b = self.bucket_of[i]
            g = p.grad
            p.grad = None
            if g.dtype != torch.float32:
                g = g.float()
            if self._fired[i]:
                # a second backward before step(): add to the slice, and reduce the bucket (again) in step()
                self._dirty[b] = True
                self._held[b].append((i, g, True))
                self._cast_bucket(b)
                self._launched.discard(b)
                return
            self._fired[i] = True
            self._held[b].append((i, g, False))
            self.pending[b] -= 1
            if self.pending[b] == 0:
                self._cast_bucket(b)
                if self.overlap and self._sync:
                    self._reduce_bucket(b, async_=True)
        return hook

    def _reduce_bucket(self, b, async_):
        lo, n = self.bucket_range[b]
        self._launched.add(b)
        if self.comm == "fused":
            if async_:
                ev = torch.cuda.Event()
                ev.record()
                self.comm_stream.wait_event(ev)
                self.ar.reduce(lo, n, 1.0 / self.world, stream=self.comm_stream)
            else:
                self.ar.reduce(lo, n, 1.0 / self.world)
        elif self.comm == "nccl":
            t = self.grad16[lo:lo + n]
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            self.reduced[lo:lo + n].copy_(t)
            self.reduced[lo:lo + n].mul_(1.0 / self.world)

    def __call__(self, *a, **kw):
        return self.module(*a, **kw)

    def step(self):
        """Finish the gradient reduction and apply the optimizer to every parameter."""
        for b, idxs in enumerate(self.buckets):
            if self.pending[b] > 0:
                # some parameters of this bucket received no gradient in this step: theirs is zero
                self._cast_bucket(b)
                for i in idxs:
                    if not self._fired[i]:
                        self.grad16[self.offs[i]:self.offs[i] + self.params[i].numel()].zero_()
        if self.world > 1:
            for b in range(len(self.buckets)):
                if b not in self._launched:
                    # late buckets take the communication stream too: kernels whose CTAs wait for other GPUs run in
                    # one order on one stream per GPU (two of them side by side can close a cycle of waits)
                    self._reduce_bucket(b, async_=self.overlap and self.comm_stream is not None)
            if self.overlap and self.comm == "fused":
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                torch.cuda.current_stream().wait_event(ev)
            grad = self.reduced
        else:
            grad = self.grad16
        self.step_count += 1
        b1, b2 = (self.momentum, 0.0) if self.mode == "sgd" else self.betas
        ops.optim_step(self.master, self.m, self.v, grad, None, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                       weight_decay=self.wd, step=self.step_count, mode=self.mode)
        self._reset()
        if self._status is not None:
            self._status.poll()

    def close(self):
        if self.region is not None:
            self.region.close()
            self.region = None

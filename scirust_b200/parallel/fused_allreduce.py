"""Fused data-parallel gradient all-reduce (csrc/comm.cu: ``sb_allreduce_bf16``).

The model's flat bf16 gradient buffer is re-homed into symmetric memory, so weight-gradient
GEMMs write straight into a buffer every peer can read. After backward (or per bucket, as the
blocks finish, on a side stream) one kernel per bucket pulls the peers' shards over NVLink, sums
them in rank order in fp32, scales by 1/world, writes the rounded shard into its own ``reduced``
buffer and then pulls the other ranks' reduced shards, so the optimizer finds the whole bucket there. Reduction order is fixed and every rank
receives identical bits.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g
from .symm import FLAG_SLOTS, SymmetricRegion

import ctypes as C

_lib.register("sb_allreduce_bf16", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.sz, _lib.f32, C.c_uint32,
                                    _lib.i32, _lib.i32, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp])
_lib.register("sb_wait_probe", [_lib.vp, _lib.i32, C.c_uint32, _lib.i32, _lib.vp, _lib.vp])


class FusedAllReduce:
    """All-reduce (sum * scale) of equally sized bf16 buffers living in one symmetric region."""

    def __init__(self, region: SymmetricRegion, src: torch.Tensor, dst: torch.Tensor, n_ctas: int = 32,
                 wait_ms: int = 0):
        self.region, self.src, self.dst = region, src, dst
        self.n_ctas, self.wait_ms = n_ctas, wait_ms
        self.epoch = 0
        # one CTA-counter word per bucket; a bucket also takes one flag slot, so the two run out together
        self.counters = torch.zeros(FLAG_SLOTS, dtype=torch.int32, device=src.device)
        self.flag_ptrs = region.flag_ptrs()
        self._buckets = {}
        self._epochs = {}

    def bucket(self, start: int, n: int):
        key = (start, n)
        b = self._buckets.get(key)
        if b is None:
            if start % 8 or n % 8:
                raise ValueError("bucket bounds must be multiples of 8 elements")
            if len(self._buckets) >= self.counters.numel():
                raise RuntimeError(f"FusedAllReduce: more than {self.counters.numel()} buckets; use larger buckets")
            slot = self.region.new_slot()
            b = (self.region.peer_ptrs(self.src[start:start + n]), self.region.peer_ptrs(self.dst[start:start + n]),
                 slot, len(self._buckets))
            self._buckets[key] = b
        return b

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def reduce(self, start: int, n: int, scale: float, epoch: int | None = None, stream=None):
        """Reduce ``src[start:start+n]`` into ``dst[start:start+n]`` on every rank. Each bucket owns a flag
        slot, and its calls are numbered by a per-bucket counter that advances identically on every rank
        (all ranks issue the same sequence of calls), so a bucket may be reduced any number of times per step.
        ``epoch`` overrides the counter (it must grow from call to call of the bucket)."""
        in_p, out_p, slot, idx = self.bucket(start, n)
        if epoch is None:
            epoch = self._epochs.get(idx, 0) + 1
        self._epochs[idx] = epoch
        r = self.region
        st = _lib.status_word(self.src.device)
        s = _lib.stream() if stream is None else stream.cuda_stream
        # buckets of tens of MB (an embedding table) are bound by bytes in flight: more CTAs
        n_ctas = self.n_ctas if n < (24 << 20) else max(self.n_ctas, 64)
        _lib.call("sb_allreduce_bf16", in_p, out_p, self.flag_ptrs, r.rank, r.world, n, float(scale), epoch, slot,
                  int(self.dst.dtype == torch.float32), self.counters.data_ptr() + 4 * idx, n_ctas, self.wait_ms,
                  st.data_ptr(), s)
        _g.launch_count += 1


class FusedGradAllReduce:
    """Gradient reducer for ``Trainer``: ``reducer(flat_grad) -> (reduced_grad, 1.0)``.

    With ``overlap=True`` each decoder layer's bucket is reduced on a communication stream as soon
    as that layer's backward has produced it; the call at the end of backward reduces what is left
    (embedding, norm gains) and joins the streams."""

    def __init__(self, model, group, overlap: bool = True, n_ctas: int = 48, out_dtype=torch.bfloat16):
        n_ctas = int(os.environ.get("SB_AR_CTAS", n_ctas))       # CTAs of one bucket's all-reduce kernel
        overlap = overlap and os.environ.get("SB_AR_OVERLAP", "1") != "0"
        self.model = model
        self.world = dist.get_world_size(group)
        n = model.flat_grad.numel()
        esz = 2 + (4 if out_dtype == torch.float32 else 2)
        self.region = SymmetricRegion(group, n * esz + 4096, device=model.flat.device)
        grad = self.region.tensor((n,), torch.bfloat16)
        self.reduced = self.region.tensor((n,), out_dtype)
        model.rebind_grad_buffer(grad)
        self.ar = FusedAllReduce(self.region, grad, self.reduced, n_ctas=n_ctas)
        self.overlap = overlap
        self.comm_stream = torch.cuda.Stream(device=model.flat.device)
        self.done = set()
        self.epoch = 0
        self.layer_buckets = model.layer_buckets()
        if overlap:
            model.on_grads_ready = self._layer_ready
        self._epoch_started = False

    def _begin(self):
        if not self._epoch_started:
            self.epoch = self.ar.next_epoch()
            self.done = set()
            self._epoch_started = True

    def _layer_ready(self, index: int):
        self._begin()
        start, n = self.layer_buckets[index]
        ev = torch.cuda.Event()
        ev.record()
        self.comm_stream.wait_event(ev)
        self.ar.reduce(start, n, 1.0 / self.world, self.epoch, stream=self.comm_stream)
        self.done.add(index)

    def __call__(self, flat_grad):
        self._begin()
        n = flat_grad.numel()
        # remaining ranges: everything not covered by an already-reduced layer bucket
        covered = sorted(self.layer_buckets[i] for i in self.done)
        pos = 0
        rest = []
        for s, ln in covered:
            if s > pos:
                rest.append((pos, s - pos))
            pos = s + ln
        if pos < n:
            rest.append((pos, n - pos))
        for s, ln in rest:
            self.ar.reduce(s, ln, 1.0 / self.world, self.epoch)
        if self.done:
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            torch.cuda.current_stream().wait_event(ev)
        self._epoch_started = False
        return self.reduced, 1.0

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
_lib.register("sb_allreduce_bf16_lean", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.sz, _lib.f32, C.c_uint32,
                                         _lib.i32, _lib.i32, _lib.vp, _lib.i32, _lib.i32, _lib.vp, _lib.vp])
_lib.register("sb_wait_probe", [_lib.vp, _lib.i32, C.c_uint32, _lib.i32, _lib.vp, _lib.vp])


def _num_sms(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148


class FusedAllReduce:
    """All-reduce (sum * scale) of equally sized bf16 buffers living in one symmetric region."""

    def __init__(self, region: SymmetricRegion, src: torch.Tensor, dst: torch.Tensor, n_ctas: int = 32,
                 wait_ms: int = 0):
        self.region, self.src, self.dst = region, src, dst
        self.n_ctas, self.wait_ms = n_ctas, wait_ms
        self.epoch = 0
        self.lean_ctas = int(os.environ.get("SB_AR_LEAN_CTAS", 0)) or _num_sms(src.device)
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

    def reduce(self, start: int, n: int, scale: float, epoch: int | None = None, stream=None, lean: bool = False):
        """Reduce ``src[start:start+n]`` into ``dst[start:start+n]`` on every rank. Each bucket owns a flag
        slot, and its calls are numbered by a per-bucket counter that advances identically on every rank
        (all ranks issue the same sequence of calls), so a bucket may be reduced any number of times per step.
        ``epoch`` overrides the counter (it must grow from call to call of the bucket). ``lean`` runs the same
        collective (same bits) in CTAs of 128 threads x 64 registers, one per SM, which fit beside a resident GEMM
        CTA: the shape for a bucket that is reduced on a side stream while backward keeps the SMs busy."""
        in_p, out_p, slot, idx = self.bucket(start, n)
        if epoch is None:
            epoch = self._epochs.get(idx, 0) + 1
        self._epochs[idx] = epoch
        r = self.region
        st = _lib.status_word(self.src.device)
        s = _lib.stream() if stream is None else stream.cuda_stream
        # buckets of tens of MB (an embedding table) are bound by bytes in flight: more CTAs
        n_ctas = self.n_ctas if n < (24 << 20) else max(self.n_ctas, 64)
        if lean:
            n_ctas = self.lean_ctas
        _lib.call("sb_allreduce_bf16_lean" if lean else "sb_allreduce_bf16", in_p, out_p, self.flag_ptrs, r.rank, r.world, n, float(scale), epoch, slot,
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
        # SB_AR_OVERLAP: "attn" (default) starts a finished layer's bucket when the NEXT layer's attention backward
        # is launched; "1" starts it as soon as the layer's backward has been issued; "0" reduces everything after
        # backward. The GEMMs are persistent kernels with a static tile schedule, so a collective that takes SMs
        # while one runs delays it by its own duration (measured: "1" gains nothing over "0"); the attention
        # backward kernels are grids of short CTAs and simply flow around it.
        mode = os.environ.get("SB_AR_OVERLAP", "attn") if overlap else "0"
        self.model = model
        self.world = dist.get_world_size(group)
        n = model.flat_grad.numel()
        esz = 2 + (4 if out_dtype == torch.float32 else 2)
        self.region = SymmetricRegion(group, n * esz + 4096, device=model.flat.device)
        grad = self.region.tensor((n,), torch.bfloat16)
        self.reduced = self.region.tensor((n,), out_dtype)
        model.rebind_grad_buffer(grad)
        self.ar = FusedAllReduce(self.region, grad, self.reduced, n_ctas=n_ctas)
        self.overlap = mode != "0"
        self.defer = mode == "attn" and hasattr(model, "on_attention_bwd")
        self.lean = os.environ.get("SB_AR_LEAN", "0") == "1"      # overlapped buckets in the small CTA shape
        lo, hi = torch.cuda.Stream.priority_range() if torch.cuda.is_available() else (0, 0)
        self.comm_stream = torch.cuda.Stream(device=model.flat.device, priority=hi)
        self.done = []          # (start, length) of the buckets already issued this step
        self.pending = []       # buckets whose gradients are complete and that wait for an attention slot
        self.epoch = 0
        self.layer_buckets = model.layer_buckets()
        self.head_bucket = None
        seg = getattr(model, "segments", {}).get("lm_head")
        if seg is not None and seg[0] % 8 == 0:
            self.head_bucket = (seg[0], (seg[1] + 7) // 8 * 8)
            if self.head_bucket[0] + self.head_bucket[1] > n:
                self.head_bucket = None
        if self.overlap:
            model.on_grads_ready = self._layer_ready
            if self.defer:
                model.on_attention_bwd = self._attention_slot
        self._epoch_started = False

    def _begin(self):
        if not self._epoch_started:
            self.epoch = self.ar.next_epoch()
            self.done = []
            self.pending = []
            self._epoch_started = True

    def _issue(self, bucket):
        start, n = bucket
        self.ar.reduce(start, n, 1.0 / self.world, self.epoch, stream=self.comm_stream, lean=self.lean)
        self.done.append(bucket)

    def _flush(self):
        """Start every pending bucket behind what the main stream has issued so far."""
        if not self.pending:
            return
        ev = torch.cuda.Event()
        ev.record()
        self.comm_stream.wait_event(ev)
        for b in self.pending:
            self._issue(b)
        self.pending = []

    def _layer_ready(self, index: int):
        self._begin()
        self.pending.append(self.layer_buckets[index])
        if not self.defer:
            self._flush()

    def _attention_slot(self, index: int):
        self._begin()
        if self.head_bucket is not None and self.head_bucket not in self.done and self.head_bucket not in self.pending \
                and index == len(self.layer_buckets) - 1:
            self.pending.append(self.head_bucket)     # the LM-head gradient is the first one backward produces
        self._flush()

    def __call__(self, flat_grad):
        self._begin()
        n = flat_grad.numel()
        # remaining ranges: everything not covered by an already-issued bucket
        covered = sorted(self.done)
        pos = 0
        rest = []
        for s, ln in covered:
            if s > pos:
                rest.append((pos, s - pos))
            pos = s + ln
        if pos < n:
            rest.append((pos, n - pos))
        if not self.overlap:
            for s, ln in rest:
                self.ar.reduce(s, ln, 1.0 / self.world, self.epoch)
        else:
            # Everything goes through the one communication stream. Two of these kernels running side by side on a
            # GPU (one per stream) could each hold part of the SMs while their remaining CTAs wait for the other to
            # leave, and with the peers having let the other kernel in first the flag waits would close a cycle
            # across GPUs: kernels whose CTAs wait for other GPUs are issued in ONE order on ONE stream per GPU.
            self.pending.extend(rest)
            self._flush()
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
            torch.cuda.current_stream().wait_event(ev)
        self._epoch_started = False
        return self.reduced, 1.0

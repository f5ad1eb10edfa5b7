"""Latency-oriented collectives for tensor-parallel inference (csrc/comm.cu: ``sb_small_collective``).

A tensor-parallel decode step all-reduces a few kilobytes twice per layer. The bandwidth-oriented
all-reduce of the training path (two flag phases, reduce-scatter + push) is the wrong shape for that,
so this channel uses one flag phase and lets every rank read all peers' partial results directly
over NVLink and add them in rank order (identical bits on every rank), writing plain local memory.
The call's epoch lives in a device word that the kernel advances itself, so a captured CUDA graph
replays correctly. ``gather_rows`` is the matching all-gather (vocabulary-sharded logits).

With ``backend="nccl"`` (or on CPU with gloo) the same calls go through ``torch.distributed``: that
is the baseline the peer-memory kernels are compared against, and the path the CPU tests exercise.

The reference has no tensor parallelism (its multi-rank code is the host all-reduce of
scirust-core/src/distributed.rs:96-167, whose rank-ordered sum this keeps).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g

_lib.register("sb_small_collective", [_lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.sz, _lib.i32,
                                      _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.vp, _lib.i32, _lib.i32, _lib.vp,
                                      _lib.vp])


class SmallCollectives:
    """One channel of small all-reduces / all-gathers over a ``SymmetricRegion``.

    Source buffers come from ``source(name, shape, dtype)`` and live in symmetric memory; a source
    may be rewritten only after a LATER collective of this channel has completed on the same rank,
    so callers alternate at least two named sources (a decoder layer's attention and MLP partials do
    that naturally)."""

    def __init__(self, group, region=None, backend: str = "fused", wait_ms: int = 0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = backend if region is not None else "nccl"
        self.region = region
        self.wait_ms = wait_ms
        self._src = {}
        if self.backend == "fused":
            dev = region.device
            self.slot = region.new_slot()
            self.flag_ptrs = region.flag_ptrs()
            self.state = torch.zeros(64, dtype=torch.int32, device=dev)   # [0] epoch word, [32] CTA counter

    def source(self, name: str, shape, dtype, device=None) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._src.get(key)
        if t is None:
            if self.backend == "fused":
                t = self.region.tensor(tuple(shape), dtype)
                t.zero_()
                ptrs = self.region.peer_ptrs(t)
            else:
                t = torch.zeros(tuple(shape), dtype=dtype, device=device)
                ptrs = None
            self._src[key] = t
            self._src[("ptrs", t.data_ptr())] = ptrs
        return t

    def _launch(self, src, mode, in_fp32, n, rows, residual, out):
        ptrs = self._src[("ptrs", src.data_ptr())]
        r = self.region
        words = src.numel() * src.element_size() * self.world // 16      # 16-byte words read by this rank
        n_ctas = max(1, min(32, words // (256 * 4)))
        st = _lib.status_word(src.device)
        _lib.call("sb_small_collective", ptrs, self.flag_ptrs, r.rank, r.world, mode, in_fp32, n, rows,
                  _lib.ptr(residual), out.data_ptr(), self.state.data_ptr(), self.slot, self.state[32:].data_ptr(),
                  n_ctas, self.wait_ms, st.data_ptr(), _lib.stream())
        _g.launch_count += 1

    def all_reduce(self, src: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None):
        """out = residual + sum over ranks of ``src`` (rank order, fp32), bf16 result in local memory."""
        if out is None:
            out = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
        if self.backend == "fused":
            n = src.numel()
            if n % 8:
                raise ValueError("all_reduce: element count must be a multiple of 8")
            self._launch(src, 0, int(src.dtype == torch.float32), n, 1, residual, out)
            return out
        parts = [torch.empty_like(src) for _ in range(self.world)]
        dist.all_gather(parts, src.contiguous(), group=self.group)
        acc = residual.float().clone() if residual is not None else torch.zeros(src.shape, dtype=torch.float32,
                                                                                 device=src.device)
        for t in parts:          # same fixed order as the kernel
            acc += t.float()
        out.copy_(acc.to(torch.bfloat16))
        return out

    def gather_rows(self, src: torch.Tensor, out: torch.Tensor):
        """``src`` [rows, n] per rank -> ``out`` [rows, world * n] (rank-major within a row)."""
        rows, n = src.shape
        if self.backend == "fused":
            words = n * src.element_size()
            if words % 16:
                raise ValueError("gather_rows: a row shard must be a multiple of 16 bytes")
            self._launch(src, 1, 0, words // 16, rows, None, out)
            return out
        parts = [torch.empty_like(src) for _ in range(self.world)]
        dist.all_gather(parts, src.contiguous(), group=self.group)
        out.view(rows, self.world, n).copy_(torch.stack(parts, 1))
        return out


class GemvAllReduceChannel:
    """Peer-mapped state of the fused row-parallel GEMV + all-reduce (``ops.decode.gemv_allreduce``): per rank a
    receive buffer ``fp32 [2][world][rows][n_max]`` (every peer stores its partial sums of a call into slot
    ``[call parity][its rank]``), one epoch word per (block of output columns, source rank), and a local epoch
    word / CTA counter that the kernel maintains, so a captured CUDA graph replays the calls correctly. All ranks
    must issue the same sequence of calls on a channel; consecutive calls alternate the buffer halves, which is what
    lets a rank run one call ahead of its slowest peer.

    The receive buffer is addressed as ``[2][world][rows][N]`` with the N of the call, so calls of different widths
    may share a channel as long as every rank uses the same width for the same call."""

    def __init__(self, region, rows: int = 8, n_max: int = 8192, wait_ms: int = 0):
        self.region, self.rows, self.n_max, self.wait_ms = region, rows, n_max, wait_ms
        self.rank, self.world = region.rank, region.world
        self.recv = region.tensor((2 * self.world * rows * n_max,), torch.float32)
        self.recv.zero_()
        self.flags = region.tensor((((n_max + 255) // 256) * 16,), torch.int32)
        self.flags.zero_()
        self._recv_ptrs = region.peer_ptrs(self.recv)
        self.flag_ptrs = region.peer_ptrs(self.flags)
        self.state = torch.zeros(64, dtype=torch.int32, device=region.device)   # [0] epoch word, [32] CTA counter
        torch.cuda.synchronize(region.device)
        dist.barrier(group=region.group)      # nobody pushes into a buffer that is still being cleared

    def recv_ptrs(self, n: int):
        return self._recv_ptrs


class ArgmaxChannel:
    """Peer-mapped state of the vocabulary-parallel fused LM head (``ops.decode.gemv_argmax``): per rank
    ``2 x world x 8`` candidate words (value bits and global column of a rank's best entry per row; a call uses the
    half of its parity), ``world`` epoch words, and a local epoch word that the kernel advances, so a captured CUDA
    graph replays the calls correctly. Every rank must issue the same sequence of calls."""

    def __init__(self, region, wait_ms: int = 0):
        self.region, self.wait_ms = region, wait_ms
        self.rank, self.world = region.rank, region.world
        self.cand = region.tensor((2 * self.world * 8,), torch.int64)
        self.cand.zero_()
        self.flags = region.tensor((16,), torch.int32)
        self.flags.zero_()
        self.cand_ptrs = region.peer_ptrs(self.cand)
        self.flag_ptrs = region.peer_ptrs(self.flags)
        self.state = torch.zeros(16, dtype=torch.int32, device=region.device)   # [0] epoch word
        torch.cuda.synchronize(region.device)
        dist.barrier(group=region.group)

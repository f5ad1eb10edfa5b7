"""Tensor parallelism with sequence-parallel activations (Megatron-style column/row sharding).

Activations between blocks are sharded over the token dimension (rank r holds rows
``[r*T/W, (r+1)*T/W)``); inside a block the QKV and gate/up projections are column-parallel and the
o_proj / down projections row-parallel. Each boundary is one fused kernel on CTA pairs
(csrc/gemm_pair_tcgen05.cu; csrc/gemm_dist_tcgen05.cu for shapes whose rows per rank are not a
multiple of 256):

* ``ag_matmul``   all-gather -> GEMM: every rank pushes its shard, 128-row chunk by chunk, into the
  peers' landing buffers with plain peer stores while the tensor cores already work on the rows that
  have arrived (own rows first); a remote row crosses NVLink once and is then read from local memory
  by TMA for every output column tile.
* ``matmul_rs``   GEMM -> reduce-scatter: the epilogue sends every finished tile straight to the
  rank that owns its rows (TMA tensor store into that rank's receive buffer, slot = source rank),
  under the main loop of the following tiles; the owner adds the W slots of a row block in rank order
  (+ residual) from local memory as soon as the block is complete.

``backend="nccl"`` runs the same math as NCCL all-gather / reduce-scatter around library GEMMs
(`torch.matmul`): the baseline configuration the fused path is measured against. The reference has
no tensor parallelism at all (src/lib.rs:133); what is kept from it is the fixed rank-order
reduction contract (scirust-core/src/distributed.rs:96-167).
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _g
from .symm import SymmetricRegion

BF = torch.bfloat16

_lib.register("sb_gemm_dist_bf16", [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                    _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                    _lib.i32, _lib.i32, _lib.i32, _lib.i32, C.c_uint32, _lib.vp, _lib.i32, _lib.i32,
                                    _lib.vp, _lib.i32, _lib.vp, _lib.vp, _lib.vp, _lib.vp])


_lib.register("sb_gemm_pair_ag_bf16", [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                       _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.vp,
                                       _lib.vp, _lib.vp, _lib.i32, _lib.i32, C.c_uint32, _lib.i32, _lib.i32, _lib.vp,
                                       _lib.vp])


_lib.register("sb_gemm_pair_rs_bf16", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.vp, _lib.i32, _lib.vp, _lib.i32, _lib.i32,
                                       _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.vp, _lib.vp, _lib.vp,
                                       _lib.vp, _lib.i32, _lib.i32, C.c_uint32, _lib.i32, _lib.vp, _lib.vp])


class TPContext:
    """Process-group state for the fused tensor-parallel kernels: a symmetric region holding the
    peer-visible activation buffers, the double-buffered reduce-scatter staging area and the flag
    slots."""

    def __init__(self, group, max_rows: int, max_cols: int, sym_bytes: int = 0, backend: str = "fused",
                 wait_ms: int = 0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = backend
        self.wait_ms = wait_ms
        # backend "host": the NCCL arm's collectives-around-library-products on CPU tensors over a gloo group (the
        # sharding logic of the models can then be checked on machines without a GPU)
        self.dev = torch.device("cpu") if backend == "host" else torch.device("cuda", torch.cuda.current_device())
        self.epoch = 0
        self.rs_calls = 0
        self.pair = os.environ.get("SB_TP_PAIR", "1") != "0"   # CTA-pair kernel for all-gather -> GEMM
        # a one-rank group normally takes the plain GEMM; SB_TP_PAIR_SINGLE=1 sends it through the fused CTA-pair
        # kernels (every "peer" is the local buffer) so that a profiler can capture them on one GPU
        self._pair_min_world = 1 if os.environ.get("SB_TP_PAIR_SINGLE", "0") == "1" else 2
        # weight gradients: SB_TP_DIRECT_WGRAD=1 keeps the kernel that reads the gathered operand from the peers tile
        # by tile (every remote tile crosses NVLink once per output column tile: slower, kept for comparison)
        self.direct_wgrad = os.environ.get("SB_TP_DIRECT_WGRAD", "0") == "1"
        # SB_TP_PROFILE=1: CUDA-event time of every product, by method and shape (``profile_report()``)
        self._prof = {} if os.environ.get("SB_TP_PROFILE", "0") == "1" else None
        if self._prof is not None:
            for name in ("ag_matmul_nn", "ag_matmul_nt", "matmul_nn_rs", "matmul_nt_rs", "ag_matmul_tn", "matmul_tn_ag"):
                setattr(self, name, self._profiled(name, getattr(self, name)))
        self._named = {}
        self._gathered = {}          # keep-name -> gathered operand of the last all-gather -> GEMM with that name
        self._peer_ptr_cache = {}
        self._status_ptr = _lib.status_word(self.dev).data_ptr() if backend == "fused" else None
        if backend == "fused":
            stage_bytes = max_rows * max_cols * 2          # W * (rows/W) * cols bf16
            total = 3 * stage_bytes + sym_bytes + (1 << 20)
            self.region = SymmetricRegion(group, total, device=self.dev)
            self.stage = [self.region.tensor((max_rows * max_cols,), BF) for _ in range(2)]
            self.stage_ptrs = [self.region.peer_ptrs(s) for s in self.stage]
            self.slot = self.region.new_slot()
            wps = self.region.words_per_slot
            self.flag_ptrs = (C.c_void_p * self.world)(
                *[b + self.region.data_bytes + self.slot * wps * 4 for b in self.region.peer_base])
            self.counters = torch.zeros(32, dtype=torch.int32, device=self.dev)
            # landing buffer of the all-gather -> GEMM products: peer-mapped, every rank pushes its shard into it
            self._ag_stage = self.region.tensor((max_rows * max_cols,), BF)
            self._ag_stage_ptrs = self.region.peer_ptrs(self._ag_stage)
            self._ag_chunk_flags = self.region.tensor((max_rows // 128 + 2,), torch.int32)
            self._ag_chunk_flags.zero_()
            self._ag_chunk_flag_ptrs = self.region.peer_ptrs(self._ag_chunk_flags)
            self._ag_flags = torch.zeros(2 * (max_rows // 128 + 2), dtype=torch.int32, device=self.dev)
            # single-CTA distributed kernel (shapes the pair kernel refuses): its own local landing buffer
            self._local_stage, self._local_stage_elems = None, max_rows * max_cols
            # reduce-scatter on the pair kernel: "block complete" epochs pushed by the peers, local counters
            self._rs_ready = self.region.tensor((8 * 512,), torch.int32)
            self._rs_ready.zero_()
            self._rs_ready_ptrs = self.region.peer_ptrs(self._rs_ready)
            self._rs_ctr = torch.zeros(max_rows // 256 + 4, dtype=torch.int32, device=self.dev)
        else:
            self.region = None

    def _profiled(self, name, fn):
        def wrapped(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            key = (name, tuple(a[0].shape), tuple(a[1].shape))
            self._prof.setdefault(key, []).append((e0, e1))
            return r
        return wrapped

    def profile_report(self, skip: int = 0):
        """{(method, shape a, shape b): (calls, total ms)} of the products recorded under SB_TP_PROFILE=1."""
        torch.cuda.synchronize()
        out = {}
        for key, evs in (self._prof or {}).items():
            evs = evs[skip:]
            out[key] = (len(evs), sum(a.elapsed_time(b) for a, b in evs))
        return out

    # peer-visible persistent buffers, keyed by name (activations that another rank's kernel reads)
    def buffer(self, name: str, shape, dtype=BF) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        t = self._named.get(key)
        if t is None:
            if self.region is not None:
                t = self.region.tensor(tuple(shape), dtype)
            else:
                t = torch.empty(tuple(shape), dtype=dtype, device=self.dev)
            self._named[key] = t
        return t

    def _peer_ptrs(self, t: torch.Tensor):
        """Per-rank addresses of a symmetric tensor, built once per buffer (the call sites reuse their buffers)."""
        key = t.data_ptr()
        p = self._peer_ptr_cache.get(key)
        if p is None:
            p = self._peer_ptr_cache[key] = self.region.peer_ptrs(t)
        return p

    def _ptrs(self, t: torch.Tensor, gathered: bool):
        if gathered:
            return self.region.peer_ptrs(t)
        return (C.c_void_p * self.world)(*([t.data_ptr()] * self.world))

    def _ag_pair(self, x_shard, w, out, M, N, K, b_mn, keep=None):
        """all-gather -> GEMM on the CTA-pair kernel (csrc/gemm_pair_tcgen05.cu): every rank pushes its shard
        into the peers' landing buffers chunk by chunk while 256 x 256 tiles are computed over two SMs. With
        ``keep`` the landing buffer is a named one that also receives the own shard, so that it holds the whole
        gathered matrix afterwards (``gathered(keep)``)."""
        self.epoch += 1
        if keep is None:
            if M * K > self._ag_stage.numel():
                raise ValueError("all-gather landing buffer too small for this product")
            stage_ptrs = self._ag_stage_ptrs
        else:
            full = self.buffer("gathered." + keep, (M, K))
            stage_ptrs = self._peer_ptrs(full)
            self._gathered[keep] = full
        n = self._ag_flags.numel() // 2
        _lib.call("sb_gemm_pair_ag_bf16", self._peer_ptrs(x_shard), w.data_ptr(), out.data_ptr(), None, M, N, K,
                  x_shard.stride(0), w.stride(0), out.stride(0), 0, int(b_mn), stage_ptrs, K,
                  self.flag_ptrs, self._ag_chunk_flag_ptrs, self._ag_flags[n:].data_ptr(),
                  self._ag_flags[2 * n - 1:].data_ptr(), self.rank, self.world, self.epoch, self.wait_ms,
                  int(keep is not None), self._status_ptr, _lib.stream())
        _g.launch_count += 1
        return out

    def gathered(self, keep: str):
        """The whole gathered operand of the last ``ag_matmul_*(..., keep=keep)`` call, or None."""
        return self._gathered.get(keep)

    def _rs_pair(self, a, w, out, residual, M, N, K, b_mn):
        """GEMM -> reduce-scatter on the CTA-pair kernel: tiles are pushed into the owners' receive buffers
        (``stage``: [W sources][rows / W][N] per rank) and the owners add the W slots block by block."""
        self.epoch += 1
        part = self.stage[self.rs_calls & 1]
        ptrs = self.stage_ptrs[self.rs_calls & 1]
        self.rs_calls += 1
        if M * N > part.numel():
            raise ValueError("reduce-scatter staging area too small for this product")
        n = self._rs_ctr.numel()
        _lib.call("sb_gemm_pair_rs_bf16", a.data_ptr(), w.data_ptr(), ptrs, N, out.data_ptr(), out.stride(0),
                  _lib.ptr(residual), residual.stride(0) if residual is not None else 0, M, N, K, a.stride(0),
                  w.stride(0), int(b_mn), self._rs_ready_ptrs, self.flag_ptrs, self._rs_ctr.data_ptr(),
                  self._rs_ctr[n - 1:].data_ptr(), self.rank, self.world, self.epoch, self.wait_ms,
                  _lib.status_word(self.dev).data_ptr(), _lib.stream())
        _g.launch_count += 1
        return out

    # SB_TP_RS_MIN_GFLOP: products below this much work per rank run as plain GEMM + NCCL reduce-scatter instead of
    # the fused kernel (0 = the fused kernel always; kept as a switch for comparisons).
    RS_FUSED_MIN_FLOP = float(os.environ.get("SB_TP_RS_MIN_GFLOP", "0")) * 1e9

    def _rs_small(self, M, N, K):
        return 2.0 * M * N * K < self.RS_FUSED_MIN_FLOP and self._pair_min_world == 2

    def _rs_unfused(self, full, residual_shard, Tl, N):
        out = torch.empty((Tl, N), dtype=BF, device=self.dev)
        dist.reduce_scatter_tensor(out, full, group=self.group)
        return out + residual_shard if residual_shard is not None else out

    def _rs_pair_ok(self, M, N):
        return (self.pair and self.world >= self._pair_min_world and M % (self.world * 256) == 0 and N % 8 == 0
                and self.world * (M // self.world // 256) <= 8 * 512 and M // 256 + 2 <= self._rs_ctr.numel())

    def _pair_ok(self, M, K):
        return (self.pair and self.world >= self._pair_min_world and M % (self.world * 256) == 0 and K % 8 == 0
                and M // 128 + 2 <= self._ag_flags.numel() // 2 and M * K <= self._ag_stage.numel())

    def _call(self, a, b, out, residual, M, N, K, a_mn, b_mn, a_gather, b_gather, scatter, bn=0):
        self.epoch += 1
        stage = None
        if scatter:
            stage = self.stage_ptrs[self.rs_calls & 1]
            self.rs_calls += 1
            if M * N > self.stage[0].numel():
                raise ValueError("reduce-scatter staging area too small for this product")
        ag_stage, ld_stage, cflags, cctr = None, 0, None, None
        if (a_gather and not a_mn and self.world > 1 and M // 128 + 2 <= self._ag_flags.numel() // 2
                and M * K <= self._local_stage_elems):
            if self._local_stage is None:
                self._local_stage = torch.empty(self._local_stage_elems, dtype=BF, device=self.dev)
            ag_stage, ld_stage = self._local_stage.data_ptr(), K
            half = self._ag_flags.numel() // 2
            cflags, cctr = self._ag_flags.data_ptr(), self._ag_flags[half:].data_ptr()
        _lib.call("sb_gemm_dist_bf16", self._ptrs(a, a_gather), self._ptrs(b, b_gather), out.data_ptr(),
                  _lib.ptr(residual), stage, self.flag_ptrs, M, N, K, a.stride(0), b.stride(0), out.stride(0),
                  residual.stride(0) if residual is not None else 0, int(a_mn), int(b_mn), int(a_gather),
                  int(b_gather), int(scatter), self.rank, self.world, self.epoch, self.counters.data_ptr(), bn,
                  self.wait_ms, ag_stage, ld_stage, cflags, cctr, _lib.status_word(self.dev).data_ptr(),
                  _lib.stream())
        _g.launch_count += 1
        return out

    # ---------------------------------------------------------------- fused products
    def _gather_nccl(self, x_shard, keep):
        Tl, K = x_shard.shape
        x = (self.buffer("gathered." + keep, (Tl * self.world, K)) if keep is not None
             else torch.empty((Tl * self.world, K), dtype=BF, device=self.dev))
        dist.all_gather_into_tensor(x, x_shard.contiguous(), group=self.group)
        if keep is not None:
            self._gathered[keep] = x
        return x

    def ag_matmul_nn(self, x_shard, w, keep=None):
        """all-gather(x_shard over rows) @ w   -> [T, N]; x_shard must come from ``buffer()``. ``keep`` names a
        buffer in which the gathered operand stays available (``gathered(keep)``) until the next call with that name:
        the weight-gradient product of the same layer reuses it instead of gathering again."""
        Tl, K = x_shard.shape
        T, N = Tl * self.world, w.shape[1]
        if self.backend != "fused":
            return torch.matmul(self._gather_nccl(x_shard, keep), w)
        out = torch.empty((T, N), dtype=BF, device=self.dev)
        if self._pair_ok(T, K):
            return self._ag_pair(x_shard, w, out, T, N, K, True, keep)
        self._gathered.pop(keep, None)
        return self._call(x_shard, w, out, None, T, N, K, False, True, True, False, False)

    def ag_matmul_nt(self, x_shard, w, keep=None):
        """all-gather(x_shard) @ wᵀ  (w [N, K]) -> [T, N]; ``keep`` as in ``ag_matmul_nn``."""
        Tl, K = x_shard.shape
        T, N = Tl * self.world, w.shape[0]
        if self.backend != "fused":
            return torch.matmul(self._gather_nccl(x_shard, keep), w.t())
        out = torch.empty((T, N), dtype=BF, device=self.dev)
        if self._pair_ok(T, K):
            return self._ag_pair(x_shard, w, out, T, N, K, False, keep)
        self._gathered.pop(keep, None)
        return self._call(x_shard, w, out, None, T, N, K, False, False, True, False, False)

    def matmul_nn_rs(self, a, w, residual_shard=None):
        """reduce-scatter over rows of (a @ w) (+ residual_shard) -> [T/W, N]."""
        T, K = a.shape
        N = w.shape[1]
        Tl = T // self.world
        if self.backend != "fused":
            full = torch.matmul(a, w)
            out = torch.empty((Tl, N), dtype=BF, device=self.dev)
            dist.reduce_scatter_tensor(out, full, group=self.group)
            return out + residual_shard if residual_shard is not None else out
        if self._rs_small(T, N, K):
            return self._rs_unfused(_g.matmul_nn(a, w), residual_shard, Tl, N)
        out = torch.empty((Tl, N), dtype=BF, device=self.dev)
        if self._rs_pair_ok(T, N):
            return self._rs_pair(a, w, out, residual_shard, T, N, K, True)
        return self._call(a, w, out, residual_shard, T, N, K, False, True, False, False, True)

    def matmul_nt_rs(self, a, w, residual_shard=None):
        """reduce-scatter over rows of (a @ wᵀ) (w [N, K]) (+ residual_shard) -> [T/W, N]."""
        T, K = a.shape
        N = w.shape[0]
        Tl = T // self.world
        if self.backend != "fused":
            full = torch.matmul(a, w.t())
            out = torch.empty((Tl, N), dtype=BF, device=self.dev)
            dist.reduce_scatter_tensor(out, full, group=self.group)
            return out + residual_shard if residual_shard is not None else out
        if self._rs_small(T, N, K):
            return self._rs_unfused(_g.matmul_nt(a, w), residual_shard, Tl, N)
        out = torch.empty((Tl, N), dtype=BF, device=self.dev)
        if self._rs_pair_ok(T, N):
            return self._rs_pair(a, w, out, residual_shard, T, N, K, False)
        return self._call(a, w, out, residual_shard, T, N, K, False, False, False, False, True)

    def ag_matmul_tn(self, x_shard, dy, out=None, residual=None, keep=None):
        """all-gather(x_shard)ᵀ @ dy -> [K_x, N]: weight gradient of a column-parallel layer
        (x sharded over tokens, dy local with all tokens). ``keep``: name under which an earlier
        ``ag_matmul_*`` left the gathered ``x``; it is then used as it is, without any communication."""
        Tl, M = x_shard.shape
        T, N = dy.shape
        full = self._gathered.get(keep) if keep is not None else None
        if full is not None and tuple(full.shape) == (T, M):
            if self.backend != "fused":
                r = torch.matmul(full.t(), dy)
                if residual is not None:
                    r = r + residual
                if out is not None:
                    out.copy_(r)
                    return out
                return r
            return _g.matmul_tn(full, dy, residual=residual, out=out)
        if self.backend != "fused":
            x = torch.empty((T, M), dtype=BF, device=self.dev)
            dist.all_gather_into_tensor(x, x_shard.contiguous(), group=self.group)
            r = torch.matmul(x.t(), dy)
            if residual is not None:
                r = r + residual
            if out is not None:
                out.copy_(r)
                return out
            return r
        if self.direct_wgrad:
            if out is None:
                out = torch.empty((M, N), dtype=BF, device=self.dev)
            return self._call(x_shard, dy, out, residual, M, N, T, True, True, True, False, False)
        # weight gradient: the gathered operand is needed whole by every output tile, so it is landed once in local
        # memory (a plain all-gather) and the product runs on the CTA-pair GEMM
        x = torch.empty((T, M), dtype=BF, device=self.dev)
        dist.all_gather_into_tensor(x, x_shard.contiguous(), group=self.group)
        return _g.matmul_tn(x, dy, residual=residual, out=out)

    def matmul_tn_ag(self, a, dy_shard, out=None, residual=None, keep=None):
        """aᵀ @ all-gather(dy_shard) -> [K_a, N]: weight gradient of a row-parallel layer
        (a local with all tokens, dy sharded over tokens); ``keep`` as in ``ag_matmul_tn``."""
        T, M = a.shape
        Tl, N = dy_shard.shape
        full = self._gathered.get(keep) if keep is not None else None
        if full is not None and tuple(full.shape) == (T, N):
            if self.backend != "fused":
                r = torch.matmul(a.t(), full)
                if residual is not None:
                    r = r + residual
                if out is not None:
                    out.copy_(r)
                    return out
                return r
            return _g.matmul_tn(a, full, residual=residual, out=out)
        if self.backend != "fused":
            dy = torch.empty((T, N), dtype=BF, device=self.dev)
            dist.all_gather_into_tensor(dy, dy_shard.contiguous(), group=self.group)
            r = torch.matmul(a.t(), dy)
            if residual is not None:
                r = r + residual
            if out is not None:
                out.copy_(r)
                return out
            return r
        if self.direct_wgrad:
            if out is None:
                out = torch.empty((M, N), dtype=BF, device=self.dev)
            return self._call(a, dy_shard, out, residual, M, N, T, True, True, False, True, False)
        dy = torch.empty((T, N), dtype=BF, device=self.dev)
        dist.all_gather_into_tensor(dy, dy_shard.contiguous(), group=self.group)
        return _g.matmul_tn(a, dy, residual=residual, out=out)

    def close(self):
        if self.region is not None:
            self.region.close()
            self.region = None

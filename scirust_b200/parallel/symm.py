"""Symmetric (peer-mapped) device memory for kernels that read and write other GPUs directly.

Every rank of a process group allocates a region of the same size with ``cudaMalloc`` (outside
the PyTorch caching allocator, because the whole allocation is exported), exchanges CUDA IPC
handles through the group, and maps each peer's region. ``SymmetricRegion.tensor(...)`` carves
torch tensors out of the local region; ``peer_ptr(rank, tensor)`` is the address of the same
bytes in a peer's region. A small flag area at the end of the region carries the epochs of the
kernels' start/finish protocol (csrc/comm.cu).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib

_lib.register("sb_malloc", [_lib.sz, C.POINTER(C.c_void_p)])
_lib.register("sb_free", [_lib.vp])
_lib.register("sb_memset", [_lib.vp, _lib.i32, _lib.sz, _lib.vp])
_lib.register("sb_ipc_get_handle", [_lib.vp, _lib.vp])
_lib.register("sb_ipc_open", [_lib.vp, C.POINTER(C.c_void_p)])
_lib.register("sb_ipc_close", [_lib.vp])

FLAG_SLOTS = 256
ALIGN = 1024


class _Raw:
    """Exposes a raw device allocation through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricRegion:
    def __init__(self, group, nbytes: int, device=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        lib = _lib.cuda()
        self.words_per_slot = lib.sb_flag_words_per_slot()
        self.flag_bytes = FLAG_SLOTS * self.words_per_slot * 4
        self.data_bytes = (nbytes + ALIGN - 1) // ALIGN * ALIGN
        total = self.data_bytes + self.flag_bytes
        p = C.c_void_p()
        _lib.check(lib.sb_malloc(total, C.byref(p)), "sb_malloc")
        self.base = p.value
        self.total = total
        _lib.check(lib.sb_memset(self.base, 0, total, None), "sb_memset")
        torch.cuda.synchronize()
        hsize = lib.sb_ipc_handle_size()
        hbuf = (C.c_char * hsize)()
        _lib.check(lib.sb_ipc_get_handle(self.base, hbuf), "cudaIpcGetMemHandle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(hbuf.raw), group=group)
        self.peer_base = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self.base)
            else:
                q = C.c_void_p()
                _lib.check(lib.sb_ipc_open(C.create_string_buffer(h, hsize), C.byref(q)), "cudaIpcOpenMemHandle")
                self.peer_base.append(q.value)
        self._bytes = torch.as_tensor(_Raw(self.base, total), device=self.device)
        self._cursor = 0
        self._carved = []
        self._next_slot = 0
        dist.barrier(group=group)

    # -- carving ---------------------------------------------------------------------------
    def tensor(self, shape, dtype) -> torch.Tensor:
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self._cursor + 255) // 256 * 256
        if start + nbytes > self.data_bytes:
            raise MemoryError("symmetric region exhausted")
        self._cursor = start + nbytes
        # a separate storage object per carve-out: views of one base tensor would share a version
        # counter, and autograd would then see every in-place write to one buffer as a change of all
        raw = torch.as_tensor(_Raw(self.base + start, nbytes), device=self.device)
        self._carved.append(raw)
        return raw.view(dtype).view(shape)

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.total:
            raise ValueError("tensor does not live in this symmetric region")
        return off

    def peer_ptr(self, rank: int, t: torch.Tensor) -> int:
        return self.peer_base[rank] + self.offset_of(t)

    def peer_ptrs(self, t: torch.Tensor):
        """ctypes array of the W addresses of ``t`` (one per rank)."""
        off = self.offset_of(t)
        return (C.c_void_p * self.world)(*[b + off for b in self.peer_base])

    def flag_ptrs(self):
        return (C.c_void_p * self.world)(*[b + self.data_bytes for b in self.peer_base])

    def local_flags(self) -> torch.Tensor:
        return self._bytes[self.data_bytes:].view(torch.int32)

    def new_slot(self) -> int:
        s = self._next_slot
        if s >= FLAG_SLOTS:
            raise RuntimeError("out of flag slots")
        self._next_slot += 1
        return s

    def close(self):
        """Collective: every rank must call it. Peers are unmapped only after all ranks have
        drained their streams, and the local region is freed only after all peers unmapped it."""
        lib = _lib.cuda()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for r, b in enumerate(self.peer_base):
            if r != self.rank and b:
                lib.sb_ipc_close(b)
        self.peer_base = []
        dist.barrier(group=self.group)
        if self.base:
            self._bytes = None
            self._carved = []
            lib.sb_free(self.base)
            self.base = 0

"""Typed, page-locked host buffers and a fixed pool of them for staging host <-> device copies.

A copy between pageable host memory and a GPU is staged by the driver and cannot overlap with compute; from page-locked
memory it is one DMA that runs beside the kernels. ``PinnedBuffer`` is a zero-initialised tensor of a fixed element type
and length, page-locked when a CUDA runtime is present (best effort: ``is_pinned`` says what was obtained) and 64-byte
aligned. ``PinnedPool`` pre-allocates ``capacity`` buffers; ``borrow`` hands one out, ``release`` takes it back and refuses
buffers of another pool or double releases; nothing is allocated after construction, so a training loop's input pipeline
never meets the allocator. ``stage_to_device`` / ``DoubleBufferedUploader`` are the two-deep upload pipeline built on it.
Reference counterpart: scirust-core/src/tensor/pinned.rs:12-357 (``PinnedBuffer<T>``, ``PinnedPool<T>``, ``PooledBuffer<T>``,
``MemoryLayout``).
"""
from __future__ import annotations

import enum
import itertools

import torch


class PinError(RuntimeError):
    pass


class MemoryLayout(enum.Enum):
    CPU = "cpu"
    PINNED = "pinned"
    GPU_UNIFIED = "gpu-unified"


_MAX_BYTES = 1 << 46


class PinnedBuffer:
    def __init__(self, length: int, dtype: torch.dtype = torch.float32):
        item = torch.empty(0, dtype=dtype).element_size()
        if length < 0 or length * item > _MAX_BYTES:
            raise PinError(f"size {length * item} bytes is invalid or too large")
        t = torch.zeros(length, dtype=dtype)
        self.pinned = False
        if torch.cuda.is_available() and length:
            try:
                t = t.pin_memory()
                self.pinned = True
            except RuntimeError:
                self.pinned = False
        self.t = t

    def __len__(self):
        return self.t.numel()

    def len_bytes(self) -> int:
        return self.t.numel() * self.t.element_size()

    def is_pinned(self) -> bool:
        return self.pinned

    def is_empty(self) -> bool:
        return self.t.numel() == 0

    def is_aligned(self, alignment: int = 64) -> bool:
        return self.t.numel() == 0 or self.t.data_ptr() % alignment == 0

    def layout(self) -> MemoryLayout:
        return MemoryLayout.PINNED if self.pinned else MemoryLayout.CPU

    def as_tensor(self) -> torch.Tensor:
        return self.t


_pool_ids = itertools.count(1)


class PooledBuffer:
    def __init__(self, buffer: PinnedBuffer, index: int, pool_id: int):
        self._buffer, self.index, self._pool_id = buffer, index, pool_id

    def __len__(self):
        return 0 if self._buffer is None else len(self._buffer)

    def len_bytes(self) -> int:
        return 0 if self._buffer is None else self._buffer.len_bytes()

    def as_tensor(self) -> torch.Tensor:
        if self._buffer is None:
            raise PinError("pooled buffer released")
        return self._buffer.t


class PinnedPool:
    def __init__(self, capacity: int, elem_count: int, dtype: torch.dtype = torch.float32):
        self.id = next(_pool_ids)
        self._buffers = [PinnedBuffer(elem_count, dtype) for _ in range(capacity)]
        self._free = list(range(capacity))

    def borrow(self) -> PooledBuffer:
        if not self._free:
            raise PinError("memory allocation failed")           # the pool is fixed: exhaustion is an allocation failure
        i = self._free.pop()
        buf, self._buffers[i] = self._buffers[i], None
        return PooledBuffer(buf, i, self.id)

    def release(self, borrowed: PooledBuffer) -> None:
        if (borrowed._pool_id != self.id or borrowed.index >= len(self._buffers) or self._buffers[borrowed.index] is not None
                or borrowed._buffer is None):
            raise PinError("buffer does not belong to this pool")
        self._buffers[borrowed.index], borrowed._buffer = borrowed._buffer, None
        self._free.append(borrowed.index)

    def available(self) -> int:
        return len(self._free)

    def capacity(self) -> int:
        return len(self._buffers)


def stage_to_device(host: torch.Tensor, staging: PooledBuffer, device, stream=None, out=None) -> torch.Tensor:
    """Copy ``host`` into the staging buffer, then asynchronously to ``device`` (on ``stream`` when given)."""
    n = host.numel()
    st = staging.as_tensor()
    if n > st.numel() or host.dtype != st.dtype:
        raise PinError(f"staging buffer holds {st.numel()} {st.dtype} elements; asked for {n} {host.dtype}")
    st[:n].copy_(host.reshape(-1))
    dst = out if out is not None else torch.empty(host.shape, dtype=host.dtype, device=device)
    if stream is not None and torch.cuda.is_available():
        with torch.cuda.stream(stream):
            dst.reshape(-1).copy_(st[:n], non_blocking=True)
    else:
        dst.reshape(-1).copy_(st[:n], non_blocking=True)
    return dst


class DoubleBufferedUploader:
    """Two staging buffers and two device buffers: batch k + 1 is staged and copied while batch k computes.
    ``submit(host)`` starts an upload and returns a ticket; ``take(ticket)`` makes the compute stream wait for that upload
    and returns the device tensor, recycling its staging buffer."""

    def __init__(self, elem_count: int, dtype, device, depth: int = 2):
        self.pool = PinnedPool(depth, elem_count, dtype)
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda" and torch.cuda.is_available()
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._dev = [torch.empty(elem_count, dtype=dtype, device=self.device) for _ in range(depth)]
        self._inflight = {}
        self._tickets = itertools.count()

    def submit(self, host: torch.Tensor) -> int:
        staging = self.pool.borrow()
        dev = self._dev[staging.index][: host.numel()].reshape(host.shape)
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))      # the previous user of this slot is done
        stage_to_device(host, staging, self.device, self.stream, dev)
        ev = None
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self.stream)
        t = next(self._tickets)
        self._inflight[t] = (staging, dev, ev)
        return t

    def take(self, ticket: int) -> torch.Tensor:
        if ticket not in self._inflight:
            raise PinError("unknown or already taken upload ticket")
        staging, dev, ev = self._inflight.pop(ticket)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        self.pool.release(staging)
        return dev

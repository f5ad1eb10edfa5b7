"""Transfer requests and caller-owned kernel workspaces.

A ``TransferRequest`` names where a tensor lives and where it should go (host, pinned host, a device, unified, a peer
device), its element type, byte length and whether it is synchronous or ordered on a stream; identical source and
destination are refused; ``canonical_record`` is a stable one-line description for logs and attestations.
A ``WorkspaceSpec`` is the (size, alignment) a kernel needs; specs compose with ``then`` (the second part aligned inside
the first), and ``KernelWorkspace`` validates a caller's buffer ONCE before a hot loop uses it without further checks
(size and base-address alignment; on a GPU the buffer is a byte tensor).
Reference counterpart: scirust-compute/src/{transfer,workspace}.rs.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .contracts import ComputeError, DeviceId, DType, MemorySpace, StreamId

TRANSFER_CONTRACT_VERSION = 1
DTYPE_CONTRACT_VERSION = 1


@dataclass(frozen=True)
class TensorResidency:
    space: MemorySpace
    device: DeviceId | None = None

    def __post_init__(self):
        needs = self.space in (MemorySpace.DEVICE, MemorySpace.UNIFIED, MemorySpace.PEER_DEVICE)
        if needs != (self.device is not None):
            raise ComputeError("device residencies name their device; host residencies do not")

    @staticmethod
    def host():
        return TensorResidency(MemorySpace.HOST)

    @staticmethod
    def host_pinned():
        return TensorResidency(MemorySpace.HOST_PINNED)

    @staticmethod
    def on(device: DeviceId):
        return TensorResidency(MemorySpace.DEVICE, device)

    def record(self) -> str:
        return self.space.value if self.device is None else f"{self.space.value}:{self.device.record()}"


class TransferKind(enum.Enum):
    SYNCHRONOUS = "sync"
    ASYNCHRONOUS = "async"


@dataclass(frozen=True)
class TransferMode:
    kind: TransferKind = TransferKind.SYNCHRONOUS
    stream: StreamId | None = None

    def __post_init__(self):
        if (self.kind is TransferKind.ASYNCHRONOUS) != (self.stream is not None):
            raise ComputeError("an asynchronous transfer names its stream; a synchronous one has none")

    @staticmethod
    def on_stream(stream: StreamId) -> "TransferMode":
        return TransferMode(TransferKind.ASYNCHRONOUS, stream)


class TransferRequestError(ComputeError):
    pass


@dataclass(frozen=True)
class TransferRequest:
    source: TensorResidency
    destination: TensorResidency
    dtype: DType
    byte_len: int
    mode: TransferMode = TransferMode()

    def __post_init__(self):
        if self.source == self.destination:
            raise TransferRequestError(f"transfer source and destination are identical: {self.source.record()}")
        if self.byte_len < 0 or self.byte_len % self.dtype.size_bytes():
            raise TransferRequestError("byte length must be a non-negative multiple of the element size")

    def crosses_nvlink(self) -> bool:
        d = {self.source.device, self.destination.device} - {None}
        return len(d) == 2

    def wants_pinned_host(self) -> bool:
        """An asynchronous host <-> device copy only overlaps with compute from page-locked host memory."""
        host = MemorySpace.HOST in (self.source.space, self.destination.space)
        return host and self.mode.kind is TransferKind.ASYNCHRONOUS

    def canonical_record(self) -> str:
        stream = "none" if self.mode.stream is None else str(self.mode.stream.value)
        return (f"scirust-transfer-v{TRANSFER_CONTRACT_VERSION};dtype_version={DTYPE_CONTRACT_VERSION};dtype={self.dtype.label};"
                f"bytes={self.byte_len};source={self.source.record()};destination={self.destination.record()};"
                f"mode={self.mode.kind.value};stream={stream}")


class WorkspaceError(ComputeError):
    pass


def _align_up(v: int, a: int) -> int:
    return (v + a - 1) & ~(a - 1)


@dataclass(frozen=True)
class WorkspaceSpec:
    size_bytes: int
    align_bytes: int = 1

    def __post_init__(self):
        if self.align_bytes <= 0 or self.align_bytes & (self.align_bytes - 1):
            raise WorkspaceError("workspace alignment must be a non-zero power of two")
        if self.size_bytes < 0:
            raise WorkspaceError("workspace size must be non-negative")

    @staticmethod
    def empty() -> "WorkspaceSpec":
        return WorkspaceSpec(0, 1)

    def is_empty(self) -> bool:
        return self.size_bytes == 0

    def then(self, nxt: "WorkspaceSpec") -> "WorkspaceSpec":
        return WorkspaceSpec(_align_up(self.size_bytes, nxt.align_bytes) + nxt.size_bytes, max(self.align_bytes, nxt.align_bytes))

    def offset_of_next(self, nxt: "WorkspaceSpec") -> int:
        return _align_up(self.size_bytes, nxt.align_bytes)


class KernelWorkspace:
    """A validated view of the first ``spec.size_bytes`` bytes of a caller's buffer (torch byte tensor, bytearray or
    anything exposing ``data_ptr()`` / the buffer protocol)."""

    def __init__(self, buffer, spec: WorkspaceSpec):
        if hasattr(buffer, "data_ptr"):
            n, addr = buffer.numel() * buffer.element_size(), buffer.data_ptr()
        else:
            import ctypes
            mv = memoryview(buffer)
            n = mv.nbytes
            addr = ctypes.addressof(ctypes.c_char.from_buffer(buffer)) if n and not mv.readonly else 0
        if n < spec.size_bytes:
            raise WorkspaceError(f"workspace too small: requires {spec.size_bytes} bytes, got {n}")
        if spec.size_bytes and addr % spec.align_bytes:
            raise WorkspaceError(f"workspace base is not aligned to {spec.align_bytes} bytes (remainder {addr % spec.align_bytes})")
        self.buffer, self.spec, self.address = buffer, spec, addr

    def __len__(self):
        return self.spec.size_bytes

    def view(self):
        return self.buffer[: self.spec.size_bytes]

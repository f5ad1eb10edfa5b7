"""Backend-neutral value types of the compute layer: element types, device identities, memory spaces, checked shapes
and strides, tensor specifications, kernel modules, launch configurations and buffer bindings. Everything validates on
construction and raises ``ComputeError`` with the reason; nothing here touches a device.

Formats: ``KernelFormat.REFERENCE`` (a named host kernel of the reference backend), ``CUDA_C`` (source for NVRTC under the
strict-IEEE option set), ``PTX`` and ``CUBIN`` (prebuilt sm_100a code). Shader formats of graphics APIs are not part of
this framework. Reference counterpart: scirust-compute/src/{dtype,device,memory,shape,strides,tensor,kernel,launch,
binding,ids,error}.rs.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass


class ComputeError(Exception):
    pass


class DType(enum.Enum):
    BOOL = ("bool", 1)
    U8 = ("u8", 1)
    I8 = ("i8", 1)
    U16 = ("u16", 2)
    I16 = ("i16", 2)
    F16 = ("f16", 2)
    BF16 = ("bf16", 2)
    U32 = ("u32", 4)
    I32 = ("i32", 4)
    F32 = ("f32", 4)
    U64 = ("u64", 8)
    I64 = ("i64", 8)
    F64 = ("f64", 8)
    F8E4M3 = ("f8e4m3", 1)        # Blackwell tensor-core operand formats
    F8E5M2 = ("f8e5m2", 1)

    @property
    def label(self) -> str:
        return self.value[0]

    def size_bytes(self) -> int:
        return self.value[1]

    def torch_dtype(self):
        import torch
        return {"bool": torch.bool, "u8": torch.uint8, "i8": torch.int8, "i16": torch.int16, "f16": torch.float16,
                "bf16": torch.bfloat16, "i32": torch.int32, "f32": torch.float32, "i64": torch.int64, "f64": torch.float64,
                "u16": torch.uint16, "u32": torch.uint32, "u64": torch.uint64, "f8e4m3": torch.float8_e4m3fn,
                "f8e5m2": torch.float8_e5m2}[self.label]


class DeviceKind(enum.Enum):
    REFERENCE = "reference"
    CPU = "cpu"
    CUDA = "cuda"


@dataclass(frozen=True)
class DeviceId:
    kind: DeviceKind
    ordinal: int = 0

    def __lt__(self, other):
        return (self.kind.value, self.ordinal) < (other.kind.value, other.ordinal)

    @staticmethod
    def reference() -> "DeviceId":
        return DeviceId(DeviceKind.REFERENCE, 0)

    @staticmethod
    def cpu() -> "DeviceId":
        return DeviceId(DeviceKind.CPU, 0)

    @staticmethod
    def cuda(ordinal: int = 0) -> "DeviceId":
        return DeviceId(DeviceKind.CUDA, ordinal)

    def record(self) -> str:
        return f"{self.kind.value}:{self.ordinal}"


class MemorySpace(enum.Enum):
    HOST = "host"
    HOST_PINNED = "host-pinned"
    DEVICE = "device"
    UNIFIED = "unified"
    PEER_DEVICE = "peer-device"        # another GPU's memory mapped over NVLink (symmetric / IPC mappings)


class Layout(enum.Enum):
    CONTIGUOUS_ROW_MAJOR = "contiguous"
    STRIDED = "strided"


_USIZE_MAX = (1 << 64) - 1


@dataclass(frozen=True)
class Shape:
    dims: tuple

    def __post_init__(self):
        object.__setattr__(self, "dims", tuple(int(d) for d in self.dims))
        if any(d < 0 for d in self.dims):
            raise ComputeError("shape dimensions must be non-negative")

    def rank(self) -> int:
        return len(self.dims)

    def checked_num_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
            if n > _USIZE_MAX:
                raise ComputeError("element count overflows the address space")
        return n


@dataclass(frozen=True)
class Strides:
    elems: tuple

    @staticmethod
    def contiguous(shape: Shape) -> "Strides":
        shape.checked_num_elements()
        out, acc = [], 1
        for d in reversed(shape.dims):
            out.append(acc)
            acc *= max(d, 1)
        return Strides(tuple(reversed(out)))

    def is_contiguous_for(self, shape: Shape) -> bool:
        return self.elems == Strides.contiguous(shape).elems


@dataclass(frozen=True)
class TensorSpec:
    dtype: DType
    shape: Shape
    strides: Strides
    layout: Layout
    device: DeviceId

    @staticmethod
    def contiguous(dtype: DType, shape: Shape, device: DeviceId) -> "TensorSpec":
        return TensorSpec(dtype, shape, Strides.contiguous(shape), Layout.CONTIGUOUS_ROW_MAJOR, device)

    def checked_byte_len(self) -> int:
        n = self.shape.checked_num_elements() * self.dtype.size_bytes()
        if n > _USIZE_MAX:
            raise ComputeError("byte size overflows the address space")
        return n

    def tma_ok(self) -> bool:
        """Whether a tiled bulk-tensor copy can describe this tensor: unit innermost stride, every outer stride and the
        innermost extent a multiple of 16 bytes."""
        if not self.shape.dims or self.strides.elems[-1] != 1:
            return False
        b = self.dtype.size_bytes()
        return (self.shape.dims[-1] * b) % 16 == 0 and all((s * b) % 16 == 0 for s in self.strides.elems[:-1])


class KernelFormat(enum.Enum):
    REFERENCE = "reference"
    CUDA_C = "cuda-c"
    PTX = "ptx"
    CUBIN = "cubin"


@dataclass(frozen=True)
class KernelModule:
    format: KernelFormat
    entry_point: str
    code: bytes

    def __post_init__(self):
        if not self.entry_point:
            raise ComputeError("kernel entry point must not be empty")
        code = self.code.encode() if isinstance(self.code, str) else bytes(self.code)
        if not code:
            raise ComputeError("kernel module code must not be empty")
        object.__setattr__(self, "code", code)


@dataclass(frozen=True)
class LaunchConfig:
    grid: tuple
    block: tuple
    shared_memory_bytes: int = 0
    cluster: tuple = (1, 1, 1)         # thread-block cluster shape (portable limit: 8 CTAs)

    def __post_init__(self):
        if len(self.grid) != 3 or len(self.block) != 3 or len(self.cluster) != 3:
            raise ComputeError("grid, block and cluster must have three dimensions")
        if 0 in self.grid:
            raise ComputeError("grid dimensions must be non-zero")
        if 0 in self.block:
            raise ComputeError("block dimensions must be non-zero")
        if 0 in self.cluster or any(g % c for g, c in zip(self.grid, self.cluster)):
            raise ComputeError("cluster dimensions must be non-zero and divide the grid")
        if self.shared_memory_bytes < 0:
            raise ComputeError("shared memory size must be non-negative")


class BufferAccess(enum.Enum):
    READ_ONLY = "read"
    WRITE_ONLY = "write"
    READ_WRITE = "read_write"

    @property
    def writes(self) -> bool:
        return self is not BufferAccess.READ_ONLY


@dataclass
class BufferBinding:
    slot: int
    buffer: object
    offset_bytes: int
    length_bytes: int
    access: BufferAccess


@dataclass(frozen=True)
class StreamId:
    value: int


@dataclass(frozen=True)
class EventId:
    value: int

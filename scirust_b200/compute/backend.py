"""The backend contract and its two implementations.

``ComputeBackend``: ``capabilities`` / ``hardware_capabilities`` / ``execution_limits``; ``allocate(bytes, alignment,
space)``, ``write`` / ``read`` with offsets, ``compile(KernelModule)``, ``create_stream``, ``launch(kernel, stream,
LaunchConfig, bindings)`` returning an event, ``wait(event)``, ``synchronize(stream)``. Every launch is validated first:
bindings inside their buffers, non-empty, and no WRITE binding overlapping any other binding of the same allocation.

* ``ReferenceBackend``: host memory (bytearrays), kernels are named host functions (``KernelFormat.REFERENCE``; the code
  bytes are the name of a registered function) that receive NumPy views of the bound ranges; launches run to completion,
  events are already signalled. It is the oracle the CUDA backend is compared with, and counts launches so a test can
  tell a kernel really ran.
* ``CudaBackend``: one GPU through the raw runtime: ``CUDA_C`` modules are compiled by NVRTC under the strict-IEEE
  option set for the device's own architecture, launches go to real streams, events are CUDA events. Pinned-host and
  device spaces are allocated through the framework's caching allocator.
Reference counterpart: scirust-compute/src/{backend,backend_layers}.rs and the adapters in scirust-gpu/src/{compute_adapter,
cuda_compute_adapter}.rs.
"""
from __future__ import annotations

import abc

import numpy as np

from .contracts import (BufferAccess, BufferBinding, ComputeError, DeviceId, DType, EventId, KernelFormat, KernelModule,
                        LaunchConfig, MemorySpace, StreamId)
from .hardware import DeviceCapabilities, ExecutionLimits, HardwareCapabilities, probe_host_cpu


def validate_bindings(bindings, size_of) -> None:
    spans = []
    for i, b in enumerate(bindings):
        if b.offset_bytes < 0 or b.length_bytes <= 0:
            raise ComputeError(f"binding {i}: range must be non-empty and start at a non-negative offset")
        if b.offset_bytes + b.length_bytes > size_of(b.buffer):
            raise ComputeError(f"binding {i}: range exceeds buffer bounds")
        spans.append((id(b.buffer), b.offset_bytes, b.offset_bytes + b.length_bytes, b.access.writes, i))
    slots = [b.slot for b in bindings]
    if len(set(slots)) != len(slots):
        raise ComputeError("binding slots must be unique")
    for a in spans:
        if not a[3]:
            continue
        for o in spans:
            if o[4] != a[4] and o[0] == a[0] and a[1] < o[2] and o[1] < a[2]:
                raise ComputeError(f"binding {a[4]} writes bytes that binding {o[4]} also touches (aliasing)")


class ComputeBackend(abc.ABC):
    @abc.abstractmethod
    def capabilities(self) -> DeviceCapabilities: ...

    def hardware_capabilities(self) -> HardwareCapabilities:
        return self.capabilities().hardware_baseline()

    def execution_limits(self) -> ExecutionLimits:
        return ExecutionLimits.from_device_capabilities(self.capabilities())

    @abc.abstractmethod
    def allocate(self, nbytes: int, alignment: int = 1, memory_space: MemorySpace = MemorySpace.DEVICE): ...

    @abc.abstractmethod
    def write(self, destination, offset_bytes: int, data: bytes) -> None: ...

    @abc.abstractmethod
    def read(self, source, offset_bytes: int, nbytes: int) -> bytes: ...

    @abc.abstractmethod
    def compile(self, module: KernelModule): ...

    @abc.abstractmethod
    def create_stream(self): ...

    @abc.abstractmethod
    def launch(self, kernel, stream, config: LaunchConfig, bindings, scalars=()): ...

    @abc.abstractmethod
    def wait(self, event) -> None: ...

    @abc.abstractmethod
    def synchronize(self, stream) -> None: ...


def _check_alloc(nbytes, alignment):
    if nbytes <= 0:
        raise ComputeError("allocation size must be positive")
    if alignment <= 0 or alignment & (alignment - 1):
        raise ComputeError("alignment must be a power of two")


class ReferenceBackend(ComputeBackend):
    KERNELS: dict = {}

    def __init__(self):
        self.launches = 0
        self._streams = 0
        self._events = 0

    @classmethod
    def register(cls, name: str):
        def deco(fn):
            cls.KERNELS[name] = fn
            return fn
        return deco

    def capabilities(self):
        return DeviceCapabilities.reference_cpu()

    def hardware_capabilities(self):
        hw = probe_host_cpu()
        hw.device = DeviceId.reference()
        return hw

    def allocate(self, nbytes, alignment=1, memory_space=MemorySpace.HOST):
        _check_alloc(nbytes, alignment)
        if memory_space not in (MemorySpace.HOST, MemorySpace.HOST_PINNED):
            raise ComputeError(f"the reference backend has no {memory_space.value} memory")
        return bytearray(nbytes)

    def write(self, destination, offset_bytes, data):
        if offset_bytes < 0 or offset_bytes + len(data) > len(destination):
            raise ComputeError("write exceeds buffer bounds")
        destination[offset_bytes:offset_bytes + len(data)] = data

    def read(self, source, offset_bytes, nbytes):
        if offset_bytes < 0 or nbytes < 0 or offset_bytes + nbytes > len(source):
            raise ComputeError("read exceeds buffer bounds")
        return bytes(source[offset_bytes:offset_bytes + nbytes])

    def compile(self, module: KernelModule):
        if module.format is not KernelFormat.REFERENCE:
            raise ComputeError(f"the reference backend cannot run {module.format.value} modules")
        name = module.code.decode()
        if name not in self.KERNELS:
            raise ComputeError(f"unknown reference kernel {name!r}")
        return (module.entry_point, self.KERNELS[name])

    def create_stream(self):
        self._streams += 1
        return StreamId(self._streams)

    def launch(self, kernel, stream, config, bindings, scalars=()):
        validate_bindings(bindings, len)
        views = {}
        for b in sorted(bindings, key=lambda b: b.slot):
            v = np.frombuffer(b.buffer, dtype=np.uint8, count=b.length_bytes, offset=b.offset_bytes)
            if not b.access.writes:
                v = v.copy()
                v.flags.writeable = False
            views[b.slot] = v
        kernel[1](config, views, *scalars)
        self.launches += 1
        self._events += 1
        return EventId(self._events)

    def wait(self, event):
        return None

    def synchronize(self, stream):
        return None


@ReferenceBackend.register("axpy_f32")
def _axpy(config, views, alpha=1.0):
    """slot 0: x (read), slot 1: y (read-write); y <- alpha * x + y."""
    x, y = views[0].view(np.float32), views[1].view(np.float32)
    y += np.float32(alpha) * x


@ReferenceBackend.register("relu_f32")
def _relu(config, views):
    x, y = views[0].view(np.float32), views[1].view(np.float32)
    np.maximum(x, np.float32(0), out=y)


class CudaBackend(ComputeBackend):
    def __init__(self, ordinal: int = 0):
        from ..runtime.raw import RawRuntime
        import torch
        self.torch = torch
        self.rt = RawRuntime(ordinal)
        self.ordinal = ordinal
        self.launches = 0

    def capabilities(self):
        p = self.torch.cuda.get_device_properties(self.ordinal)
        return DeviceCapabilities(DeviceId.cuda(self.ordinal), p.name,
                                  [DType.BOOL, DType.U8, DType.I8, DType.I16, DType.F16, DType.BF16, DType.I32, DType.F32, DType.I64,
                                   DType.F64, DType.F8E4M3, DType.F8E5M2], p.total_memory, (1024, 1024, 64), True)

    def hardware_capabilities(self):
        from .hardware import probe_cuda
        return probe_cuda(self.ordinal)

    def execution_limits(self):
        from .hardware import cuda_limits
        return cuda_limits(self.ordinal)

    def allocate(self, nbytes, alignment=256, memory_space=MemorySpace.DEVICE):
        _check_alloc(nbytes, alignment)
        if memory_space is MemorySpace.DEVICE:
            buf = self.rt.allocate(nbytes)
        elif memory_space is MemorySpace.HOST_PINNED:
            from ..runtime.raw import RawBuffer
            buf = RawBuffer(nbytes, self.torch.zeros(nbytes, dtype=self.torch.uint8).pin_memory())
        else:
            raise ComputeError(f"the CUDA backend does not allocate {memory_space.value} memory")
        if buf.ptr % alignment:
            raise ComputeError(f"allocator returned a base not aligned to {alignment} bytes")
        return buf

    def write(self, destination, offset_bytes, data):
        self.rt.write(destination, bytes(data), offset_bytes)

    def read(self, source, offset_bytes, nbytes):
        return self.rt.read(source, offset_bytes, nbytes)

    def compile(self, module: KernelModule):
        if module.format is not KernelFormat.CUDA_C:
            raise ComputeError(f"the CUDA backend compiles cuda-c modules; got {module.format.value}")
        return self.rt.compile(module.code.decode(), module.entry_point)

    def create_stream(self):
        return self.torch.cuda.Stream(device=self.rt.device)

    def launch(self, kernel, stream, config, bindings, scalars=()):
        from ..runtime.raw import RawAccess, RawBinding, RawLaunchConfig
        validate_bindings(bindings, lambda b: b.logical_bytes)
        if config.cluster != (1, 1, 1):
            raise ComputeError("cluster launches go through the framework's own kernels, not through raw modules")
        acc = {BufferAccess.READ_ONLY: RawAccess.READ, BufferAccess.WRITE_ONLY: RawAccess.WRITE, BufferAccess.READ_WRITE: RawAccess.READ_WRITE}
        raw = [RawBinding(b.buffer, acc[b.access], b.offset_bytes, b.length_bytes) for b in sorted(bindings, key=lambda b: b.slot)]
        with self.torch.cuda.stream(stream):
            ev = self.rt.launch(kernel, RawLaunchConfig(tuple(config.grid), tuple(config.block), config.shared_memory_bytes), raw, scalars)
        self.launches += 1
        return ev

    def wait(self, event):
        event.synchronize()

    def synchronize(self, stream):
        stream.synchronize()

"""Raw CUDA runtime: explicit buffers, run-time compiled kernels with pinned IEEE options, validated launches.

The generic layer under the operator library, for code that brings its own CUDA C (the canonical reference
adapter, user kernels, experiments): one context and one ordered stream, ``allocate`` / ``write`` / ``read``,
``compile_cuda_c`` through NVRTC for ``compute_100a`` with the four floating-point options pinned
(``--ftz=false --prec-sqrt=true --prec-div=true --fmad=false``: IEEE results that do not depend on contraction or
fast division), and ``launch`` with the checks a generic launcher owes its callers before anything reaches the GPU:

* geometry: no zero dimension, grid / block dimensions, threads per block and dynamic shared memory within the
  device's limits;
* bindings: every ``(buffer, offset, length)`` lies inside its allocation and is not empty;
* aliasing: bindings that name the SAME allocation form a group; a group with a writer may not contain any other
  binding whose byte range overlaps the writer's (two readers may share bytes; disjoint ranges of one allocation may
  be read and written in one launch). Identity is the allocation object, never an address comparison across
  allocations.

Counterpart of the reference's ``CudaRawRuntime`` (scirust-cuda/src/raw_runtime.rs:153-659: options table :308-323,
``compile_cuda_c`` :348-405, ``launch`` :438-580, ``validate_launch`` :598-659). Validation and compilation need no
GPU; allocation, copies and launches do.
"""
from __future__ import annotations

import ctypes as C
import enum
import glob
from dataclasses import dataclass

STRICT_IEEE_OPTIONS = ("--ftz=false", "--prec-sqrt=true", "--prec-div=true", "--fmad=false")
DEFAULT_ARCH = "compute_100a"

# Limits of a B200 (sm_100a); a live runtime replaces them with what the driver reports.
DEFAULT_LIMITS = {"max_grid": (2**31 - 1, 65535, 65535), "max_block": (1024, 1024, 64), "max_threads": 1024,
                  "max_smem": 227 * 1024}


class RawError(RuntimeError):
    pass


class RawAccess(enum.Enum):
    READ = "read"
    WRITE = "write"
    READ_WRITE = "read_write"

    @property
    def writes(self) -> bool:
        return self is not RawAccess.READ


@dataclass(frozen=True)
class RawLaunchConfig:
    grid: tuple
    block: tuple
    shared_memory_bytes: int = 0


class RawBuffer:
    """One device allocation of ``nbytes`` (a torch byte tensor keeps it alive)."""

    def __init__(self, nbytes: int, tensor=None):
        self.logical_bytes = int(nbytes)
        self.tensor = tensor

    @property
    def ptr(self) -> int:
        if self.tensor is None:
            raise RawError("buffer has no device storage (validation-only buffer)")
        return self.tensor.data_ptr()

    def same_allocation(self, other: "RawBuffer") -> bool:
        return self is other


@dataclass
class RawBinding:
    buffer: RawBuffer
    access: RawAccess
    offset_bytes: int = 0
    length_bytes: int | None = None

    def span(self):
        n = self.buffer.logical_bytes - self.offset_bytes if self.length_bytes is None else self.length_bytes
        return self.offset_bytes, self.offset_bytes + n


def validate_launch_geometry(cfg: RawLaunchConfig, limits: dict = DEFAULT_LIMITS) -> None:
    if len(cfg.grid) != 3 or len(cfg.block) != 3:
        raise RawError("grid and block must have three dimensions")
    if 0 in cfg.grid:
        raise RawError("CUDA grid dimensions must be non-zero")
    if 0 in cfg.block:
        raise RawError("CUDA block dimensions must be non-zero")
    for ax in range(3):
        if cfg.grid[ax] < 0 or cfg.grid[ax] > limits["max_grid"][ax]:
            raise RawError(f"CUDA grid dimension {ax} exceeds the device limit")
        if cfg.block[ax] < 0 or cfg.block[ax] > limits["max_block"][ax]:
            raise RawError(f"CUDA block dimension {ax} exceeds the device limit")
    threads = cfg.block[0] * cfg.block[1] * cfg.block[2]
    if threads > limits["max_threads"]:
        raise RawError(f"CUDA block requests {threads} threads, device limit is {limits['max_threads']}")
    if cfg.shared_memory_bytes < 0 or cfg.shared_memory_bytes > limits["max_smem"]:
        raise RawError(f"CUDA launch requests {cfg.shared_memory_bytes} shared-memory bytes, device limit is "
                       f"{limits['max_smem']}")


def validate_bindings(bindings) -> None:
    for i, b in enumerate(bindings):
        lo, hi = b.span()
        if lo < 0 or hi < lo:
            raise RawError(f"binding {i}: CUDA binding range overflow")
        if hi > b.buffer.logical_bytes:
            raise RawError(f"binding {i}: CUDA binding exceeds buffer bounds")
        if hi == lo:
            raise RawError(f"binding {i}: CUDA binding length must be non-zero")


def validate_alias_groups(bindings) -> None:
    """Group bindings by allocation in first-appearance order; inside a group a writer's bytes may not be touched by
    any other binding."""
    groups: list = []
    for i, b in enumerate(bindings):
        for g in groups:
            if bindings[g[0]].buffer.same_allocation(b.buffer):
                g.append(i)
                break
        else:
            groups.append([i])
    for g in groups:
        for x in g:
            if not bindings[x].access.writes:
                continue
            wlo, whi = bindings[x].span()
            for y in g:
                if y == x:
                    continue
                lo, hi = bindings[y].span()
                if lo < whi and wlo < hi:
                    raise RawError(f"bindings {min(x, y)} and {max(x, y)} alias the same allocation and at least one "
                                   f"of them writes the shared bytes")


# ------------------------------------------------------------------------------------------- NVRTC
def _nvrtc():
    import site
    cands = []
    for sp in site.getsitepackages():
        cands += glob.glob(sp + "/nvidia/cuda_nvrtc/lib/libnvrtc.so*")
    cands += glob.glob("/usr/local/cuda/lib64/libnvrtc.so*")
    cands = sorted(c for c in cands if "builtins" not in c)
    if not cands:
        raise RawError("libnvrtc not found")
    return C.CDLL(cands[0])


def compile_cuda_c(source: str, arch: str = DEFAULT_ARCH, extra_options=(), strict_ieee: bool = True) -> bytes:
    """CUDA C -> PTX with NVRTC. ``strict_ieee`` pins the four floating-point options; callers cannot switch on
    fast-math through ``extra_options`` (rejected), which would break bit-reproducibility."""
    for o in extra_options:
        if "fast-math" in o or "fast_math" in o or o.startswith(("--ftz", "--prec-", "--fmad", "-ftz", "-prec-", "-fmad")):
            raise RawError(f"option {o!r} would override the pinned floating-point behaviour")
    opts = [f"--gpu-architecture={arch}", *(STRICT_IEEE_OPTIONS if strict_ieee else ()), *extra_options]
    lib = _nvrtc()
    prog = C.c_void_p()
    if lib.nvrtcCreateProgram(C.byref(prog), source.encode(), b"raw_kernel.cu", 0, None, None) != 0:
        raise RawError("nvrtcCreateProgram failed")
    arr = (C.c_char_p * len(opts))(*[o.encode() for o in opts])
    rc = lib.nvrtcCompileProgram(prog, len(opts), arr)
    if rc != 0:
        n = C.c_size_t()
        lib.nvrtcGetProgramLogSize(prog, C.byref(n))
        log = C.create_string_buffer(n.value)
        lib.nvrtcGetProgramLog(prog, log)
        lib.nvrtcDestroyProgram(C.byref(prog))
        raise RawError("NVRTC compilation failed:\n" + log.value.decode(errors="replace"))
    n = C.c_size_t()
    lib.nvrtcGetPTXSize(prog, C.byref(n))
    ptx = C.create_string_buffer(n.value)
    lib.nvrtcGetPTX(prog, ptx)
    lib.nvrtcDestroyProgram(C.byref(prog))
    return ptx.raw


class RawKernel:
    def __init__(self, name: str, ptx: bytes, function=None, module=None):
        self.name, self.ptx, self.function, self.module = name, ptx, function, module


class RawRuntime:
    """One CUDA device, its primary context and one ordered stream (torch's current stream of that device)."""

    def __init__(self, device_index: int = 0):
        import torch
        if not torch.cuda.is_available():
            raise RawError("no CUDA device")
        self.torch = torch
        self.device = torch.device("cuda", device_index)
        torch.zeros(1, device=self.device)                   # primary context current on this thread
        p = torch.cuda.get_device_properties(device_index)
        self.limits = {"max_grid": (2**31 - 1, 65535, 65535), "max_block": (1024, 1024, 64),
                       "max_threads": p.max_threads_per_multi_processor and 1024,
                       "max_smem": getattr(p, "shared_memory_per_block_optin", 227 * 1024)}
        self.arch = f"compute_{p.major}{p.minor}a" if (p.major, p.minor) >= (9, 0) else f"compute_{p.major}{p.minor}"
        self.cu = C.CDLL("libcuda.so.1")
        self.cu.cuLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 6 + [C.c_uint, C.c_void_p, C.c_void_p, C.c_void_p]

    # -- memory
    def allocate(self, nbytes: int) -> RawBuffer:
        if nbytes <= 0:
            raise RawError("allocation size must be positive")
        return RawBuffer(nbytes, self.torch.zeros(nbytes, dtype=self.torch.uint8, device=self.device))

    def write(self, buf: RawBuffer, data: bytes, offset: int = 0) -> None:
        if offset < 0 or offset + len(data) > buf.logical_bytes:
            raise RawError("write exceeds buffer bounds")
        src = self.torch.frombuffer(bytearray(data), dtype=self.torch.uint8)
        buf.tensor[offset:offset + len(data)].copy_(src)

    def read(self, buf: RawBuffer, offset: int = 0, nbytes: int | None = None) -> bytes:
        n = buf.logical_bytes - offset if nbytes is None else nbytes
        if offset < 0 or n < 0 or offset + n > buf.logical_bytes:
            raise RawError("read exceeds buffer bounds")
        return bytes(buf.tensor[offset:offset + n].cpu().numpy().tobytes())

    # -- kernels
    def compile(self, source: str, entry: str, extra_options=()) -> RawKernel:
        ptx = compile_cuda_c(source, self.arch, extra_options)
        mod, fn = C.c_void_p(), C.c_void_p()
        if self.cu.cuModuleLoadData(C.byref(mod), ptx) != 0:
            raise RawError("cuModuleLoadData failed")
        if self.cu.cuModuleGetFunction(C.byref(fn), mod, entry.encode()) != 0:
            raise RawError(f"entry point {entry!r} not found in the module")
        return RawKernel(entry, ptx, fn, mod)

    def launch(self, kernel: RawKernel, cfg: RawLaunchConfig, bindings, scalars=()):
        """Kernel parameters = one pointer per binding (base + offset), in binding order, then ``scalars`` (ctypes
        values). Returns a CUDA event recorded behind the launch."""
        validate_launch_geometry(cfg, self.limits)
        validate_bindings(bindings)
        validate_alias_groups(bindings)
        vals = [C.c_void_p(b.buffer.ptr + b.offset_bytes) for b in bindings] + list(scalars)
        ptrs = (C.c_void_p * len(vals))(*[C.addressof(v) for v in vals])
        if cfg.shared_memory_bytes > 48 * 1024:
            # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8
            if self.cu.cuFuncSetAttribute(kernel.function, 8, cfg.shared_memory_bytes) != 0:
                raise RawError("could not raise the kernel's dynamic shared-memory limit")
        stream = self.torch.cuda.current_stream(self.device)
        rc = self.cu.cuLaunchKernel(kernel.function, *cfg.grid, *cfg.block, cfg.shared_memory_bytes,
                                    stream.cuda_stream, ptrs, None)
        if rc != 0:
            raise RawError(f"cuLaunchKernel({kernel.name}) failed with code {rc}")
        ev = self.torch.cuda.Event()
        ev.record(stream)
        return ev

    def synchronize(self) -> None:
        self.torch.cuda.synchronize(self.device)

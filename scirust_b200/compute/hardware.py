"""What a device can do, stated as three-valued facts (supported / unsupported / UNKNOWN): architecture, instruction-set
features, numeric formats for storage / arithmetic / accumulation, matrix acceleration, memory spaces, execution features
and reproducibility modes. Unknown is never rounded to yes: a planner may only use an unknown fact when its policy allows
indeterminate matches.

Blackwell features are first-class: ``TCGEN05`` (5th-gen tensor cores), ``TMEM`` (tensor memory), ``TMA`` (bulk tensor
copies), ``CLUSTERS`` / ``CTA_PAIR``, ``FP8_MMA`` / ``FP4_MMA`` / ``INT8_MMA``, ``NVLINK_P2P`` and ``MULTIMEM``.
``probe_cuda`` reads them off a live device (compute capability 10.x => the Blackwell set); ``b200_declared`` is the same
profile stated without a device, for planning on a machine that has none; ``probe_host_cpu`` reads the host's flags.
``canonical_hardware_profile_bytes`` is a stable byte encoding used as a cache key by the autotuner.
Reference counterpart: scirust-compute/src/{hardware,capabilities,hwprobe,profile_encoding}.rs.
"""
from __future__ import annotations

import enum
import platform
from dataclasses import dataclass, field

from .contracts import DeviceId, DeviceKind, DType, MemorySpace


class SupportLevel(enum.Enum):
    UNKNOWN = 0
    UNSUPPORTED = 1
    SUPPORTED = 2

    def is_supported(self) -> bool:
        return self is SupportLevel.SUPPORTED

    @staticmethod
    def from_known(value: bool) -> "SupportLevel":
        return SupportLevel.SUPPORTED if value else SupportLevel.UNSUPPORTED


class CapabilitySet:
    def __init__(self, supported=(), unsupported=()):
        self._s, self._u = list(supported), list(unsupported)

    def support_level(self, value) -> SupportLevel:
        if value in self._s:
            return SupportLevel.SUPPORTED
        if value in self._u:
            return SupportLevel.UNSUPPORTED
        return SupportLevel.UNKNOWN

    def supports(self, value) -> bool:
        return value in self._s

    def is_empty(self) -> bool:
        return not self._s and not self._u

    def supported_values(self):
        return list(self._s)

    def unsupported_values(self):
        return list(self._u)

    def set_support(self, value, level: SupportLevel) -> None:
        self._s = [v for v in self._s if v != value]
        self._u = [v for v in self._u if v != value]
        if level is SupportLevel.SUPPORTED:
            self._s.append(value)
        elif level is SupportLevel.UNSUPPORTED:
            self._u.append(value)

    def __eq__(self, other):
        return isinstance(other, CapabilitySet) and sorted(map(repr, self._s)) == sorted(map(repr, other._s)) \
            and sorted(map(repr, self._u)) == sorted(map(repr, other._u))


class ArchitectureFamily(enum.Enum):
    X86_64 = "x86_64"
    AARCH64 = "aarch64"
    NVIDIA_GPU = "nvidia-gpu"
    OTHER = "other"
    UNKNOWN = "unknown"


@dataclass(frozen=True)
class Architecture:
    family: ArchitectureFamily = ArchitectureFamily.UNKNOWN
    name: str | None = None

    @staticmethod
    def current_host() -> "Architecture":
        m = platform.machine().lower()
        fam = {"x86_64": ArchitectureFamily.X86_64, "amd64": ArchitectureFamily.X86_64, "aarch64": ArchitectureFamily.AARCH64,
               "arm64": ArchitectureFamily.AARCH64}.get(m, ArchitectureFamily.UNKNOWN)
        return Architecture(fam)


class IsaFeature(enum.Enum):
    # host
    SSE2 = "sse2"
    AVX2 = "avx2"
    FMA = "fma"
    AVX512F = "avx512f"
    AVX512_VNNI = "avx512_vnni"
    AVX512_BF16 = "avx512_bf16"
    AMX_TILE = "amx_tile"
    AMX_INT8 = "amx_int8"
    AMX_BF16 = "amx_bf16"
    NEON = "neon"
    SVE = "sve"
    # NVIDIA
    MMA_SYNC = "mma_sync"
    WGMMA = "wgmma"
    TCGEN05 = "tcgen05"
    TMEM = "tmem"
    TMA = "tma"
    CLUSTERS = "clusters"
    CTA_PAIR = "cta_pair"
    FP8_MMA = "fp8_mma"
    FP4_MMA = "fp4_mma"
    INT8_MMA = "int8_mma"
    NVLINK_P2P = "nvlink_p2p"
    MULTIMEM = "multimem"


class VectorModel(enum.Enum):
    SCALAR = "scalar"
    FIXED_WIDTH = "fixed"
    SCALABLE = "scalable"
    SIMT = "simt"
    UNKNOWN = "unknown"


class ReproducibilityLevel(enum.Enum):
    BIT_EXACT = "bit-exact"
    DETERMINISTIC = "deterministic"
    NUMERICALLY_EQUIVALENT = "numerically-equivalent"
    FAST_APPROXIMATE = "fast-approximate"


@dataclass
class IsaCapabilities:
    features: CapabilitySet = field(default_factory=CapabilitySet)
    vector_model: VectorModel = VectorModel.UNKNOWN
    min_vector_bits: int | None = None
    max_vector_bits: int | None = None

    def supports(self, f) -> bool:
        return self.features.supports(f)


@dataclass
class NumericCapabilities:
    storage_dtypes: CapabilitySet = field(default_factory=CapabilitySet)
    arithmetic_dtypes: CapabilitySet = field(default_factory=CapabilitySet)
    accumulation_dtypes: CapabilitySet = field(default_factory=CapabilitySet)


@dataclass
class MatrixCapabilities:
    accelerated: SupportLevel = SupportLevel.UNKNOWN
    input_dtypes: CapabilitySet = field(default_factory=CapabilitySet)
    accumulation_dtypes: CapabilitySet = field(default_factory=CapabilitySet)


@dataclass
class MemoryCapabilities:
    spaces: CapabilitySet = field(default_factory=CapabilitySet)
    coherent_host_device: SupportLevel = SupportLevel.UNKNOWN
    unified_addressing: SupportLevel = SupportLevel.UNKNOWN
    async_transfers: SupportLevel = SupportLevel.UNKNOWN
    capacity_bytes: int | None = None
    shared_memory_per_block: int | None = None
    tensor_memory_per_sm: int | None = None
    l2_bytes: int | None = None


@dataclass
class ExecutionCapabilities:
    async_execution: SupportLevel = SupportLevel.UNKNOWN
    ordered_streams: SupportLevel = SupportLevel.UNKNOWN
    subgroup_operations: SupportLevel = SupportLevel.UNKNOWN
    atomic_i64: SupportLevel = SupportLevel.UNKNOWN
    graph_capture: SupportLevel = SupportLevel.UNKNOWN
    multiprocessors: int | None = None


@dataclass
class ReproducibilityCapabilities:
    modes: CapabilitySet = field(default_factory=CapabilitySet)

    def support_level(self, level) -> SupportLevel:
        return self.modes.support_level(level)


@dataclass
class DeviceCapabilities:
    device: DeviceId
    name: str
    supported_dtypes: list
    max_buffer_bytes: int | None
    max_workgroup_size: tuple
    supports_async_execution: bool

    @staticmethod
    def reference_cpu() -> "DeviceCapabilities":
        return DeviceCapabilities(DeviceId.reference(), "reference-cpu", [DType.F32], None, (1, 1, 1), False)

    def supports_dtype(self, d: DType) -> bool:
        return d in self.supported_dtypes

    def hardware_baseline(self) -> "HardwareCapabilities":
        return HardwareCapabilities.from_device_capabilities(self)


@dataclass
class HardwareCapabilities:
    device: DeviceId
    architecture: Architecture = field(default_factory=Architecture)
    isa: IsaCapabilities = field(default_factory=IsaCapabilities)
    numeric: NumericCapabilities = field(default_factory=NumericCapabilities)
    matrix: MatrixCapabilities = field(default_factory=MatrixCapabilities)
    memory: MemoryCapabilities = field(default_factory=MemoryCapabilities)
    execution: ExecutionCapabilities = field(default_factory=ExecutionCapabilities)
    reproducibility: ReproducibilityCapabilities = field(default_factory=ReproducibilityCapabilities)

    @staticmethod
    def from_device_capabilities(c: DeviceCapabilities) -> "HardwareCapabilities":
        """Only what the legacy description states; nothing optional is invented."""
        arch = Architecture.current_host() if c.device.kind in (DeviceKind.REFERENCE, DeviceKind.CPU) else Architecture()
        storage = CapabilitySet()
        for d in DType:
            storage.set_support(d, SupportLevel.from_known(c.supports_dtype(d)))
        hw = HardwareCapabilities(c.device, arch)
        hw.numeric.storage_dtypes = storage
        hw.execution.async_execution = SupportLevel.from_known(c.supports_async_execution)
        host = c.device.kind in (DeviceKind.REFERENCE, DeviceKind.CPU)
        hw.memory.spaces.set_support(MemorySpace.HOST if host else MemorySpace.DEVICE, SupportLevel.SUPPORTED)
        return hw


@dataclass(frozen=True)
class ExecutionLimits:
    max_workgroup_size: tuple = (None, None, None)
    max_threads_per_block: int | None = None
    max_shared_memory_bytes: int | None = None
    max_cluster_size: int | None = None

    @staticmethod
    def from_device_capabilities(c: DeviceCapabilities) -> "ExecutionLimits":
        return ExecutionLimits(tuple(c.max_workgroup_size))


_BLACKWELL = (IsaFeature.MMA_SYNC, IsaFeature.TCGEN05, IsaFeature.TMEM, IsaFeature.TMA, IsaFeature.CLUSTERS, IsaFeature.CTA_PAIR,
              IsaFeature.FP8_MMA, IsaFeature.FP4_MMA, IsaFeature.INT8_MMA)
_GPU_STORAGE = (DType.BOOL, DType.U8, DType.I8, DType.I16, DType.F16, DType.BF16, DType.I32, DType.F32, DType.I64, DType.F64,
                DType.F8E4M3, DType.F8E5M2)


def _nvidia_profile(device: DeviceId, name: str, cc: tuple, sms, mem, smem, l2, peers: SupportLevel) -> HardwareCapabilities:
    hw = HardwareCapabilities(device, Architecture(ArchitectureFamily.NVIDIA_GPU, f"sm_{cc[0]}{cc[1]}"))
    f = hw.isa.features
    blackwell_dc = cc[0] == 10
    for feat in _BLACKWELL:
        f.set_support(feat, SupportLevel.from_known(blackwell_dc or (feat is IsaFeature.MMA_SYNC and cc >= (7, 0))
                                                    or (feat in (IsaFeature.TMA, IsaFeature.CLUSTERS, IsaFeature.FP8_MMA) and cc >= (9, 0))))
    f.set_support(IsaFeature.WGMMA, SupportLevel.from_known(cc == (9, 0)))
    f.set_support(IsaFeature.NVLINK_P2P, peers)
    f.set_support(IsaFeature.MULTIMEM, peers if cc >= (9, 0) else SupportLevel.UNSUPPORTED)
    hw.isa.vector_model, hw.isa.min_vector_bits, hw.isa.max_vector_bits = VectorModel.SIMT, 32 * 32, 32 * 128
    for d in _GPU_STORAGE:
        hw.numeric.storage_dtypes.set_support(d, SupportLevel.SUPPORTED)
    for d in (DType.F16, DType.BF16, DType.F32, DType.F64, DType.I32, DType.I64):
        hw.numeric.arithmetic_dtypes.set_support(d, SupportLevel.SUPPORTED)
    for d in (DType.F32, DType.F64, DType.I32):
        hw.numeric.accumulation_dtypes.set_support(d, SupportLevel.SUPPORTED)
    hw.matrix.accelerated = SupportLevel.from_known(cc >= (7, 0))
    for d in (DType.F16, DType.BF16, DType.I8) + ((DType.F8E4M3, DType.F8E5M2) if cc >= (8, 9) else ()):
        hw.matrix.input_dtypes.set_support(d, SupportLevel.SUPPORTED)
    for d in (DType.F32, DType.I32):
        hw.matrix.accumulation_dtypes.set_support(d, SupportLevel.SUPPORTED)
    m = hw.memory
    for s in (MemorySpace.DEVICE, MemorySpace.HOST_PINNED, MemorySpace.UNIFIED):
        m.spaces.set_support(s, SupportLevel.SUPPORTED)
    m.spaces.set_support(MemorySpace.PEER_DEVICE, peers)
    m.coherent_host_device, m.unified_addressing, m.async_transfers = SupportLevel.UNSUPPORTED, SupportLevel.SUPPORTED, SupportLevel.SUPPORTED
    m.capacity_bytes, m.shared_memory_per_block, m.l2_bytes = mem, smem, l2
    m.tensor_memory_per_sm = 256 * 1024 if blackwell_dc else None
    e = hw.execution
    e.async_execution = e.ordered_streams = e.subgroup_operations = e.atomic_i64 = e.graph_capture = SupportLevel.SUPPORTED
    e.multiprocessors = sms
    for lvl in ReproducibilityLevel:
        hw.reproducibility.modes.set_support(lvl, SupportLevel.SUPPORTED)
    return hw


def b200_declared(ordinal: int = 0, peers: bool = True) -> HardwareCapabilities:
    """The B200 profile as declared facts (148 SMs, 180 GB HBM3e, 227 KB shared memory per CTA, 126 MB L2)."""
    return _nvidia_profile(DeviceId.cuda(ordinal), "NVIDIA B200", (10, 0), 148, 180 * 10 ** 9, 227 * 1024, 126 * 2 ** 20,
                           SupportLevel.from_known(peers))


def b200_limits() -> ExecutionLimits:
    return ExecutionLimits((1024, 1024, 64), 1024, 227 * 1024, 16)


def probe_cuda(ordinal: int = 0) -> HardwareCapabilities:
    import torch
    if not torch.cuda.is_available() or ordinal >= torch.cuda.device_count():
        raise RuntimeError("probe_cuda: no such CUDA device")
    p = torch.cuda.get_device_properties(ordinal)
    n = torch.cuda.device_count()
    peers = SupportLevel.UNSUPPORTED
    if n > 1:
        peers = SupportLevel.from_known(all(torch.cuda.can_device_access_peer(ordinal, j) for j in range(n) if j != ordinal))
    return _nvidia_profile(DeviceId.cuda(ordinal), p.name, (p.major, p.minor), p.multi_processor_count, p.total_memory,
                           getattr(p, "shared_memory_per_block_optin", None), getattr(p, "L2_cache_size", None), peers)


def cuda_limits(ordinal: int = 0) -> ExecutionLimits:
    import torch
    p = torch.cuda.get_device_properties(ordinal)
    return ExecutionLimits((1024, 1024, 64), 1024, getattr(p, "shared_memory_per_block_optin", None), 16 if p.major >= 9 else 1)


def probe_host_cpu() -> HardwareCapabilities:
    hw = HardwareCapabilities(DeviceId.cpu(), Architecture.current_host())
    flags = set()
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith(("flags", "Features")):
                    flags = set(line.split(":", 1)[1].split())
                    break
    except OSError:
        pass
    table = {"sse2": IsaFeature.SSE2, "avx2": IsaFeature.AVX2, "fma": IsaFeature.FMA, "avx512f": IsaFeature.AVX512F,
             "avx512_vnni": IsaFeature.AVX512_VNNI, "avx512_bf16": IsaFeature.AVX512_BF16, "amx_tile": IsaFeature.AMX_TILE,
             "amx_int8": IsaFeature.AMX_INT8, "amx_bf16": IsaFeature.AMX_BF16, "asimd": IsaFeature.NEON, "sve": IsaFeature.SVE}
    if flags:                                                        # a readable flag list makes absences KNOWN
        for name, feat in table.items():
            hw.isa.features.set_support(feat, SupportLevel.from_known(name in flags))
        wide = 512 if "avx512f" in flags else 256 if "avx2" in flags else 128
        hw.isa.vector_model, hw.isa.min_vector_bits, hw.isa.max_vector_bits = VectorModel.FIXED_WIDTH, 128, wide
    for d in (DType.F32, DType.F64, DType.I32, DType.I64, DType.I8, DType.U8, DType.BF16, DType.F16):
        hw.numeric.storage_dtypes.set_support(d, SupportLevel.SUPPORTED)
    for d in (DType.F32, DType.F64, DType.I32, DType.I64):
        hw.numeric.arithmetic_dtypes.set_support(d, SupportLevel.SUPPORTED)
        hw.numeric.accumulation_dtypes.set_support(d, SupportLevel.SUPPORTED)
    hw.matrix.accelerated = SupportLevel.from_known("amx_tile" in flags) if flags else SupportLevel.UNKNOWN
    hw.memory.spaces.set_support(MemorySpace.HOST, SupportLevel.SUPPORTED)
    hw.memory.spaces.set_support(MemorySpace.DEVICE, SupportLevel.UNSUPPORTED)
    hw.execution.async_execution, hw.execution.atomic_i64 = SupportLevel.UNSUPPORTED, SupportLevel.SUPPORTED
    hw.reproducibility.modes.set_support(ReproducibilityLevel.BIT_EXACT, SupportLevel.SUPPORTED)
    hw.reproducibility.modes.set_support(ReproducibilityLevel.DETERMINISTIC, SupportLevel.SUPPORTED)
    return hw


def _enc_set(cs: CapabilitySet, key) -> bytes:
    s = sorted(key(v) for v in cs.supported_values())
    u = sorted(key(v) for v in cs.unsupported_values())
    return ("+" + ",".join(s) + "-" + ",".join(u)).encode()


def canonical_hardware_profile_bytes(hw: HardwareCapabilities) -> bytes:
    """Order-independent, versioned encoding of a profile: equal facts give equal bytes whatever order they were set in."""
    lab = lambda d: d.label if isinstance(d, DType) else d.value
    num = lambda v: b"?" if v is None else str(v).encode()
    parts = [b"scirust-b200-hw-v1", hw.device.record().encode(), hw.architecture.family.value.encode(),
             (hw.architecture.name or "").encode(), _enc_set(hw.isa.features, lab), hw.isa.vector_model.value.encode(),
             num(hw.isa.min_vector_bits), num(hw.isa.max_vector_bits), _enc_set(hw.numeric.storage_dtypes, lab),
             _enc_set(hw.numeric.arithmetic_dtypes, lab), _enc_set(hw.numeric.accumulation_dtypes, lab),
             str(hw.matrix.accelerated.value).encode(), _enc_set(hw.matrix.input_dtypes, lab),
             _enc_set(hw.matrix.accumulation_dtypes, lab), _enc_set(hw.memory.spaces, lab),
             bytes([hw.memory.coherent_host_device.value, hw.memory.unified_addressing.value, hw.memory.async_transfers.value]),
             num(hw.memory.capacity_bytes), num(hw.memory.shared_memory_per_block), num(hw.memory.tensor_memory_per_sm),
             num(hw.memory.l2_bytes),
             bytes([hw.execution.async_execution.value, hw.execution.ordered_streams.value, hw.execution.subgroup_operations.value,
                    hw.execution.atomic_i64.value, hw.execution.graph_capture.value]), num(hw.execution.multiprocessors),
             _enc_set(hw.reproducibility.modes, lab)]
    return b"|".join(parts)

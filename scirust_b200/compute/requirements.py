"""Matching what a kernel NEEDS against what a device HAS, and choosing among implementations.

``KernelRequirements`` lists dtypes (storage / arithmetic / accumulation), instruction-set features, the vector model,
matrix acceleration, memory spaces, execution features and a reproducibility level. ``match_requirements`` returns
``compatible`` (every fact known and satisfied), ``incompatible`` (some fact known and violated) or ``indeterminate``
(nothing violated, something unknown), with one issue per unmet or unknown item. ``ImplementationRequirements`` adds
launch-shape needs (minimum block size per axis, shared memory, cluster size) checked against ``ExecutionLimits``.
``select_implementation`` keeps the eligible candidates (indeterminate ones only if the policy allows), prefers
compatible over indeterminate, then the LOWER priority number, then the name.

``GEMM_CANDIDATES`` states the requirements of this framework's own GEMM paths (CTA-pair tcgen05, single-CTA tcgen05,
library fallback), so the same machinery answers "which GEMM runs here" for a B200, an older GPU or a CPU.
Reference counterpart: scirust-compute/src/{requirements,implementation}.rs.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from .contracts import DType, MemorySpace
from .hardware import (ExecutionLimits, HardwareCapabilities, IsaFeature, ReproducibilityLevel, SupportLevel, VectorModel)


class SupportRequirement(enum.Enum):
    ANY = "any"
    REQUIRED = "required"
    FORBIDDEN = "forbidden"


@dataclass(frozen=True)
class VectorRequirement:
    kind: str = "any"                 # any | scalar | vectorized | fixed | scalable | simt
    min_bits: int | None = None


@dataclass
class KernelRequirements:
    storage_dtypes: list = field(default_factory=list)
    arithmetic_dtypes: list = field(default_factory=list)
    accumulation_dtypes: list = field(default_factory=list)
    required_isa: list = field(default_factory=list)
    vector: VectorRequirement = VectorRequirement()
    matrix_acceleration: SupportRequirement = SupportRequirement.ANY
    memory_spaces: list = field(default_factory=list)
    async_execution: SupportRequirement = SupportRequirement.ANY
    subgroup_operations: SupportRequirement = SupportRequirement.ANY
    atomic_i64: SupportRequirement = SupportRequirement.ANY
    reproducibility: ReproducibilityLevel | None = None


class MatchDisposition(enum.Enum):
    COMPATIBLE = 0
    INDETERMINATE = 1
    INCOMPATIBLE = 2


@dataclass(frozen=True)
class RequirementIssue:
    kind: str                 # e.g. storage-dtype-unknown, isa-unsupported, vector-width-insufficient ...
    detail: object = None


@dataclass
class MatchReport:
    disposition: MatchDisposition
    issues: list

    def is_compatible(self) -> bool:
        return self.disposition is MatchDisposition.COMPATIBLE

    def is_incompatible(self) -> bool:
        return self.disposition is MatchDisposition.INCOMPATIBLE


class _State:
    def __init__(self):
        self.issues, self.unknown, self.bad = [], False, False

    def add(self, level: SupportLevel, name: str, detail):
        if level is SupportLevel.UNKNOWN:
            self.unknown = True
            self.issues.append(RequirementIssue(f"{name}-unknown", detail))
        elif level is SupportLevel.UNSUPPORTED:
            self.bad = True
            self.issues.append(RequirementIssue(f"{name}-unsupported", detail))

    def support(self, req: SupportRequirement, observed: SupportLevel, name: str):
        if req is SupportRequirement.ANY:
            return
        if observed is SupportLevel.UNKNOWN:
            self.unknown = True
            self.issues.append(RequirementIssue(f"{name}-unknown"))
        elif (observed is SupportLevel.SUPPORTED) == (req is SupportRequirement.FORBIDDEN):
            self.bad = True
            self.issues.append(RequirementIssue(f"{name}-mismatch", (req, observed)))

    def finish(self) -> MatchReport:
        d = MatchDisposition.INCOMPATIBLE if self.bad else MatchDisposition.INDETERMINATE if self.unknown else MatchDisposition.COMPATIBLE
        return MatchReport(d, self.issues)


def match_requirements(req: KernelRequirements, hw: HardwareCapabilities) -> MatchReport:
    st = _State()
    for values, have, name in ((req.storage_dtypes, hw.numeric.storage_dtypes, "storage-dtype"),
                               (req.arithmetic_dtypes, hw.numeric.arithmetic_dtypes, "arithmetic-dtype"),
                               (req.accumulation_dtypes, hw.numeric.accumulation_dtypes, "accumulation-dtype"),
                               (req.required_isa, hw.isa.features, "isa"),
                               (req.memory_spaces, hw.memory.spaces, "memory-space")):
        for v in values:
            st.add(have.support_level(v), name, v)
    v = req.vector
    if v.kind != "any":
        obs = hw.isa.vector_model
        if obs is VectorModel.UNKNOWN:
            st.unknown = True
            st.issues.append(RequirementIssue("vector-model-unknown"))
        else:
            ok = {"scalar": obs is VectorModel.SCALAR, "fixed": obs is VectorModel.FIXED_WIDTH, "scalable": obs is VectorModel.SCALABLE,
                  "simt": obs is VectorModel.SIMT,
                  "vectorized": obs in (VectorModel.FIXED_WIDTH, VectorModel.SCALABLE, VectorModel.SIMT)}[v.kind]
            if not ok:
                st.bad = True
                st.issues.append(RequirementIssue("vector-model-incompatible", (v, obs)))
            elif v.min_bits is not None:
                if hw.isa.max_vector_bits is None:
                    st.unknown = True
                    st.issues.append(RequirementIssue("vector-width-unknown", v.min_bits))
                elif hw.isa.max_vector_bits < v.min_bits:
                    st.bad = True
                    st.issues.append(RequirementIssue("vector-width-insufficient", (v.min_bits, hw.isa.max_vector_bits)))
    st.support(req.matrix_acceleration, hw.matrix.accelerated, "matrix-acceleration")
    st.support(req.async_execution, hw.execution.async_execution, "async-execution")
    st.support(req.subgroup_operations, hw.execution.subgroup_operations, "subgroup-operations")
    st.support(req.atomic_i64, hw.execution.atomic_i64, "atomic-i64")
    if req.reproducibility is not None:
        st.add(hw.reproducibility.support_level(req.reproducibility), "reproducibility", req.reproducibility)
    return st.finish()


@dataclass(frozen=True)
class PlannerPolicy:
    allow_indeterminate: bool = False


@dataclass
class ExecutionCandidate:
    name: str
    priority: int
    capabilities: HardwareCapabilities


@dataclass
class Selection:
    name: str
    priority: int
    report: object


def _better(a: Selection, b: Selection) -> bool:
    ka = (a.report.disposition.value, a.priority, a.name)
    return ka < (b.report.disposition.value, b.priority, b.name)


def _eligible(d: MatchDisposition, policy: PlannerPolicy) -> bool:
    return d is MatchDisposition.COMPATIBLE or (d is MatchDisposition.INDETERMINATE and policy.allow_indeterminate)


def select_candidate(req: KernelRequirements, candidates, policy: PlannerPolicy = PlannerPolicy()):
    """Which DEVICE profile should run a kernel."""
    best = None
    for c in candidates:
        rep = match_requirements(req, c.capabilities)
        if _eligible(rep.disposition, policy):
            s = Selection(c.name, c.priority, rep)
            if best is None or _better(s, best):
                best = s
    return best


@dataclass(frozen=True)
class WorkgroupRequirement:
    min_size: tuple = (None, None, None)
    shared_memory_bytes: int = 0
    cluster_size: int = 1

    @staticmethod
    def x(minimum: int, shared_memory_bytes: int = 0, cluster_size: int = 1) -> "WorkgroupRequirement":
        return WorkgroupRequirement((minimum, None, None), shared_memory_bytes, cluster_size)


@dataclass
class ImplementationRequirements:
    kernel: KernelRequirements
    workgroup: WorkgroupRequirement = WorkgroupRequirement()

    def with_workgroup(self, w: WorkgroupRequirement) -> "ImplementationRequirements":
        return ImplementationRequirements(self.kernel, w)


@dataclass
class ImplementationCandidate:
    name: str
    priority: int
    requirements: ImplementationRequirements


@dataclass
class ImplementationMatchReport:
    disposition: MatchDisposition
    kernel: MatchReport
    issues: list


def match_implementation(req: ImplementationRequirements, hw: HardwareCapabilities, limits: ExecutionLimits) -> ImplementationMatchReport:
    kernel = match_requirements(req.kernel, hw)
    issues, unknown, bad = [], False, False

    def check(need, have, name):
        nonlocal unknown, bad
        if not need:
            return
        if have is None:
            unknown = True
            issues.append(RequirementIssue(f"{name}-limit-unknown", need))
        elif have < need:
            bad = True
            issues.append(RequirementIssue(f"{name}-limit-insufficient", (need, have)))

    for ax, need in zip("xyz", req.workgroup.min_size):
        check(need, limits.max_workgroup_size["xyz".index(ax)], f"workgroup-{ax}")
    check(req.workgroup.shared_memory_bytes, limits.max_shared_memory_bytes, "shared-memory")
    check(req.workgroup.cluster_size if req.workgroup.cluster_size > 1 else 0, limits.max_cluster_size, "cluster-size")
    if kernel.disposition is MatchDisposition.INCOMPATIBLE or bad:
        d = MatchDisposition.INCOMPATIBLE
    elif kernel.disposition is MatchDisposition.INDETERMINATE or unknown:
        d = MatchDisposition.INDETERMINATE
    else:
        d = MatchDisposition.COMPATIBLE
    return ImplementationMatchReport(d, kernel, issues)


def select_implementation(hw: HardwareCapabilities, limits: ExecutionLimits, candidates, policy: PlannerPolicy = PlannerPolicy()):
    """Which KERNEL implementation should run on a device."""
    best = None
    for c in candidates:
        rep = match_implementation(c.requirements, hw, limits)
        if _eligible(rep.disposition, policy):
            s = Selection(c.name, c.priority, rep)
            if best is None or _better(s, best):
                best = s
    return best


def _gemm(isa, smem, cluster, block) -> ImplementationRequirements:
    k = KernelRequirements(storage_dtypes=[DType.BF16], accumulation_dtypes=[DType.F32], required_isa=list(isa),
                           matrix_acceleration=SupportRequirement.REQUIRED, memory_spaces=[MemorySpace.DEVICE],
                           reproducibility=ReproducibilityLevel.DETERMINISTIC)
    return ImplementationRequirements(k, WorkgroupRequirement.x(block, smem, cluster))


GEMM_CANDIDATES = [
    ImplementationCandidate("tcgen05-cta-pair", 0, _gemm((IsaFeature.TCGEN05, IsaFeature.TMEM, IsaFeature.TMA, IsaFeature.CTA_PAIR),
                                                         200 * 1024, 2, 320)),
    ImplementationCandidate("tcgen05-single-cta", 1, _gemm((IsaFeature.TCGEN05, IsaFeature.TMEM, IsaFeature.TMA), 180 * 1024, 1, 192)),
    ImplementationCandidate("library-gemm", 9, ImplementationRequirements(
        KernelRequirements(storage_dtypes=[DType.BF16], memory_spaces=[MemorySpace.DEVICE]))),
    ImplementationCandidate("host-fp32-fixed-order", 20, ImplementationRequirements(
        KernelRequirements(storage_dtypes=[DType.F32], memory_spaces=[MemorySpace.HOST],
                           reproducibility=ReproducibilityLevel.BIT_EXACT))),
]

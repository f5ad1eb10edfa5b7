"""Backend-neutral compute contracts, hardware / topology description, requirement matching and evidence-based kernel
selection (``contracts``, ``hardware``, ``requirements``, ``topology``, ``transfer``, ``backend``, ``autotune``)."""
from .contracts import (BufferAccess, BufferBinding, ComputeError, DeviceId, DeviceKind, DType, KernelFormat, KernelModule,  # noqa: F401
                        LaunchConfig, Layout, MemorySpace, Shape, Strides, TensorSpec)
from .hardware import (DeviceCapabilities, ExecutionLimits, HardwareCapabilities, IsaFeature, SupportLevel, b200_declared,  # noqa: F401
                       canonical_hardware_profile_bytes, probe_host_cpu)
from .requirements import (GEMM_CANDIDATES, KernelRequirements, PlannerPolicy, match_requirements, select_candidate,  # noqa: F401
                           select_implementation)
from .topology import SystemTopology, nvswitch_declared, probe_host_topology  # noqa: F401
from .backend import ComputeBackend, ReferenceBackend  # noqa: F401

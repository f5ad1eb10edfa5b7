"""Canonical tensor facade: a small typed IR, its planning pipeline and the sessions that execute it.

``Graph`` -> ``ExecutionPlan`` -> ``MemoryPlan`` -> ``LoweredPlan`` -> adapter (CPU statement or the CUDA canonical
kernels), plus ``grad`` / ``vmap`` graph transforms and the SPMD session over a ``DeviceMesh``.
"""
from .ir import Graph, GraphError, Value, grad, vmap  # noqa: F401
from .fusion import cuda_source, find_groups, lower_fused  # noqa: F401
from .plan import ExecutionPlan, LoweredPlan, MemoryPlan, lower, plan_execution, plan_memory  # noqa: F401
from .runtime import (ReferenceJitSession, ReferencePlanRuntime, ReferenceSpmdSession, conformance_cases,  # noqa: F401
                      run_conformance)

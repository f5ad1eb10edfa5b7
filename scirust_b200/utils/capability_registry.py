"""One queryable list of the compute paths that exist in this process and whether they are usable: for diagnostics,
logs and benchmark provenance (a read-side registry, not a dispatch layer). Availability is three-valued: True / False
after a real probe (loading the library, asking the driver), None when a path is present but has not been probed. The
host entry is seeded from the CPU probe; ``register_default_capabilities`` adds the native CPU runtime, the CUDA kernel
library and each visible GPU; ``capability_summary`` is the one-line form that `scirust info` prints.
Reference counterpart: scirust-core/src/compute_capability.rs.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass

DOMAINS = ("cpu-simd", "cpu-native", "cuda")


@dataclass(frozen=True)
class Capability:
    domain: str
    name: str
    detail: str = ""
    available: bool | None = None


_lock = threading.Lock()
_registry: list = []


def register_capability(cap: Capability) -> None:
    """Adds or replaces the entry with the same (domain, name)."""
    if cap.domain not in DOMAINS:
        raise ValueError(f"unknown compute domain {cap.domain!r}")
    with _lock:
        _registry[:] = [c for c in _registry if (c.domain, c.name) != (cap.domain, cap.name)]
        _registry.append(cap)


def capabilities(domain: str | None = None) -> list:
    with _lock:
        return [c for c in sorted(_registry, key=lambda c: (DOMAINS.index(c.domain), c.name)) if domain in (None, c.domain)]


def clear() -> None:
    with _lock:
        _registry.clear()


def register_default_capabilities(probe: bool = True) -> list:
    from ..compute.hardware import probe_host_cpu
    hw = probe_host_cpu()
    feats = [f.value for f in hw.isa.features.supported_values()]
    tier = next((f for f in ("avx512f", "avx2", "sse2", "neon", "sve") if f in feats), "scalar")
    register_capability(Capability("cpu-simd", tier, f"vector bits {hw.isa.max_vector_bits}; " + ",".join(sorted(feats)), True))
    from .. import _build
    rt_ok = cu_ok = None
    if probe:
        try:
            from ..ops import _lib
            _lib.rt()
            rt_ok = True
        except Exception:  # noqa: BLE001
            rt_ok = False
    register_capability(Capability("cpu-native", "rt", str(_build.RT_LIB.name), rt_ok))
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if probe:
        cu_ok = False
        if n:
            try:
                from ..ops import _lib
                _lib.cuda()
                cu_ok = True
            except Exception:  # noqa: BLE001
                cu_ok = False
    register_capability(Capability("cuda", "kernels", f"{_build.CUDA_LIB.name} (sm_100a: tcgen05 / TMEM / TMA)",
                                   cu_ok if n else (False if probe else None)))
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        register_capability(Capability("cuda", f"gpu{i}", f"{p.name} sm_{p.major}{p.minor} {p.multi_processor_count} SMs "
                                                           f"{p.total_memory >> 30} GiB", True))
    return capabilities()


def capability_summary() -> str:
    def mark(c):
        return {True: "+", False: "-", None: "?"}[c.available]
    return "; ".join(f"{c.domain}:{c.name}{mark(c)}" for c in capabilities()) or "none"

"""Every public module imports on a machine without a CUDA device and without touching the native CUDA library."""
import importlib
import pkgutil

import scirust_b200


def test_every_module_imports_without_a_device():
    skipped, failed = [], []
    for m in pkgutil.walk_packages(scirust_b200.__path__, "scirust_b200."):
        if ".csrc" in m.name or ".lib" in m.name:
            continue
        try:
            importlib.import_module(m.name)
        except Exception as e:  # noqa: BLE001
            failed.append((m.name, f"{type(e).__name__}: {e}"))
    assert not failed, failed
    names = {m.name for m in pkgutil.walk_packages(scirust_b200.__path__, "scirust_b200.")}
    for expected in ("dsp", "fixed", "geometry", "physics", "ode", "symbolic", "einsum", "interp", "stats", "learning", "causal",
                     "sequential", "estimation", "monitoring", "retrieval", "nlp", "vqnet", "quantum", "aot", "homomorphic"):
        assert f"scirust_b200.{expected}" in names, expected                  # the map in the package docstring is not stale
        assert expected in scirust_b200.__doc__

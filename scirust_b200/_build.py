"""In-tree native build: nvcc for the sm_100a CUDA library, g++ for the CPU runtime.

Outputs land in ``scirust_b200/lib/`` next to the sources so that a snapshot of the
repository carries the binaries with it:

* ``libscirust_b200_cuda.so``  - every ``csrc/*.cu`` (tcgen05 GEMM, attention, decode, comm ...)
* ``libscirust_b200_rt.so``    - every ``csrc/*.cpp`` (CPU runtime: fixed-order fp32 math,
  arena / paged-KV block allocators, TCP tree all-reduce, samplers); no CUDA dependency.

A source is recompiled when its object is older than it or than any header.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

CUDA_LIB = LIB / "libscirust_b200_cuda.so"
RT_LIB = LIB / "libscirust_b200_rt.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]
# Deterministic fp32 paths are compiled without contraction or fast division so the
# arithmetic is IEEE and reproducible (the reference's NVRTC build pins the same four
# options: scirust-cuda/src/raw_runtime.rs:308-323).
STRICT_FLAGS = ["-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(src: Path, headers: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in [src, *headers]:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _stale(src: Path, obj: Path, headers: list[Path], flags: list[str]) -> bool:
    """Content-addressed staleness (file times do not survive a copy of the tree): the object is
    current when the digest recorded beside it matches source + headers + flags."""
    tag = obj.with_suffix(obj.suffix + ".sha")
    if not obj.exists() or not tag.exists():
        return True
    return tag.read_text().strip() != _digest(src, headers, flags)


def _stamp(src: Path, obj: Path, headers: list[Path], flags: list[str]) -> None:
    obj.with_suffix(obj.suffix + ".sha").write_text(_digest(src, headers, flags))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    stamps = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        flags = list(NVCC_FLAGS)
        if src.stem.endswith("_strict"):
            flags += STRICT_FLAGS
        if force or _stale(src, obj, headers, flags):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append([nvcc, *flags, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
            stamps.append((src, obj, flags))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
        for src, obj, flags in stamps:
            _stamp(src, obj, headers, flags)
    if jobs or not CUDA_LIB.exists():
        # link beside the target and rename: a reader (or a copy of the tree) never sees a half-written library
        tmp = CUDA_LIB.with_suffix(".so.tmp")
        _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"])
        os.replace(tmp, CUDA_LIB)
    return CUDA_LIB


def build_rt(force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.hpp"))
    sources = sorted(CSRC.glob("*.cpp"))
    cxx = os.environ.get("CXX", "g++")
    objs, jobs, stamps = [], [], []
    for src in sources:
        obj = OBJ / (src.stem + ".cpp.o")
        objs.append(obj)
        if force or _stale(src, obj, headers, CXX_FLAGS):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
            stamps.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
        for src, obj in stamps:
            _stamp(src, obj, headers, CXX_FLAGS)
    if sources and (jobs or not RT_LIB.exists()):
        tmp = RT_LIB.with_suffix(".so.tmp")
        _run([cxx, "-shared", "-pthread", "-o", str(tmp), *map(str, objs)])
        os.replace(tmp, RT_LIB)
    return RT_LIB


_DECL_RE = None


def cuda_entry_points() -> list[tuple[str, str]]:
    """``(file name, declaration)`` of every ``extern "C"`` entry point defined in ``csrc/*.cu``: the C ABI of
    ``libscirust_b200_cuda.so``. Declarations are the definitions' signatures with the body cut off."""
    import re
    global _DECL_RE
    if _DECL_RE is None:
        _DECL_RE = re.compile(r'^extern "C" ([^;{]*?\))\s*\{', re.S | re.M)
    out = []
    for src in sorted(CSRC.glob("*.cu")):
        for m in _DECL_RE.finditer(src.read_text()):
            out.append((src.name, " ".join(m.group(1).split())))
    return out


API_BEGIN = "// ---- entry points (generated from the definitions by scirust_b200._build.write_api_header) ----"
API_END = "// ---- end of entry points ----"


def api_header_text() -> str:
    """api.h: the fixed preamble (error codes) plus one declaration per entry point, grouped by source file."""
    path = CSRC / "api.h"
    text = path.read_text()
    head = text.split("#ifdef __cplusplus")[0]
    lines = [head.rstrip(), "", "#ifdef __cplusplus", 'extern "C" {', "#endif", "", API_BEGIN]
    cur = None
    for fname, decl in cuda_entry_points():
        if fname != cur:
            lines += ["", f"// {fname}"]
            cur = fname
        lines.append(decl + ";")
    lines += ["", API_END, "", "#ifdef __cplusplus", "}", "#endif", ""]
    return "\n".join(lines)


def write_api_header() -> bool:
    """Regenerate ``csrc/api.h``; returns True when the file changed."""
    path = CSRC / "api.h"
    new = api_header_text()
    if path.read_text() == new:
        return False
    path.write_text(new)
    return True


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force=force, verbose=verbose)
    build_rt(force=force)


if __name__ == "__main__":
    if "--api-header" in sys.argv:
        print("api.h", "rewritten" if write_api_header() else "up to date")
        sys.exit(0)
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", CUDA_LIB, RT_LIB)

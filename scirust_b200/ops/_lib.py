"""ctypes bindings for the two native libraries.

``cuda()`` returns the handle of ``libscirust_b200_cuda.so`` (sm_100a kernels) and
``rt()`` the handle of ``libscirust_b200_rt.so`` (CPU runtime). Both are built in-tree by
``scirust_b200._build``; if a library is missing it is built on first use when a compiler
is present, otherwise a clear error is raised - on a GPU machine the ops never fall back
to another implementation silently.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

from .. import _build

_cuda = None
_rt = None

vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

ERRORS = {1: "bad argument", 2: "misaligned pointer or pitch", 3: "driver entry point unavailable",
          4: "kernel launch failed", 5: "size beyond supported maximum", 6: "runtime error"}

STATUS = {0: "ok", 1: "timeout: TMA stage never filled", 2: "timeout: stage never freed",
          3: "timeout: accumulator never completed", 4: "timeout: accumulator never drained",
          5: "timeout: peer flag never arrived", 6: "timeout", 7: "bad argument on device"}

_CUDA_SIGS = {
    "sb_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp, vp],
    "sb_gemm_pair_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, i32, vp, vp],
    "sb_rmsnorm_fwd": [vp, vp, vp, vp, i32, i32, i32, i32, f32, vp],
    "sb_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, vp],
    "sb_rope": [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, i32, vp],
    "sb_swiglu_fwd": [vp, vp, i32, i32, vp],
    "sb_swiglu_bwd": [vp, vp, vp, i32, i32, vp],
    "sb_add_bf16": [vp, vp, vp, sz, vp],
    "sb_embed_fwd": [vp, vp, vp, i32, i32, i32, vp],
    "sb_embed_bwd": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "sb_ce_fwd_bwd": [vp, vp, vp, vp, i32, i32, i32, f32, vp],
    "sb_ce_shard_stats": [vp, vp, vp, i32, i32, i32, i32, vp],
    "sb_ce_shard_grad": [vp, vp, vp, vp, i32, i32, i32, i32, f32, vp],
    "sb_sumsq": [vp, sz, i32, vp, vp, i32, vp],
    "sb_optim_step": [vp, vp, vp, vp, i32, vp, sz, sz, f32, f32, f32, f32, f32, f32, f32, vp, f32, f32, i32, vp],
    "sb_cast": [vp, vp, sz, i32, f32, vp],
}


class NativeError(RuntimeError):
    pass


class CollectiveTimeout(NativeError):
    """A bounded wait inside a kernel (peer flag, mbarrier) ran out; the data that kernel was to produce is
    incomplete, so the step that contained it must not be trusted."""

    def __init__(self, code: int):
        super().__init__(f"device kernel reported: {STATUS.get(code, code)}")
        self.code = code


def _load(path: Path, builder) -> C.CDLL:
    if not path.exists():
        builder()
    if not path.exists():
        raise NativeError(f"native library {path.name} is missing and could not be built")
    return C.CDLL(str(path))


def cuda() -> C.CDLL:
    global _cuda
    if _cuda is None:
        lib = _load(_build.CUDA_LIB, _build.build_cuda)
        for name, sig in _CUDA_SIGS.items():
            if hasattr(lib, name):
                fn = getattr(lib, name)
                fn.argtypes = sig
                fn.restype = i32
        _cuda = lib
    return _cuda


def register(name: str, sig: list) -> None:
    """Declare the signature of an entry point defined in another ops module."""
    _CUDA_SIGS[name] = sig
    if _cuda is not None and hasattr(_cuda, name):
        fn = getattr(_cuda, name)
        fn.argtypes = sig
        fn.restype = i32


def rt() -> C.CDLL:
    global _rt
    if _rt is None:
        _rt = _load(_build.RT_LIB, _build.build_rt)
    return _rt


def ptr(t) -> int | None:
    if t is None:
        return None
    return t.data_ptr()


# --------------------------------------------------------------------------------------------------
# Debug build of the op layer (SB_DEBUG_POISON=1): every buffer an op allocates for a kernel to fill is
#   * poisoned: all payload bytes 0xFF (bf16 / fp32 NaN, integer -1), so anything a kernel was supposed to write and
#     did not shows up in the first comparison instead of reading as a plausible stale value;
#   * fenced: 256 canary bytes (0xA5) on both sides, checked at every `check_status()` and by `check_canaries()`,
#     so a kernel that writes a tile past the end of its output is caught at the next synchronisation point.
# The stand-in for a memory-checking tool on hosts where none may be run; off by default (one branch per allocation).
# --------------------------------------------------------------------------------------------------
DEBUG_POISON = os.environ.get("SB_DEBUG_POISON") == "1"
_GUARD = 256
_fenced: list = []          # (weak reference to the backing byte buffer, payload bytes, tag)


def empty(shape, dtype, device, tag: str = "") -> torch.Tensor:
    """``torch.empty`` for op outputs and workspaces; poisoned and fenced in the debug build."""
    if not DEBUG_POISON or torch.device(device).type != "cuda":
        return torch.empty(shape, dtype=dtype, device=device)
    return fenced_empty(shape, dtype, device, tag)


def fenced_empty(shape, dtype, device, tag: str = "") -> torch.Tensor:
    import weakref
    n = 1
    for d in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)):
        n *= int(d)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    pad = (-nbytes) % 16
    raw = torch.empty(nbytes + pad + 2 * _GUARD, dtype=torch.uint8, device=device)
    raw[:_GUARD].fill_(0xA5)
    raw[_GUARD + nbytes:].fill_(0xA5)
    raw[_GUARD:_GUARD + nbytes].fill_(0xFF)
    out = raw[_GUARD:_GUARD + nbytes].view(dtype).view(shape)
    out._sb_fence = raw          # the fences are watched for as long as the tensor handed out is alive
    _fenced.append((weakref.ref(raw), nbytes, tag or f"{tuple(out.shape)} {dtype}"))
    if len(_fenced) > 4096:
        _fenced[:] = [e for e in _fenced if e[0]() is not None]
    return out


def check_canaries() -> None:
    """Debug build: raise if any live fenced buffer has a damaged canary (synchronises)."""
    if not _fenced:
        return
    live = []
    for ref, nbytes, tag in _fenced:
        raw = ref()
        if raw is None:
            continue
        live.append((ref, nbytes, tag))
        lo_ok = bool((raw[:_GUARD] == 0xA5).all())
        hi_ok = bool((raw[_GUARD + nbytes:] == 0xA5).all())
        if not (lo_ok and hi_ok):
            side = "before" if not lo_ok else "past the end of"
            raise NativeError(f"a kernel wrote {side} a buffer it was given: {tag}")
    _fenced[:] = live


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what}: {ERRORS.get(rc, rc)}")


def call(name: str, *args) -> None:
    fn = getattr(cuda(), name)
    check(fn(*args), name)


_status_words: dict[int, torch.Tensor] = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write an error code into."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[key] = w
    return w


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises if any kernel recorded a timeout."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise CollectiveTimeout(code)
    if DEBUG_POISON:
        check_canaries()


class DeferredStatus:
    """Reads the status word without stalling the stream: ``poll()`` queues a 4-byte copy into pinned host
    memory behind the work already issued and examines the copy queued by the PREVIOUS ``poll()`` (which has
    normally landed by then; otherwise its event is waited for). A non-zero code raises ``CollectiveTimeout``
    one call late at most, before another optimizer step can build on a partial reduction."""

    def __init__(self, device=None):
        self.word = status_word(device)
        self.host = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.events = [None, None]
        self.turn = 0

    def poll(self) -> None:
        cur, prev = self.turn, self.turn ^ 1
        if self.events[prev] is not None:
            self.events[prev].synchronize()
            code = int(self.host[prev][0])
            if code != 0:
                self.events = [None, None]
                self.word.zero_()
                raise CollectiveTimeout(code)
        self.host[cur].copy_(self.word, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[cur] = ev
        self.turn = prev

    def flush(self) -> None:
        """Synchronising check of everything issued so far."""
        self.events = [None, None]
        check_status(self.word.device)

"""bf16 GEMM on the hand-written tcgen05/TMEM/TMA kernel (csrc/gemm_tcgen05.cu).

Three storage forms cover forward, input-gradient and weight-gradient products without
any transpose copy (the reference calls cuBLASLt for the same three forms,
scirust-cuda/src/chain.rs:1037,1177,1228):

* ``matmul_nn(x[M,K], w[K,N])``       forward with ``[in, out]`` weights (x·W layout)
* ``matmul_nt(a[M,K], b[N,K])``       a · bᵀ (input gradient, tied LM head)
* ``matmul_tn(a[K,M], b[K,N])``       aᵀ · b (weight gradient), split-K in fixed order

CPU tensors take the plain PyTorch path (fp32 accumulate, bf16 result) so model logic can
be tested without a GPU; CUDA tensors always run the native kernel.
"""
from __future__ import annotations

import os

import torch

from . import _lib

_sm_count: dict[int, int] = {}
_workspaces: dict = {}


def num_sms(device=None) -> int:
    """Streaming multiprocessors of the device (148 on a B200), asked of the driver once per device."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    n = _sm_count.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_count[idx] = n
    return n

# Count of native kernel launches, for benchmark reporting.
launch_count = 0


def _workspace(nfloats: int, device) -> torch.Tensor:
    """Split-K / balanced-schedule scratch, one buffer per (device, stream): two products issued on two streams
    (backward on one, a collective's GEMM on another) must not share partial sums. The buffer is allocated while
    its stream is current, so the caching allocator orders its reuse on that stream."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _lib.stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nfloats:
        ws = _lib.empty(max(nfloats, 1 << 22), torch.float32, device)
        _workspaces[key] = ws
    return ws


def _pick_splits(M: int, N: int, K: int, bn: int) -> int:
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    num_kb = (K + 63) // 64
    sms = num_sms()
    if tiles >= sms // 2 or num_kb < 16:
        return 1
    # as many k-splits as keep tiles * splits within ONE wave of CTAs (a second, nearly empty wave doubles the time)
    s = min(max(1, sms // tiles), num_kb // 8, 16)
    return max(1, s)


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.dtype != torch.bfloat16 or t.stride(1) != 1:
        raise ValueError(f"{name}: expected a 2-D bf16 matrix with unit inner stride, got "
                         f"{tuple(t.shape)} {t.dtype} strides {t.stride()}")


# CTA-pair kernel (csrc/gemm_pair_tcgen05.cu): 256 x 256 tiles on two SMs. "auto" uses it for
# products with at least one full wave of such tiles and no split-K; SB_GEMM_PAIR=0/1 forces it.
PAIR_MODE = os.environ.get("SB_GEMM_PAIR", "auto")
BALANCED = os.environ.get("SB_GEMM_BALANCED", "1") != "0"
# SwiGLU forward / backward inside the GEMM epilogues (bit-identical to the separate kernels). Off by
# default: measured on one box back to back, the training step took 30.9 ms with the fused epilogues and
# 29.3 ms without - with K = 1024 a tile's main loop is too short to hide an epilogue that does exponentials,
# divisions and (backward) global loads before it can hand the accumulator back to the tensor cores.
FUSE_SWIGLU = os.environ.get("SB_FUSE_SWIGLU", "0") == "1"


# The balanced schedule pays a fix-up pass and fp32 scratch traffic (measured: about 20 us on 74 CTA pairs). Measured
# per shape on the training step's products (TFLOP/s, plain tiles against balanced):
#   3.46 waves (gate_up dgrad)  1248 / 1108     0.86 waves (LM-head dgrad)  1570 / 1129     0.59 waves (down wgrad) 1069 / 905
#   1.19 waves (gate_up wgrad)  1108 / 1367     6.76 waves (LM-head wgrad)  1245 / 1093
# so it is used when K is long AND the tiles make at least one whole wave AND the last, partial wave would leave more
# than 15 % of the machine idle; with less than one wave whole tiles (or explicit split-K) stay.
_BALANCED_MIN_K = 4096


# Long-K products with few output tiles (weight gradients: K = tokens) on CTA pairs with the balanced schedule:
# measured slower than explicit split-K on the single-CTA kernel (qkv wgrad 690 against 745 TFLOP/s, wo wgrad 531
# against 570), so off unless asked for.
_PAIR_LONGK = os.environ.get("SB_GEMM_PAIR_LONGK", "0") != "0"


def _use_pair(M, N, K, splits, bn) -> bool:
    if PAIR_MODE == "0" or splits not in (None, 1) or bn not in (None, 256):
        return False
    if PAIR_MODE == "1":
        return True
    pair_tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if pair_tiles >= 40 and K >= 256:
        return True
    return _PAIR_LONGK and BALANCED and pair_tiles >= 4 and K >= 8192 and M >= 256 and N >= 256


def _use_balanced(tiles: int, workers: int, K: int) -> bool:
    if not BALANCED or K < _BALANCED_MIN_K:
        return False
    if _BALANCED_MIN_K == 0:
        return True                       # tests force the schedule on every shape
    if tiles < workers:
        return _PAIR_LONGK and K >= 8192 and 2 * tiles < workers
    waves = tiles / workers
    whole = -(-tiles // workers)
    return tiles % workers != 0 and waves / whole < 0.85


class _Bias:
    """A [N] (or [1, N]) bf16 row added to every output row: the residual operand of the kernels with a
    zero row pitch, so the bias epilogue is the residual epilogue."""

    def __init__(self, t: torch.Tensor, N: int):
        t = t.reshape(-1)
        if t.numel() != N or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("bias must be a contiguous bf16 vector of N elements")
        self.t = t

    def data_ptr(self):
        return self.t.data_ptr()

    def stride(self, _dim):
        return 0


def _gemm(a, b, M, N, K, a_mn, b_mn, out, residual, splits, bn, bias=None):
    global launch_count
    if bias is not None:
        if residual is not None:
            raise ValueError("give either a residual or a bias")
        residual = _Bias(bias, N)
    _check2d(a, "a")
    _check2d(b, "b")
    if out is None:
        out = _lib.empty((M, N), torch.bfloat16, a.device)
    else:
        _check2d(out, "out")
        if tuple(out.shape) != (M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected {(M, N)}")
    if residual is not None and not isinstance(residual, _Bias):
        _check2d(residual, "residual")
        if tuple(residual.shape) != (M, N):
            raise ValueError("residual shape mismatch")
    if _use_pair(M, N, K, splits, bn):
        st = _lib.status_word(a.device)
        pair_tiles = ((M + 255) // 256) * ((N + 255) // 256)
        pairs = num_sms(a.device) // 2
        ws = _workspace(pairs * 3 * 256 * 256, a.device) if _use_balanced(pair_tiles, pairs, K) else None
        _lib.call("sb_gemm_pair_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None, M, N, K,
                  a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                  int(a_mn), int(b_mn), _lib.ptr(ws), None, 0, 0, None, 0, st.data_ptr(), _lib.stream())
        launch_count += 1
        return out
    if bn is None:
        bn = 128 if N <= 128 else 256
    if splits is None:
        # balanced schedule: whole waves one tile per CTA, the last partial wave's k-blocks dealt out
        # evenly over all SMs and finished by a fix-up pass (fixed k order)
        tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
        splits = 0 if _use_balanced(tiles, num_sms(a.device), K) else _pick_splits(M, N, K, bn)
    if splits == 0:
        ws = _workspace(num_sms(a.device) * 3 * 128 * 256, a.device)
    else:
        ws = _workspace(splits * M * N, a.device) if splits > 1 else None
    st = _lib.status_word(a.device)
    _lib.call("sb_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None, M, N, K,
              a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
              int(a_mn), int(b_mn), splits, _lib.ptr(ws), bn, st.data_ptr(), _lib.stream())
    launch_count += 2 if splits > 1 else 1
    return out



def _ref(a, b, residual, out):
    y = a.float() @ b.float()
    if residual is not None:
        y = y + residual.float()
    y = y.to(torch.bfloat16)
    if out is not None:
        out.copy_(y)
        return out
    return y


def matmul_nn(x, w, residual=None, out=None, splits=None, bn=None, bias=None):
    """x[M,K] @ w[K,N] (+ residual [M,N] | + bias [N]) -> bf16 [M,N]."""
    M, K = x.shape
    K2, N = w.shape
    if K != K2:
        raise ValueError(f"matmul_nn: inner dims differ ({K} vs {K2})")
    if not x.is_cuda:
        return _ref(x, w, residual if bias is None else bias.reshape(1, -1), out)
    return _gemm(x, w, M, N, K, False, True, out, residual, splits, bn, bias)


def matmul_nn_swiglu(x, wgu, out=None, act=None):
    """Gate/up projection with the SwiGLU fused into the GEMM epilogue: returns ``(gu, act)`` with
    ``gu = x @ wgu`` (bf16 ``[M, 2*ff]`` = [gate | up], kept for the backward pass) and
    ``act = silu(gate) * up`` (bf16 ``[M, ff]``), bit-identical to ``swiglu_fwd(matmul_nn(x, wgu))``.
    Runs on the CTA-pair kernel (each CTA of a pair stages one half: gate columns / matching up columns)."""
    global launch_count
    M, K = x.shape
    K2, N = wgu.shape
    ff = N // 2
    if K != K2 or N % 2:
        raise ValueError("matmul_nn_swiglu: shape mismatch")
    fused = x.is_cuda and PAIR_MODE != "0" and FUSE_SWIGLU and ff % 8 == 0 and M >= 256
    if not fused:
        from . import basic
        gu = matmul_nn(x, wgu, out=out)
        return gu, basic.swiglu_fwd(gu, out=act)
    _check2d(x, "x")
    _check2d(wgu, "wgu")
    if out is None:
        out = _lib.empty((M, N), torch.bfloat16, x.device)
    if act is None:
        act = _lib.empty((M, ff), torch.bfloat16, x.device)
    st = _lib.status_word(x.device)
    _lib.call("sb_gemm_pair_bf16", x.data_ptr(), wgu.data_ptr(), out.data_ptr(), None, M, N, K, x.stride(0),
              wgu.stride(0), out.stride(0), 0, 0, 1, None, act.data_ptr(), act.stride(0), ff, None, 0, st.data_ptr(),
              _lib.stream())
    launch_count += 1
    return out, act


def matmul_nt_swiglu_bwd(dy, wd, gu, out=None):
    """Backward of the SwiGLU feed-forward's middle: ``dgu = swiglu_bwd(gu, dy @ wdᵀ)`` with the
    element-wise part in the GEMM epilogue (``dy [M, d]``, ``wd [ff, d]``, ``gu [M, 2*ff]`` saved by the
    forward pass) -> bf16 ``[M, 2*ff]``; bit-identical to the two-step path."""
    global launch_count
    M, K = dy.shape
    ff, K2 = wd.shape
    if K != K2 or tuple(gu.shape) != (M, 2 * ff):
        raise ValueError("matmul_nt_swiglu_bwd: shape mismatch")
    fused = dy.is_cuda and PAIR_MODE != "0" and FUSE_SWIGLU and ff % 8 == 0 and M >= 256
    if not fused:
        from . import basic
        return basic.swiglu_bwd(gu, matmul_nt(dy, wd), out=out)
    _check2d(dy, "dy")
    _check2d(wd, "wd")
    _check2d(gu, "gu")
    if out is None:
        out = _lib.empty((M, 2 * ff), torch.bfloat16, dy.device)
    st = _lib.status_word(dy.device)
    _lib.call("sb_gemm_pair_bf16", dy.data_ptr(), wd.data_ptr(), out.data_ptr(), None, M, ff, K, dy.stride(0),
              wd.stride(0), out.stride(0), 0, 0, 0, None, None, 0, 0, gu.data_ptr(), gu.stride(0), st.data_ptr(),
              _lib.stream())
    launch_count += 1
    return out


def matmul_nt(a, b, residual=None, out=None, splits=None, bn=None, bias=None):
    """a[M,K] @ b[N,K]ᵀ (+ residual [M,N] | + bias [N]) -> bf16 [M,N]."""
    M, K = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError(f"matmul_nt: inner dims differ ({K} vs {K2})")
    if not a.is_cuda:
        return _ref(a, b.t(), residual if bias is None else bias.reshape(1, -1), out)
    return _gemm(a, b, M, N, K, False, False, out, residual, splits, bn, bias)


def matmul_tn(a, b, residual=None, out=None, splits=None, bn=None):
    """a[K,M]ᵀ @ b[K,N] (+ residual) -> bf16 [M,N]; the weight-gradient form."""
    K, M = a.shape
    K2, N = b.shape
    if K != K2:
        raise ValueError(f"matmul_tn: inner dims differ ({K} vs {K2})")
    if not a.is_cuda:
        return _ref(a.t(), b, residual, out)
    return _gemm(a, b, M, N, K, True, True, out, residual, splits, bn)


def matmul_tt_a(a, b, residual=None, out=None, splits=None, bn=None):
    """a[K,M]ᵀ @ b[N,K]ᵀ -> bf16 [M,N] (A MN-major, B K-major); completes the set."""
    K, M = a.shape
    N, K2 = b.shape
    if K != K2:
        raise ValueError("matmul_tt_a: inner dims differ")
    if not a.is_cuda:
        return _ref(a.t(), b.t(), residual, out)
    return _gemm(a, b, M, N, K, True, False, out, residual, splits, bn)

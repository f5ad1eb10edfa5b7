"""Decode-time ops (csrc/decode.cu): weight-streaming GEMV for bf16 / int8 per-channel weights,
paged-KV append, split-KV GQA flash-decode, arg-max with device feedback, per-channel
quantisation. CPU tensors take the fp32 PyTorch statement of the same arithmetic."""
from __future__ import annotations

import math
import os

import torch

from . import _lib
from . import gemm as _g

BF = torch.bfloat16
vp, i32, f32 = _lib.vp, _lib.i32, _lib.f32
_lib.register("sb_gemv", [vp, i32, vp, i32, vp, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, i32, vp, f32, vp, vp])
_lib.register("sb_rope_kv_append", [vp, i32, i32, i32, i32, vp, vp, vp, vp, i32, i32, vp, vp, i32, vp])
_lib.register("sb_kv_append", [vp, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp, i32, vp])
_lib.register("sb_decode_attention", [vp, i32, vp, vp, i32, i32, vp, i32, i32, i32, i32, i32, f32, vp, vp, vp, vp, i32,
                                      vp])
_lib.register("sb_argmax", [vp, i32, i32, vp, vp, vp, vp, i32, i32, vp])
_lib.register("sb_quantize_per_channel", [vp, i32, i32, i32, vp, vp, vp])
_lib.register("sb_dequantize", [vp, vp, i32, i32, vp, vp])

_lib.register("sb_gemm_w8", [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp])

_ws: dict = {}


def _workspace(n, device):
    key = (str(device), _lib.stream())        # per stream: concurrent calls on two streams must not share scratch
    w = _ws.get(key)
    if w is None or w.numel() < n:
        w = _lib.empty(max(n, 1 << 22), torch.float32, device)
        _ws[key] = w
    return w


_lib.register("sb_set_pdl", [i32])


class dependent_launch:
    """Context manager: launch the decode-path kernels (GEMV, RoPE+append, flash-decode) inside the
    block with programmatic dependent launch, so each kernel's weight prefetch overlaps the tail of
    its predecessor. Only for call chains whose weights are not produced by the preceding kernel.
    Off unless ``SB_PDL=1``: with the 64 KB weight ring (three CTAs per SM) the early-scheduled
    dependents measured slower than plain stream order (4.85 against 3.69 ms per token at
    Llama-3-8B shape); with the earlier 96 KB ring it gained 5 %."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and os.environ.get("SB_PDL", "0") == "1"

    def __enter__(self):
        if self.enabled:
            _lib.call("sb_set_pdl", 1)
        return self

    def __exit__(self, *exc):
        if self.enabled:
            _lib.call("sb_set_pdl", 0)
        return False


_gemv_ws: dict = {}


def _gemv_workspace(n, device):
    """Workspace of the GEMV: 4096 counter words (kept zero by the kernel) + split partials; one per (device,
    stream), so that GEMVs issued on two streams share neither counters nor partial sums."""
    key = (str(device), _lib.stream())
    w = _gemv_ws.get(key)
    if w is None or w.numel() < n:
        w = torch.zeros(max(n, 1 << 22), dtype=torch.float32, device=device)
        _gemv_ws[key] = w
    return w


class QuantWeight:
    """int8 weight ``q [K, N]`` with one fp32 scale per output column (x.W layout):
    ``W ~= q * scale[None, :]`` (scirust-core/src/quantization.rs:95-125)."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor):
        self.q, self.scale = q, scale
        self._qt = None

    def transposed(self) -> torch.Tensor:
        """The codes as ``[N, K]`` (K contiguous, rows padded to 16 bytes): the operand layout of the W8A8 GEMM."""
        if self._qt is None:
            K, N = self.q.shape
            Kp = (K + 15) // 16 * 16
            t = torch.zeros((N, Kp), dtype=torch.int8, device=self.q.device)
            t[:, :K] = self.q.t()
            self._qt = t
        return self._qt

    @property
    def shape(self):
        return self.q.shape

    def dequantize(self) -> torch.Tensor:
        if not self.q.is_cuda:
            return (self.q.float() * self.scale[None, :]).to(BF)
        K, N = self.q.shape
        w = _lib.empty((K, N), BF, self.q.device)
        _lib.call("sb_dequantize", self.q.data_ptr(), self.scale.data_ptr(), K, N, w.data_ptr(), _lib.stream())
        _g.launch_count += 1
        return w


def quantize_per_channel(w: torch.Tensor) -> QuantWeight:
    K, N = w.shape
    if not w.is_cuda:
        wf = w.float()
        mx = wf.abs().amax(0)
        scale = torch.where(mx == 0, torch.ones_like(mx), mx / 127.0)
        v = wf / scale[None, :]
        q = torch.where(v >= 0, torch.floor(v + 0.5), torch.ceil(v - 0.5)).clamp(-128, 127).to(torch.int8)
        return QuantWeight(q, scale)
    w = w.contiguous()
    scale = _lib.empty(N, torch.float32, w.device)
    q = _lib.empty((K, N), torch.int8, w.device)
    _lib.call("sb_quantize_per_channel", w.data_ptr(), K, N, w.stride(0), scale.data_ptr(), q.data_ptr(),
              _lib.stream())
    _g.launch_count += 2
    return QuantWeight(q, scale)


def gemv_max_rows(w) -> int:
    """Rows up to which the weight-streaming kernels beat the tcgen05 GEMM (one block of 8 MMA columns; with 16
    or 32 rows the tensor-core GEMV is bound by the mma.sync rate: 58 and 111 us against 33 us for 117 MB)."""
    return 8


def _auto_splits(N, K, cols, M=1, quant=False):
    """k-splits of the weight-streaming GEMV: about two CTAs per SM, and a staged slice of X that fits the
    kernel's 64 KB: 16 bytes per k (8 rows of 16-bit values) in the tensor-core kernels, (K / splits) rows x
    {1,2,4,8} floats in the FMA kernels that SB_GEMV_FMA=1 selects."""
    ctas = (N + cols - 1) // cols
    s = max(1, min(148 * 2 // max(ctas, 1), K // 64))
    if ctas > 148 * 2 and not quant:
        # several waves of column blocks (an LM head): eight k-splits keep more CTAs streaming at once and shorten
        # the tail (4096 x 128256: 213 us with one split, 176 us with eight)
        s = max(1, min(8, K // 512))
    lim = 4096                                # 16 bytes of staged X per k in the tensor-core kernels
    if os.environ.get("SB_GEMV_FMA") == "1":
        mb = 1 if M <= 1 else 2 if M <= 2 else 4 if M <= 4 else 8
        lim = min(lim, 65536 // (4 * mb) // 8 * 8)
    return max(s, (K + lim - 1) // lim)


def gemv(x, w, residual=None, out=None, out_f32=None, splits=None, rms_weight=None, eps=1e-5, swiglu=False):
    """y[M,N] = f(x)[M,K] @ W (+ residual) for small M, streaming W once. ``w`` is a bf16 ``[K, N]``
    matrix or a ``QuantWeight``. Rows are processed in groups of 8. ``rms_weight`` fuses the RMSNorm of
    ``x`` into the load; ``swiglu`` treats ``x`` as a fused ``[gate | up]`` row of width 2K."""
    quant = isinstance(w, QuantWeight)
    wm = w.q if quant else w
    K, N = wm.shape
    M = x.shape[0]
    if not x.is_cuda:
        if rms_weight is not None:
            xf = x.float()
            x = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * rms_weight.float()).to(BF)
        elif swiglu:
            g, u = x[:, :K].float(), x[:, K:].float()
            x = (g * torch.sigmoid(g) * u).to(BF)
        wf = (w.q.float() if quant else w.float())
        y = x.float() @ wf
        if quant:
            y = y * w.scale[None, :]
        if residual is not None:
            y = y + residual.float()
        if out_f32 is not None:
            out_f32.copy_(y)
        if out is not None:
            out.copy_(y.to(BF))
            return out
        return y.to(BF) if out_f32 is None else out_f32
    if out is None and out_f32 is None:
        out = _lib.empty((M, N), BF, x.device)
    grp = 8                                   # rows per call
    if splits is None:
        splits = _auto_splits(N, K, 512 if quant else 256, min(M, grp), quant)
    splits = max(splits, (K + 4095) // 4096)
    ws = _gemv_workspace(4096 + splits * min(M, grp) * N, x.device)
    st = _lib.status_word(x.device)
    for m0 in range(0, M, grp):
        mb = min(grp, M - m0)
        xs = x[m0:m0 + mb]
        _lib.call("sb_gemv", xs.data_ptr(), xs.stride(0), wm.data_ptr(), wm.stride(0),
                  w.scale.data_ptr() if quant else None,
                  residual[m0:m0 + mb].data_ptr() if residual is not None else None,
                  residual.stride(0) if residual is not None else 0,
                  out[m0:m0 + mb].data_ptr() if out is not None else None, out.stride(0) if out is not None else 0,
                  out_f32[m0:m0 + mb].data_ptr() if out_f32 is not None else None, mb, N, K, int(quant), splits,
                  ws.data_ptr(), 1 if rms_weight is not None else (2 if swiglu else 0), _lib.ptr(rms_weight),
                  float(eps), st.data_ptr(), _lib.stream())
        _g.launch_count += 1
    return out if out is not None else out_f32


_lib.register("sb_gemv_allreduce", [vp, i32, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, i32, vp, f32,
                                    vp, vp, vp, vp, i32, i32, i32, i32, vp, vp])


def gemv_allreduce(x, w, chan, residual=None, out=None, splits=None, swiglu=False):
    """out[M,N] = residual + sum over the ranks of ``chan`` of f(x_r)[M,K_r] @ W_r, M <= 8, in ONE launch per rank:
    the row-parallel product of tensor-parallel decoding with its all-reduce done by the CTAs that finish each block
    of output columns (csrc/decode.cu: ``sb_gemv_allreduce``). ``chan`` is a ``GemvAllReduceChannel``
    (parallel/small_collectives.py) that owns the peer-mapped receive buffers, flags and the epoch word."""
    quant = isinstance(w, QuantWeight)
    wm = w.q if quant else w
    K, N = wm.shape
    M = x.shape[0]
    if M > chan.rows or N > chan.n_max:
        raise ValueError("gemv_allreduce: product larger than the channel was sized for")
    if out is None:
        out = _lib.empty((M, N), BF, x.device)
    if splits is None:
        splits = _auto_splits(N, K, 512 if quant else 256, M, quant)
    splits = max(splits, (K + 4095) // 4096)
    ws = _gemv_workspace(4096 + splits * M * N, x.device)
    st = _lib.status_word(x.device)
    _lib.call("sb_gemv_allreduce", x.data_ptr(), x.stride(0), wm.data_ptr(), wm.stride(0),
              w.scale.data_ptr() if quant else None, _lib.ptr(residual),
              residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0), M, N, K, int(quant),
              splits, ws.data_ptr(), 2 if swiglu else 0, None, 1e-5, chan.recv_ptrs(N), chan.flag_ptrs,
              chan.state.data_ptr(), chan.state.data_ptr() + 128, chan.rank, chan.world, chan.rows, chan.wait_ms,
              st.data_ptr(), _lib.stream())
    _g.launch_count += 1
    return out


_lib.register("sb_gemv_argmax", [vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp, f32, vp, vp, vp, i32,
                                 i32, i32, vp, vp, vp, i32, i32, i32, vp, vp])
_amax_ws: dict = {}


def gemv_argmax(x, w, out_tokens=None, rms_weight=None, eps=1e-5, logits=None, chan=None, col_offset=0,
                generated=None, step=0, splits=None):
    """Greedy token of every row of ``f(x)[M,K] @ W`` (M <= 8) in ONE launch: the LM-head GEMV reduces its own
    outputs to one (value, column) per row and the last CTA writes the int64 token to ``out_tokens`` (the
    device-side feedback buffer), so the logits never make a round trip through memory unless ``logits`` (fp32
    [M, N]) is given (csrc/decode.cu: ``sb_gemv_argmax``; rule of scirust-cuda/src/bf16_lm_head_argmax.rs:46-176).
    ``chan`` (an ``ArgmaxChannel``) and ``col_offset`` make it the vocabulary-parallel head: every rank reduces its
    shard and the ranks exchange W candidates inside the same launch."""
    quant = isinstance(w, QuantWeight)
    wm = w.q if quant else w
    K, N = wm.shape
    M = x.shape[0]
    if M > 8:
        raise ValueError("gemv_argmax: at most 8 rows")
    if not x.is_cuda:
        lg = logits if logits is not None else torch.empty((M, N), dtype=torch.float32)
        gemv(x, w, out_f32=lg, rms_weight=rms_weight, eps=eps)
        if chan is not None:
            raise ValueError("gemv_argmax: the vocabulary-parallel form needs CUDA tensors")
        return argmax_rows(lg, out_tokens=out_tokens, generated=generated, step=step)
    if out_tokens is None:
        out_tokens = _lib.empty(M, torch.int64, x.device)
    if splits is None:
        splits = _auto_splits(N, K, 512 if quant else 256, M, quant)
    splits = max(splits, (K + 4095) // 4096)
    ws = _gemv_workspace(4096 + splits * M * N, x.device)
    key = (str(x.device), _lib.stream())
    aws = _amax_ws.get(key)
    if aws is None:
        aws = _amax_ws[key] = torch.zeros(16 + 2 * 8 * 4096, dtype=torch.int32, device=x.device)
    st = _lib.status_word(x.device)
    _lib.call("sb_gemv_argmax", x.data_ptr(), x.stride(0), wm.data_ptr(), wm.stride(0),
              w.scale.data_ptr() if quant else None, _lib.ptr(logits), M, N, K, int(quant), splits, ws.data_ptr(),
              1 if rms_weight is not None else 0, _lib.ptr(rms_weight), float(eps), aws.data_ptr(),
              out_tokens.data_ptr(), _lib.ptr(generated), generated.stride(0) if generated is not None else 0, step,
              col_offset, chan.cand_ptrs if chan is not None else None, chan.flag_ptrs if chan is not None else None,
              chan.state.data_ptr() if chan is not None else None, chan.rank if chan is not None else 0,
              chan.world if chan is not None else 1, chan.wait_ms if chan is not None else 0, st.data_ptr(),
              _lib.stream())
    _g.launch_count += 1
    return out_tokens


_lib.register("sb_gemm_skinny", [vp, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp])
SKINNY_MAX_ROWS = 64


def skinny_ok(x, w) -> bool:
    """Whether ``matmul_skinny`` takes this product: CUDA, 9..64 rows, and a weight layout its TMA maps accept."""
    if not x.is_cuda or os.environ.get("SB_SKINNY", "1") == "0":
        return False
    M = x.shape[0]
    if M <= 8 or M > SKINNY_MAX_ROWS:
        return False
    if isinstance(w, QuantWeight):
        K, N = w.q.shape
        return os.environ.get("SB_W8A8", "1") != "0" and K % 16 == 0 and N % 8 == 0
    K, N = w.shape
    return N % 8 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0


def matmul_skinny(x, w, residual=None, out=None, splits=0):
    """y[M,N] = x[M,K] @ W (+ residual) for 9..64 rows on the weight-streaming tcgen05 kernel
    (csrc/gemm_skinny_tcgen05.cu): the weight tile is the 128-row MMA operand and the activations the narrow one, so
    nearly all shared memory holds weight bytes in flight. ``w`` bf16 ``[K, N]``, or a ``QuantWeight`` (W8A8: the
    activations are quantised per row, the product is exact in int32 and rescaled once)."""
    quant = isinstance(w, QuantWeight)
    M, K = x.shape
    N = (w.q if quant else w).shape[1]
    if out is None:
        out = _lib.empty((M, N), BF, x.device)
    if quant:
        xq, sx = quantize_rows(x)
        xq = xq if xq.stride(0) % 16 == 0 else xq.contiguous()
        wt = w.transposed()
        args = (xq.data_ptr(), xq.stride(0), wt.data_ptr(), wt.stride(0))
        scales = (sx.data_ptr(), w.scale.data_ptr())
    else:
        args = (x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0))
        scales = (None, None)
    nt = (N + 127) // 128
    bke = 128 if quant else 64
    nkb = (K + bke - 1) // bke
    est = splits if splits > 0 else max(1, min(148 // max(nt, 1), max(nkb // 4, 1)))
    ws = _workspace(est * M * N, x.device) if est > 1 else None
    _lib.call("sb_gemm_skinny", *args, out.data_ptr(), out.stride(0), _lib.ptr(residual),
              residual.stride(0) if residual is not None else 0, M, N, K, int(quant), *scales,
              est, _lib.ptr(ws), _lib.status_word(x.device).data_ptr(), _lib.stream())
    _g.launch_count += 2 if est > 1 else 1
    return out


def matmul_int8(x, w: QuantWeight, residual=None, out=None):
    """The int8-weight product for batched decoding (more rows than the GEMV takes, fewer than prefill): the W8A8
    integer-tensor-core kernel (``matmul_w8a8``, the reference's dynamic-activation arithmetic) unless ``SB_W8A8=0``
    or the shape does not fit it, else the W8A16 dequant-fused kernel (``matmul_w8``)."""
    K, N = w.q.shape
    if x.is_cuda and os.environ.get("SB_W8A8", "1") != "0" and K % 16 == 0 and N % 8 == 0:
        return matmul_w8a8(x, w, residual=residual, out=out)
    return matmul_w8(x, w, residual=residual, out=out)


def matmul_w8(x, w: QuantWeight, residual=None, out=None, splits=None):
    """y[M,N] = (x[M,K] @ int8 W) * scale (+ residual) on the dequant-fused tcgen05 GEMM
    (csrc/gemm_w8_tcgen05.cu): the int8 codes are widened to bf16 in shared memory, so the weights
    cross HBM once as int8. For M <= 8 prefer ``gemv``."""
    M, K = x.shape
    N = w.q.shape[1]
    if not x.is_cuda:
        y = (x.float() @ w.q.float()) * w.scale[None, :]
        if residual is not None:
            y = y + residual.float()
        return y.to(BF)
    if out is None:
        out = _lib.empty((M, N), BF, x.device)
    if splits is None:
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        nkb = (K + 63) // 64
        splits = 1 if tiles >= 74 or nkb < 16 else max(1, min((148 + tiles - 1) // tiles, nkb // 8, 16))
    ws = _workspace(splits * M * N, x.device) if splits > 1 else None
    _lib.call("sb_gemm_w8", x.data_ptr(), w.q.data_ptr(), w.scale.data_ptr(), out.data_ptr(), _lib.ptr(residual), M, N,
              K, x.stride(0), w.q.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0, splits,
              _lib.ptr(ws), _lib.status_word(x.device).data_ptr(), _lib.stream())
    _g.launch_count += 2 if splits > 1 else 1
    return out


_lib.register("sb_quantize_rows", [vp, i32, vp, i32, vp, i32, i32, vp])
_lib.register("sb_gemm_i8", [vp, i32, vp, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, vp, vp, vp])


def quantize_rows(x):
    """Dynamic per-row activation quantisation: ``(q int8 [M, K], scale fp32 [M])`` with ``scale = max|x| / 127`` (1 for
    a zero row) and round half away from zero (scirust-core/src/quantization.rs:150-170)."""
    M, K = x.shape
    if not x.is_cuda:
        xf = x.float()
        mx = xf.abs().amax(1)
        s = torch.where(mx == 0, torch.ones_like(mx), mx / 127.0)
        v = xf / s[:, None]
        q = torch.where(v >= 0, torch.floor(v + 0.5), torch.ceil(v - 0.5)).clamp(-128, 127).to(torch.int8)
        return q, s
    Kp = (K + 15) // 16 * 16
    q = _lib.empty((M, Kp), torch.int8, x.device)
    s = _lib.empty((M,), torch.float32, x.device)
    if Kp != K:
        q.zero_()
    _lib.call("sb_quantize_rows", x.data_ptr(), x.stride(0), q.data_ptr(), Kp, s.data_ptr(), M, K, _lib.stream())
    _g.launch_count += 1
    return q[:, :K], s


def matmul_w8a8(x, w: QuantWeight, residual=None, out=None, splits=None):
    """y[M,N] = (quant_rows(x) . int8 W) * sx[m] * sw[n] (+ residual): the reference's quantised linear layer
    (dynamic per-row activation scales, int32 accumulation, one rescale; quantization.rs:150-190) on the integer
    tensor cores (csrc/gemm_i8_tcgen05.cu, tcgen05.mma.kind::i8). The int8 weights stream from HBM once and go from TMA
    straight into the MMA; integer accumulation makes the result independent of tiling and split-K. ``w`` keeps a
    K-major transposed copy of its codes for this kernel (made on first use)."""
    M, K = x.shape
    N = w.q.shape[1]
    xq, sx = quantize_rows(x)
    if not x.is_cuda:
        y = (xq.to(torch.int64) @ w.q.to(torch.int64)).float() * (sx[:, None] * w.scale[None, :])
        if residual is not None:
            y = y + residual.float()
        return y.to(BF)
    if K % 16 or N % 8:
        raise ValueError("matmul_w8a8: K must be a multiple of 16 and N of 8")
    qt = w.transposed()
    if out is None:
        out = _lib.empty((M, N), BF, x.device)
    if splits is None:
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        nkb = (K + 127) // 128
        splits = 1 if tiles >= 100 else max(1, min((148 * 2) // max(tiles, 1), nkb // 4, 16))
    ws = _workspace(splits * M * N, x.device) if splits > 1 else None
    xq_full = xq if xq.stride(0) % 16 == 0 else xq.contiguous()
    _lib.call("sb_gemm_i8", xq_full.data_ptr(), xq_full.stride(0), sx.data_ptr(), qt.data_ptr(), qt.stride(0),
              w.scale.data_ptr(), out.data_ptr(), out.stride(0), _lib.ptr(residual),
              residual.stride(0) if residual is not None else 0, M, N, K, splits, _lib.ptr(ws),
              _lib.status_word(x.device).data_ptr(), _lib.stream())
    _g.launch_count += 2 if splits > 1 else 1
    return out


def kv_append(qkv, H, Hkv, dh, pool, block_table, page, seq_of, pos):
    """Copy k/v heads of each row of ``qkv`` into the paged pool ``[n_blocks, 2, Hkv, page, dh]``."""
    n = qkv.shape[0]
    if not qkv.is_cuda:
        for t in range(n):
            b, p = int(seq_of[t]), int(pos[t])
            blk = int(block_table[b, p // page])
            kv = qkv[t, H * dh:].reshape(2, Hkv, dh)
            pool[blk, :, :, p % page, :] = kv
        return
    _lib.call("sb_kv_append", qkv.data_ptr(), qkv.stride(0), H, Hkv, dh, pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], page, seq_of.data_ptr(), pos.data_ptr(), n, _lib.stream())
    _g.launch_count += 1


def rope_kv_append(qkv, H, Hkv, dh, cos_t, sin_t, pool, block_table, page, seq_of, pos):
    """Decode step: rotate q/k of each new token in place at ``pos`` and append k, v to the pool."""
    if not qkv.is_cuda:
        from . import basic
        basic.rope_(qkv, H + Hkv, dh, 1, cos_t, sin_t, positions=pos)
        return kv_append(qkv, H, Hkv, dh, pool, block_table, page, seq_of, pos)
    _lib.call("sb_rope_kv_append", qkv.data_ptr(), qkv.stride(0), H, Hkv, dh, cos_t.data_ptr(), sin_t.data_ptr(),
              pool.data_ptr(), block_table.data_ptr(), block_table.shape[1], page, seq_of.data_ptr(), pos.data_ptr(),
              qkv.shape[0], _lib.stream())
    _g.launch_count += 1


def decode_attention_ref(q, pool, block_table, page, seq_len, H, Hkv, dh, scale=None):
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    B = q.shape[0]
    out = torch.zeros((B, H * dh), dtype=torch.float32, device=q.device)
    G = H // Hkv
    for b in range(B):
        L = int(seq_len[b])
        nb = (L + page - 1) // page
        blocks = block_table[b, :nb].long()
        kv = pool[blocks].float()                     # [nb, 2, Hkv, page, dh]
        k = kv[:, 0].permute(1, 0, 2, 3).reshape(Hkv, nb * page, dh)[:, :L]
        v = kv[:, 1].permute(1, 0, 2, 3).reshape(Hkv, nb * page, dh)[:, :L]
        qb = q[b, :H * dh].float().reshape(Hkv, G, dh)
        s = torch.einsum("hgd,hld->hgl", qb, k) * scale
        o = torch.einsum("hgl,hld->hgd", torch.softmax(s, -1), v)
        out[b] = o.reshape(-1)
    return out


def decode_attention(q, pool, block_table, page, seq_len, H, Hkv, dh, scale=None, n_splits=None, max_len=None):
    """Single-query GQA attention of each sequence over its paged KV. q: [B, >= H*dh] (RoPE'd)."""
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    B = q.shape[0]
    if not q.is_cuda:
        return decode_attention_ref(q, pool, block_table, page, seq_len, H, Hkv, dh, scale).to(BF)
    if n_splits is None:
        L = max_len if max_len is not None else block_table.shape[1] * page
        # about four 128-thread CTAs per SM, at least two 64-position tiles per split
        n_splits = max(1, min(64, (148 * 4 + B * Hkv - 1) // max(1, B * Hkv), (L + 127) // 128))
    ws = _workspace(B * H * n_splits * (dh + 2), q.device)
    ctr = _gemv_workspace(4096, q.device) if B * Hkv <= 2048 else None
    if ctr is None:
        raise ValueError("decode_attention: batch * kv_heads above 2048 is not supported")
    part_o = ws[:B * H * n_splits * dh]
    part_ml = ws[B * H * n_splits * dh:B * H * n_splits * (dh + 2)]
    out = _lib.empty((B, H * dh), BF, q.device)
    _lib.call("sb_decode_attention", q.data_ptr(), q.stride(0), pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], page, seq_len.data_ptr(), B, H, Hkv, dh, n_splits, float(scale),
              part_o.data_ptr(), part_ml.data_ptr(), ctr[2048:].data_ptr(), out.data_ptr(), out.stride(0),
              _lib.stream())
    _g.launch_count += 1
    return out


def argmax_rows(logits_f32, out_tokens=None, generated=None, step=0):
    """Greedy token per row (first maximum wins). Writes int64 tokens on the device."""
    rows, V = logits_f32.shape
    if not logits_f32.is_cuda:
        tok = torch.tensor([int(torch.argmax(r)) if not torch.isnan(r).any() else _nan_safe_argmax(r)
                            for r in logits_f32], dtype=torch.int64)
        if out_tokens is not None:
            out_tokens.copy_(tok)
            tok = out_tokens
        if generated is not None:
            generated[:, step] = tok
        return tok
    slabs = (V + 4095) // 4096
    pval = _lib.empty(rows * slabs, torch.float32, logits_f32.device)
    pidx = _lib.empty(rows * slabs, torch.int32, logits_f32.device)
    if out_tokens is None:
        out_tokens = _lib.empty(rows, torch.int64, logits_f32.device)
    _lib.call("sb_argmax", logits_f32.data_ptr(), rows, V, pval.data_ptr(), pidx.data_ptr(), out_tokens.data_ptr(),
              _lib.ptr(generated), generated.stride(0) if generated is not None else 0, step, _lib.stream())
    _g.launch_count += 2
    return out_tokens


def _nan_safe_argmax(r):
    best, bv = 0, float(r[0])
    for j in range(1, r.numel()):
        v = float(r[j])
        if v > bv:
            bv, best = v, j
    return best

"""GQA flash attention (prefill / training) on the tcgen05 kernels in csrc/attention_*_tcgen05.cu.

The activation layout is the fused projection output ``qkv [B*S, (H + 2*Hkv) * dh]`` (q heads, k heads,
v heads; RoPE already applied to q and k), so no per-head slicing copies exist (the reference slices and
re-concatenates per head: scirust-sciagent/src/cuda_model.rs:796-869).
"""
from __future__ import annotations

import math
import os

import torch

from . import _lib
from . import gemm as _g

_lib.register("sb_attention_fwd", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                   _lib.i32, _lib.i32, _lib.f32, _lib.i32, _lib.vp, _lib.vp])
_lib.register("sb_attention_fwd_pp", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32,
                                      _lib.i32, _lib.i32, _lib.f32, _lib.i32, _lib.vp, _lib.vp])
_lib.register("sb_attention_bwd", [_lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.i32,
                                   _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.i32, _lib.f32,
                                   _lib.i32, _lib.vp, _lib.vp])

# Head dimension 64 runs the kernel with two query tiles per CTA (output accumulator kept in tensor memory,
# rescaled only when a row maximum grows by more than 2^8); SB_ATT_FWD=single selects the one-tile kernel.
FWD_TWO_TILES = os.environ.get("SB_ATT_FWD", "pair") != "single"

# The backward pass spills its dS tiles (bf16 [B*H, S, S]) to a scratch buffer so that dQ is a streamed
# product instead of a second pass over scores and exponentials; above this size it recomputes instead.
DS_SCRATCH_LIMIT_BYTES = int(os.environ.get("SB_ATT_DS_SCRATCH_MB", "4096")) << 20
_ds_scratch: dict = {}


def _scratch(B, S, H, device):
    n = B * H * S * ((S + 63) // 64 * 64)
    if n * 2 > DS_SCRATCH_LIMIT_BYTES:
        return None
    key = str(device)
    t = _ds_scratch.get(key)
    if t is None or t.numel() < n:
        t = _lib.empty(n, torch.bfloat16, device)
        _ds_scratch[key] = t
    return t


def attention_ref(qkv, B, S, H, Hkv, dh, causal=True, scale=None):
    """fp32 dense reference: returns (O [B*S, H*dh] fp32, LSE [B,H,S] fp32)."""
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    x = qkv.float().reshape(B, S, H + 2 * Hkv, dh)
    q = x[:, :, :H].permute(0, 2, 1, 3)
    k = x[:, :, H:H + Hkv].permute(0, 2, 1, 3).repeat_interleave(H // Hkv, 1)
    v = x[:, :, H + Hkv:].permute(0, 2, 1, 3).repeat_interleave(H // Hkv, 1)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if causal:
        mask = torch.triu(torch.ones(S, S, dtype=torch.bool, device=qkv.device), 1)
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.matmul(torch.softmax(s, -1), v)
    return o.permute(0, 2, 1, 3).reshape(B * S, H * dh), lse


def attention_fwd(qkv, B, S, H, Hkv, dh, causal=True, scale=None, want_lse=True):
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    if not qkv.is_cuda:
        o, lse = attention_ref(qkv, B, S, H, Hkv, dh, causal, scale)
        return o.to(qkv.dtype), lse
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.dtype != torch.bfloat16:
        raise ValueError("qkv must be a 2-D bf16 matrix with unit inner stride")
    out = _lib.empty((B * S, H * dh), torch.bfloat16, qkv.device)
    lse = _lib.empty((B, H, S), torch.float32, qkv.device) if want_lse else None
    entry = "sb_attention_fwd_pp" if (FWD_TWO_TILES and dh == 64) else "sb_attention_fwd"
    _lib.call(entry, qkv.data_ptr(), out.data_ptr(), _lib.ptr(lse), B, S, H, Hkv, dh, qkv.stride(0),
              out.stride(0), float(scale), int(causal), _lib.status_word(qkv.device).data_ptr(), _lib.stream())
    _g.launch_count += 1
    return out, lse


def attention_bwd_ref(qkv, do, B, S, H, Hkv, dh, causal=True, scale=None):
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        o, _ = attention_ref(x, B, S, H, Hkv, dh, causal, scale)
        (g,) = torch.autograd.grad(o, x, do.float())
    return g


def attention_bwd_flash_ref(qkv, o, lse, do, B, S, H, Hkv, dh, causal=True, scale=None):
    """fp32 statement of the flash backward, written on the SAVED normaliser and output like the kernels:
    P = exp(S - lse), delta = rowsum(dO * O), dS = P * (dP - delta). With the block's own (o, lse) it equals
    ``attention_bwd_ref``; with the merged (o, lse) of a ring of KV blocks it is that block's share of the gradient,
    which is what context parallelism needs."""
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    rep = H // Hkv
    x = qkv.float().reshape(B, S, H + 2 * Hkv, dh)
    q = x[:, :, :H].permute(0, 2, 1, 3)
    k = x[:, :, H:H + Hkv].permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    v = x[:, :, H + Hkv:].permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    dof = do.float().reshape(B, S, H, dh).permute(0, 2, 1, 3)
    of = o.float().reshape(B, S, H, dh).permute(0, 2, 1, 3)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    p = torch.exp(s - lse.float()[..., None])
    if causal:
        p = p.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=qkv.device), 1), 0.0)
    p = torch.nan_to_num(p, nan=0.0)                       # rows with lse = -inf (no visible key) contribute nothing
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, v.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta)
    dq = torch.matmul(ds, k) * scale
    dk = torch.matmul(ds.transpose(-1, -2), q) * scale
    dk = dk.reshape(B, Hkv, rep, S, dh).sum(2)
    dv = dv.reshape(B, Hkv, rep, S, dh).sum(2)
    g = torch.cat([dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)], 2)
    return g.reshape(B * S, (H + 2 * Hkv) * dh)


def attention_bwd(qkv, o, lse, do, B, S, H, Hkv, dh, causal=True, scale=None):
    """Gradient w.r.t. the fused qkv matrix (same layout), deterministic (no atomics)."""
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    if not qkv.is_cuda:
        return attention_bwd_flash_ref(qkv, o, lse, do, B, S, H, Hkv, dh, causal, scale).to(qkv.dtype)
    dqkv = torch.empty_like(qkv)
    delta = _lib.empty((B, H, S, 2), torch.float32, qkv.device)
    ds = _scratch(B, S, H, qkv.device)
    _lib.call("sb_attention_bwd", qkv.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(), dqkv.data_ptr(),
              delta.data_ptr(), _lib.ptr(ds), B, S, H, Hkv, dh, qkv.stride(0), o.stride(0), do.stride(0), float(scale),
              int(causal), _lib.status_word(qkv.device).data_ptr(), _lib.stream())
    _g.launch_count += 3
    return dqkv

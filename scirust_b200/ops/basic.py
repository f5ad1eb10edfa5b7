"""Bandwidth-bound ops: RMSNorm, RoPE, SwiGLU, embedding, softmax-cross-entropy, sum of
squares, fused optimizer step, casts. CUDA tensors run csrc/kernels_basic.cu; CPU tensors
run the fp32 PyTorch statement of the same arithmetic (also the oracle in the tests).

Reference semantics: scirust-cuda/src/chain.rs (rmsnorm_fast :423, rope :225, swiglu :55,
embed :247/:579, ce_loss_grad :637, adamw_norm :707, sumsq :742) and the CPU oracles in
scirust-gpu/src/ops.rs (cpu_rms_norm :131, cpu_rope :634, cpu_adamw_step :970,
cpu_cross_entropy :997).
"""
from __future__ import annotations

import math

import torch

from . import _lib
from . import gemm as _g

BF = torch.bfloat16


def _count(n=1):
    _g.launch_count += n


# --------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps=1e-5, out=None, want_inv=True):
    """y = x * rsqrt(mean(x², -1) + eps) * w ; returns (y, inv_rms fp32 [rows] or None)."""
    rows, cols = x.shape
    if not x.is_cuda:
        xf = x.float()
        inv = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = (xf * inv[:, None] * w.float()).to(x.dtype)
        if out is not None:
            out.copy_(y)
            y = out
        return y, (inv if want_inv else None)
    if out is None:
        out = _lib.empty((rows, cols), BF, x.device)
    inv = _lib.empty(rows, torch.float32, x.device) if want_inv else None
    _lib.call("sb_rmsnorm_fwd", x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(inv), rows, cols,
              x.stride(0), out.stride(0), float(eps), _lib.stream())
    _count()
    return out, inv


def rmsnorm_bwd(dy, x, w, inv, dres=None, dw_out=None, want_dw=True):
    """Returns (dx [+ dres], dw). dw is written into ``dw_out`` (bf16 or fp32 [cols]) if given."""
    rows, cols = x.shape
    if not x.is_cuda:
        xf, g = x.float(), dy.float() * w.float()
        r = inv[:, None]
        dx = r * (g - xf * r * r * (g * xf).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.float()
        dw = (dy.float() * xf * r).sum(0) if want_dw else None
        if dw is not None and dw_out is not None:
            dw_out.copy_(dw.to(dw_out.dtype))
            dw = dw_out
        return dx.to(x.dtype), dw
    x = x.contiguous()
    dy = dy.contiguous()
    dx = torch.empty_like(x)
    part = dwf = dwb = None
    if want_dw:
        chunks = (rows + 255) // 256
        part = _lib.empty(chunks * cols, torch.float32, x.device)
        if dw_out is None:
            dw_out = _lib.empty(cols, torch.float32, x.device)
        if dw_out.dtype == torch.float32:
            dwf = dw_out
        else:
            dwb = dw_out
    _lib.call("sb_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), inv.data_ptr(), _lib.ptr(dres),
              dx.data_ptr(), _lib.ptr(part), _lib.ptr(dwf), _lib.ptr(dwb), rows, cols, _lib.stream())
    _count(3 if want_dw else 1)
    return dx, dw_out


# --------------------------------------------------------------------------- RoPE
_rope_tables: dict = {}


def rope_table(max_pos: int, dh: int, theta: float, device):
    """fp32 cos/sin tables [max_pos, dh/2] with head-local frequency theta^(-2p/dh)."""
    key = (max_pos, dh, float(theta), str(device))
    t = _rope_tables.get(key)
    if t is None:
        p = torch.arange(dh // 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * p / dh)
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * freq[None, :]
        t = (torch.cos(ang).float().to(device).contiguous(), torch.sin(ang).float().to(device).contiguous())
        _rope_tables[key] = t
    return t


def rope_(x, n_heads, dh, seq_len, cos_t, sin_t, offset=0, positions=None, backward=False):
    """Rotate the first n_heads*dh columns of x [rows, ld] in place (interleaved pairs)."""
    rows = x.shape[0]
    if not x.is_cuda:
        if positions is None:
            pos = (torch.arange(rows) % seq_len) + offset
        else:
            pos = positions.long()
        c = cos_t[pos][:, None, :]
        s = sin_t[pos][:, None, :] * (-1.0 if backward else 1.0)
        v = x[:, : n_heads * dh].float().reshape(rows, n_heads, dh // 2, 2)
        x0, x1 = v[..., 0], v[..., 1]
        o = torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).reshape(rows, n_heads * dh)
        x[:, : n_heads * dh] = o.to(x.dtype)
        return x
    _lib.call("sb_rope", x.data_ptr(), x.stride(0), rows, n_heads, dh, seq_len, offset, _lib.ptr(positions),
              cos_t.data_ptr(), sin_t.data_ptr(), int(backward), _lib.stream())
    _count()
    return x


# --------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(gu, out=None):
    """gu [rows, 2*ff] = [gate | up] -> silu(gate) * up  [rows, ff]."""
    rows, two_ff = gu.shape
    ff = two_ff // 2
    if not gu.is_cuda:
        g, u = gu[:, :ff].float(), gu[:, ff:].float()
        return (g * torch.sigmoid(g) * u).to(gu.dtype)
    if out is None:
        out = _lib.empty((rows, ff), BF, gu.device)
    _lib.call("sb_swiglu_fwd", gu.data_ptr(), out.data_ptr(), rows, ff, _lib.stream())
    _count()
    return out


def swiglu_bwd(gu, dh, out=None):
    rows, two_ff = gu.shape
    ff = two_ff // 2
    if not gu.is_cuda:
        g, u, d = gu[:, :ff].float(), gu[:, ff:].float(), dh.float()
        s = torch.sigmoid(g)
        return torch.cat((d * u * s * (1 + g * (1 - s)), d * g * s), 1).to(gu.dtype)
    if out is None:
        out = torch.empty_like(gu)
    _lib.call("sb_swiglu_bwd", gu.data_ptr(), dh.data_ptr(), out.data_ptr(), rows, ff, _lib.stream())
    _count()
    return out


def add(a, b, out=None):
    if not a.is_cuda:
        return (a.float() + b.float()).to(a.dtype)
    if out is None:
        out = torch.empty_like(a)
    _lib.call("sb_add_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _lib.stream())
    _count()
    return out


# --------------------------------------------------------------------------- embedding
def embed_fwd(table, tokens):
    n = tokens.numel()
    vocab, d = table.shape
    if not table.is_cuda:
        return table[tokens.reshape(-1).clamp(0, vocab - 1)]
    out = _lib.empty((n, d), table.dtype, table.device)
    _lib.call("sb_embed_fwd", table.data_ptr(), tokens.data_ptr(), out.data_ptr(), n, d, vocab, _lib.stream())
    _count()
    return out


def embed_bwd(dy, tokens, dtable, accumulate=True):
    """dtable[tok] (+)= sum of dy rows with that token, added in ascending row order."""
    vocab, d = dtable.shape
    flat = tokens.reshape(-1)
    n = flat.numel()
    if not dy.is_cuda:
        acc = dtable.float() if accumulate else torch.zeros_like(dtable, dtype=torch.float32)
        acc.index_add_(0, flat.clamp(0, vocab - 1), dy.float())
        dtable.copy_(acc.to(dtable.dtype))
        return dtable
    if not accumulate:
        dtable.zero_()
    sorted_tok, perm = torch.sort(flat, stable=True)
    _lib.call("sb_embed_bwd", dy.data_ptr(), sorted_tok.data_ptr(), perm.data_ptr(), dtable.data_ptr(), n, d,
              vocab, 1, _lib.stream())
    _count()
    return dtable


# --------------------------------------------------------------------------- cross entropy
def ce_fwd_bwd(logits, targets, grad_scale, dlogits=None, in_place=True):
    """Per-row loss (fp32) and d = (softmax - onehot) * grad_scale.

    With ``in_place`` the gradient overwrites ``logits``. Targets >= vocab clamp to the last
    id; negative targets are ignored (zero loss, zero gradient).
    """
    rows, cols = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        tg = targets.reshape(-1).clamp(max=cols - 1)
        ign = tg < 0
        tgc = tg.clamp(min=0)
        lse = torch.logsumexp(lf, -1)
        loss = lse - lf.gather(1, tgc[:, None])[:, 0]
        p = torch.softmax(lf, -1)
        p[torch.arange(rows), tgc] -= 1
        p *= grad_scale
        loss = torch.where(ign, torch.zeros_like(loss), loss)
        p[ign] = 0
        d = p.to(logits.dtype)
        if in_place:
            logits.copy_(d)
            d = logits
        return loss, d
    loss = _lib.empty(rows, torch.float32, logits.device)
    if dlogits is None:
        dlogits = logits if in_place else torch.empty_like(logits)
    _lib.call("sb_ce_fwd_bwd", logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), dlogits.data_ptr(), rows,
              cols, logits.stride(0), float(grad_scale), _lib.stream())
    _count()
    return loss, dlogits


def ce_shard_stats(logits, targets, v0):
    """Per-row (max, sum exp(x - max), target logit or 0) of the vocabulary shard [v0, v0 + cols): fp32 [rows, 3]."""
    rows, cols = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        m = lf.max(-1).values
        s = torch.exp(lf - m[:, None]).sum(-1)
        loc = targets.reshape(-1) - v0
        own = (loc >= 0) & (loc < cols) & (targets.reshape(-1) >= 0)
        t = torch.where(own, lf.gather(1, loc.clamp(0, cols - 1)[:, None])[:, 0], torch.zeros_like(m))
        return torch.stack([m, s, t], 1)
    stats = _lib.empty((rows, 3), torch.float32, logits.device)
    _lib.call("sb_ce_shard_stats", logits.data_ptr(), targets.data_ptr(), stats.data_ptr(), rows, cols,
              logits.stride(0), int(v0), _lib.stream())
    _count()
    return stats


def ce_shard_grad(logits, targets, v0, lse, grad_scale, in_place=True):
    """(exp(x - lse) - onehot) * grad_scale over the shard's columns; rows with a negative target give zeros."""
    rows, cols = logits.shape
    if not logits.is_cuda:
        p = torch.exp(logits.float() - lse[:, None])
        loc = targets.reshape(-1) - v0
        own = (loc >= 0) & (loc < cols)
        rws = torch.arange(rows)[own]
        p[rws, loc[own]] -= 1
        p *= grad_scale
        p[targets.reshape(-1) < 0] = 0
        d = p.to(logits.dtype)
        if in_place:
            logits.copy_(d)
            d = logits
        return d
    out = logits if in_place else torch.empty_like(logits)
    _lib.call("sb_ce_shard_grad", logits.data_ptr(), targets.data_ptr(), lse.data_ptr(), out.data_ptr(), rows, cols,
              logits.stride(0), int(v0), float(grad_scale), _lib.stream())
    _count()
    return out


def ce_loss_only(logits, targets):
    rows, cols = logits.shape
    if not logits.is_cuda:
        return ce_fwd_bwd(logits.clone(), targets, 0.0)[0]
    loss = _lib.empty(rows, torch.float32, logits.device)
    _lib.call("sb_ce_fwd_bwd", logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), None, rows, cols,
              logits.stride(0), 0.0, _lib.stream())
    _count()
    return loss


# --------------------------------------------------------------------------- reductions / optimizer
def sumsq(g, out=None, accumulate=False):
    """Deterministic sum of squares of a flat bf16/fp32 buffer -> fp32 scalar tensor [1]."""
    n = g.numel()
    if not g.is_cuda:
        s = g.float().pow(2).sum().reshape(1)
        if out is not None:
            out.copy_(out + s if accumulate else s)
            return out
        return s
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=g.device)
    part = _lib.empty((n + 4095) // 4096, torch.float32, g.device)
    _lib.call("sb_sumsq", g.data_ptr(), n, int(g.dtype == BF), part.data_ptr(), out.data_ptr(), int(accumulate),
              _lib.stream())
    _count(2)
    return out


MODE = {"adamw": 0, "adam": 1, "sgd": 2}


def optim_step(p, m, v, grad, p_bf16, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1,
               decay_end=None, grad_sumsq=None, max_grad_norm=0.0, grad_scale=1.0, mode="adamw"):
    """One fused optimizer step over flat buffers (fp32 p/m/v, bf16 or fp32 grad)."""
    n = p.numel()
    if decay_end is None:
        decay_end = n
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not p.is_cuda:
        scale = grad_scale
        if grad_sumsq is not None:
            sq = float(grad_sumsq[0]) * grad_scale * grad_scale
            if not (sq >= 0.0) or sq > 3.0e38:
                return
            norm = math.sqrt(sq)
            if max_grad_norm > 0 and norm > max_grad_norm:
                scale *= max_grad_norm / norm
        g = grad.float() * scale
        wd = torch.zeros(n)
        wd[:decay_end] = weight_decay
        if mode == "sgd":
            g = g + wd * p
            m.mul_(beta1).add_(g)
            p.sub_(lr * m)
        else:
            if mode == "adam":
                g = g + wd * p
            m.mul_(beta1).add_((1 - beta1) * g)
            v.mul_(beta2).add_((1 - beta2) * g * g)
            upd = (m / bc1) / (torch.sqrt(v / bc2) + eps)
            if mode == "adamw":
                upd = upd + wd * p
            p.sub_(lr * upd)
        if p_bf16 is not None:
            p_bf16.copy_(p.to(BF))
        return
    _lib.call("sb_optim_step", p.data_ptr(), m.data_ptr(), _lib.ptr(v), grad.data_ptr(), int(grad.dtype == BF),
              _lib.ptr(p_bf16), n, decay_end, float(lr), float(beta1), float(beta2), float(eps),
              float(weight_decay), float(bc1), float(bc2), _lib.ptr(grad_sumsq), float(max_grad_norm),
              float(grad_scale), MODE[mode], _lib.stream())
    _count()


_lib.register("sb_multi_cast_f32_bf16", [_lib.vp, _lib.vp, _lib.vp, _lib.i32, _lib.vp, _lib.i32, _lib.vp])


def multi_cast_to_bf16(srcs, dst, offsets, accumulate: bool = False):
    """Round fp32 tensors ``srcs[i]`` into ``dst[offsets[i] : offsets[i] + srcs[i].numel()]`` (flat bf16) with one
    launch per 96 tensors; ``accumulate`` adds to what the slice holds (fp32 add, one rounding)."""
    if not dst.is_cuda:
        for s_, o in zip(srcs, offsets):
            sl = dst[o:o + s_.numel()]
            v = s_.reshape(-1).float()
            sl.copy_((sl.float() + v) if accumulate else v)
        return
    import ctypes as C
    for c0 in range(0, len(srcs), 96):
        chunk = [t if t.is_contiguous() else t.contiguous() for t in srcs[c0:c0 + 96]]
        for t in chunk:
            if t.dtype != torch.float32:
                raise TypeError("multi_cast_to_bf16 takes fp32 sources")
        k = len(chunk)
        ps = (C.c_void_p * k)(*[t.data_ptr() for t in chunk])
        os_ = (C.c_ulonglong * k)(*[int(o) for o in offsets[c0:c0 + 96]])
        ns = (C.c_ulonglong * k)(*[t.numel() for t in chunk])
        _lib.call("sb_multi_cast_f32_bf16", ps, os_, ns, k, dst.data_ptr(), int(accumulate), _lib.stream())
        _count()

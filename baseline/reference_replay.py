"""Replay of the reference's CUDA route ("Route B") for the benchmark's reference arm.

The reference (CHECKUPAUTO/scirust) is a Rust workspace; without a Rust toolchain it cannot be built, but
its device code is CUDA C kept as string constants inside ``scirust-cuda/src/*.rs`` and compiled at run
time by NVRTC, and its GEMMs are cuBLASLt bf16 calls. This harness runs exactly that device work:

* the kernel source is read verbatim, at run time, from the copy of the reference kept under
  ``baseline/_ref/`` (``scirust-cuda/src/chain.rs``: the ``KERNELS_SRC`` string) and compiled by libnvrtc
  with no options, as ``cudarc::nvrtc::compile_ptx`` does (scirust-cuda/src/chain.rs:898);
* every operator of ``CudaChain`` is issued the way the reference issues it: a fresh zero-filled output
  per operator (``alloc_zeros`` = allocation + fill), the reference's grid/block shapes
  (``LaunchConfig::for_num_elems`` = blocks of 1024 threads; one block of 256 per row for the row kernels)
  and its three bf16 GEMM forms (``A.B``, ``A.B^T``, ``A^T.B``: chain.rs:1037-1083, 1177-1266) as cuBLAS
  bf16 GEMMs with fp32 accumulation through ``torch.mm``;
* the model code follows ``scirust-sciagent/src/cuda_model.rs`` call for call: three separate q/k/v
  products, attention as a loop over sequences and heads with materialised score matrices
  (``block_train`` :874-946, ``attention_train_sequence`` :795-832), the cached backward (:958-1100), the
  training step with per-tensor ``sumsq`` + ``adamw_norm`` launches (:1393-1523) and the cached decoder
  (``prefill_cached`` / ``decode_step_cached`` / ``generate_cached`` :450-581).

Nothing of this framework (kernels, models, engine) is imported here. Two host-side differences favour the
reference and are stated in the output: allocations come from PyTorch's caching allocator rather than
``cuMemAllocAsync``, and kernels are launched through ctypes on libcuda.
"""
from __future__ import annotations

import ctypes as C
import glob
import json
import math
import os
import re
import statistics
import sys
import time
from pathlib import Path

import torch

REF_ROOT = Path(__file__).resolve().parent / "_ref"
BF = torch.bfloat16


# ------------------------------------------------------------------------------------------------
# NVRTC + driver plumbing
# ------------------------------------------------------------------------------------------------
def _find_nvrtc() -> str:
    import site
    cands = []
    for sp in site.getsitepackages():
        cands += glob.glob(sp + "/nvidia/cuda_nvrtc/lib/libnvrtc.so*")
    cands += glob.glob("/usr/local/cuda/lib64/libnvrtc.so*")
    cands = [c for c in cands if "builtins" not in c]
    if not cands:
        raise RuntimeError("libnvrtc not found")
    return sorted(cands)[0]


def kernel_source() -> str:
    path = REF_ROOT / "scirust-cuda" / "src" / "chain.rs"
    if not path.exists():
        raise FileNotFoundError(f"{path} is missing: stage the reference sources under baseline/_ref first")
    text = path.read_text()
    m = re.search(r'const KERNELS_SRC: &str = r#"(.*?)"#;', text, re.S)
    if not m:
        raise RuntimeError("KERNELS_SRC not found in chain.rs")
    return m.group(1)


def compile_ptx(src: str) -> bytes:
    """NVRTC with no options (the reference's ``compile_ptx`` default)."""
    nvrtc = C.CDLL(_find_nvrtc())
    prog = C.c_void_p()
    rc = nvrtc.nvrtcCreateProgram(C.byref(prog), src.encode(), b"scirust_kernels.cu", 0, None, None)
    if rc != 0:
        raise RuntimeError(f"nvrtcCreateProgram: {rc}")
    rc = nvrtc.nvrtcCompileProgram(prog, 0, None)
    if rc != 0:
        n = C.c_size_t()
        nvrtc.nvrtcGetProgramLogSize(prog, C.byref(n))
        log = C.create_string_buffer(n.value)
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC compile failed:\n" + log.value.decode(errors="replace"))
    n = C.c_size_t()
    nvrtc.nvrtcGetPTXSize(prog, C.byref(n))
    ptx = C.create_string_buffer(n.value)
    nvrtc.nvrtcGetPTX(prog, ptx)
    nvrtc.nvrtcDestroyProgram(C.byref(prog))
    return ptx.raw


_CTYPE = {"size_t": C.c_size_t, "float": C.c_float, "int": C.c_int, "unsigned int": C.c_uint}


def parse_signatures(src: str) -> dict:
    """kernel name -> list of ctypes types (``c_void_p`` for pointers), read from the CUDA C source."""
    out = {}
    for m in re.finditer(r'extern "C" __global__ void (\w+)\s*\((.*?)\)\s*\{', src, re.S):
        name, params = m.group(1), m.group(2)
        types = []
        for p in params.split(","):
            p = " ".join(p.split())
            if "*" in p:
                types.append(C.c_void_p)
                continue
            t = re.sub(r"\bconst\b", "", p).strip()
            t = " ".join(t.split()[:-1])        # drop the parameter name
            if t not in _CTYPE:
                raise RuntimeError(f"{name}: unsupported parameter type {t!r}")
            types.append(_CTYPE[t])
        out[name] = types
    return out


class Kernels:
    """The reference's NVRTC module: every ``extern "C"`` kernel, launchable on torch's current stream."""

    def __init__(self):
        src = kernel_source()
        self.sigs = parse_signatures(src)
        ptx = compile_ptx(src)
        self.cu = C.CDLL("libcuda.so.1")
        self.cu.cuLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 6 + [C.c_uint, C.c_void_p, C.c_void_p,
                                                                          C.c_void_p]
        torch.zeros(1, device="cuda")          # make the primary context current on this thread
        mod = C.c_void_p()
        rc = self.cu.cuModuleLoadData(C.byref(mod), ptx)
        if rc != 0:
            raise RuntimeError(f"cuModuleLoadData: {rc}")
        self.fn = {}
        for name in self.sigs:
            f = C.c_void_p()
            rc = self.cu.cuModuleGetFunction(C.byref(f), mod, name.encode())
            if rc != 0:
                raise RuntimeError(f"cuModuleGetFunction({name}): {rc}")
            self.fn[name] = f
        self.launches = 0

    def launch(self, name: str, grid: int, block: int, *args):
        types = self.sigs[name]
        if len(args) != len(types):
            raise TypeError(f"{name}: {len(args)} arguments for {len(types)} parameters")
        vals = []
        for a, t in zip(args, types):
            if t is C.c_void_p:
                vals.append(C.c_void_p(a.data_ptr() if isinstance(a, torch.Tensor) else int(a)))
            else:
                vals.append(t(a))
        ptrs = (C.c_void_p * len(vals))(*[C.addressof(v) for v in vals])
        rc = self.cu.cuLaunchKernel(self.fn[name], max(1, grid), 1, 1, block, 1, 1, 0,
                                    torch.cuda.current_stream().cuda_stream, ptrs, None)
        if rc != 0:
            raise RuntimeError(f"cuLaunchKernel({name}): {rc}")
        self.launches += 1


def _elems(n: int):
    """``LaunchConfig::for_num_elems``: blocks of 1024 threads."""
    return (n + 1023) // 1024, 1024


# ------------------------------------------------------------------------------------------------
# CudaChain: one method per reference operator (same kernels, same launch shapes, fresh zeroed output)
# ------------------------------------------------------------------------------------------------
class Chain:
    def __init__(self):
        self.k = Kernels()
        self.gemms = 0

    @staticmethod
    def zeros(rows, cols, dtype=BF):
        return torch.zeros((rows, cols), dtype=dtype, device="cuda")

    # GEMM forms (cuBLAS bf16, fp32 accumulate, bf16 out)
    def matmul(self, a, b):
        self.gemms += 1
        c = self.zeros(a.shape[0], b.shape[1])
        return torch.mm(a, b, out=c)

    def matmul_bt(self, a, b):
        self.gemms += 1
        c = self.zeros(a.shape[0], b.shape[0])
        return torch.mm(a, b.t(), out=c)

    def matmul_at(self, a, b):
        self.gemms += 1
        c = self.zeros(a.shape[1], b.shape[1])
        return torch.mm(a.t(), b, out=c)

    def _binary(self, name, a, b):
        n = a.numel()
        c = self.zeros(*a.shape)
        self.k.launch(name, *_elems(n), c, a, b, n)
        return c

    def add(self, a, b):
        return self._binary("add_kernel", a, b)

    def swiglu(self, g, u):
        return self._binary("swiglu_kernel", g, u)

    def rms_norm(self, x, w, eps):
        rows, cols = x.shape
        out = self.zeros(rows, cols)
        self.k.launch("rmsnorm_fast_kernel", rows, 256, out, x, w, rows, cols, eps)
        return out

    def slice_cols(self, x, start, ncols):
        rows, src = x.shape
        out = self.zeros(rows, ncols)
        self.k.launch("slice_cols_kernel", *_elems(rows * ncols), out, x, rows, src, start, ncols)
        return out

    def concat_cols(self, parts):
        rows = parts[0].shape[0]
        cols = sum(p.shape[1] for p in parts)
        out = self.zeros(rows, cols)
        c0 = 0
        for p in parts:
            self.k.launch("place_cols_into_kernel", *_elems(rows * p.shape[1]), out, p, rows, p.shape[1], c0, cols)
            c0 += p.shape[1]
        return out

    def slice_rows(self, x, start, nrows):
        cols = x.shape[1]
        out = self.zeros(nrows, cols)
        self.k.launch("slice_rows_kernel", *_elems(nrows * cols), out, x, cols, start, nrows)
        return out

    def concat_rows(self, parts):
        cols = parts[0].shape[1]
        rows = sum(p.shape[0] for p in parts)
        out = self.zeros(rows, cols)
        r0 = 0
        for p in parts:
            self.k.launch("place_rows_kernel", *_elems(p.shape[0] * cols), out, p, cols, r0, p.shape[0])
            r0 += p.shape[0]
        return out

    def softmax(self, x):
        rows, cols = x.shape
        out = self.zeros(rows, cols)
        self.k.launch("softmax_fast_kernel", rows, 256, out, x, rows, cols)
        return out

    def attention_scores_ltr(self, q, keys):
        rows, dim = q.shape
        seq = keys.shape[0]
        out = self.zeros(rows, seq)
        self.k.launch("attention_scores_ltr_kernel", *_elems(rows * seq), out, q, keys, rows, seq, dim)
        return out

    def attention_context(self, w, v):
        rows, seq = w.shape
        dim = v.shape[1]
        out = self.zeros(rows, dim)
        self.k.launch("attention_context_kernel", *_elems(rows * dim), out, w, v, rows, seq, dim)
        return out

    def scale_causal_mask(self, x, scale, causal):
        rows, cols = x.shape
        out = self.zeros(rows, cols)
        self.k.launch("scale_mask_kernel", *_elems(rows * cols), out, x, rows, cols, scale, int(causal))
        return out

    def rope_head_local(self, x, head_dim, seq_len, offset, theta):
        rows, dim = x.shape
        out = self.zeros(rows, dim)
        self.k.launch("rope_kernel", *_elems(rows * (dim // 2)), out, x, rows, dim, head_dim, seq_len, offset, theta)
        return out

    def embed(self, tokens_host, table):
        toks = tokens_host.to("cuda", non_blocking=True)          # clone_htod of the u32 ids
        n, d = toks.numel(), table.shape[1]
        out = self.zeros(n, d)
        self.k.launch("embed_kernel", *_elems(n * d), out, toks, table, n, d)
        return out

    # ---- backward adjoints
    def softmax_backward(self, y, dy):
        rows, cols = y.shape
        dx = self.zeros(rows, cols)
        self.k.launch("softmax_bwd_fast_kernel", rows, 256, dx, y, dy, rows, cols)
        return dx

    def swiglu_backward(self, a, b, dc):
        n = a.numel()
        da, db = self.zeros(*a.shape), self.zeros(*a.shape)
        self.k.launch("swiglu_bwd_kernel", *_elems(n), da, db, a, b, dc, n)
        return da, db

    def rms_norm_backward(self, x, w, dy, eps):
        rows, cols = x.shape
        dx = self.zeros(rows, cols)
        self.k.launch("rmsnorm_bwd_fast_kernel", rows, 256, dx, x, w, dy, rows, cols, eps)
        return dx

    def rms_norm_gain_backward(self, x, dy, eps):
        rows, cols = x.shape
        inv = torch.zeros(rows, dtype=torch.float32, device="cuda")
        self.k.launch("rmsnorm_inv_kernel", rows, 256, inv, x, rows, cols, eps)
        dw = self.zeros(1, cols)
        self.k.launch("rmsnorm_gain_bwd_fast_kernel", *_elems(cols), dw, x, dy, inv, rows, cols)
        return dw

    def scale_causal_mask_backward(self, dout, scale, causal):
        rows, cols = dout.shape
        din = self.zeros(rows, cols)
        self.k.launch("scale_mask_bwd_kernel", *_elems(rows * cols), din, dout, rows, cols, scale, int(causal))
        return din

    def rope_head_local_backward(self, dy, head_dim, seq_len, offset, theta):
        rows, dim = dy.shape
        dx = self.zeros(rows, dim)
        self.k.launch("rope_bwd_kernel", *_elems(rows * (dim // 2)), dx, dy, rows, dim, head_dim, seq_len, offset,
                      theta)
        return dx

    def embed_backward(self, tokens_host, dout, vocab):
        # host-side sort of (token, row) pairs, as the reference does on the CPU (chain.rs embed_backward)
        n, d = tokens_host.numel(), dout.shape[1]
        tok = tokens_host.to(torch.int64).clamp(max=vocab - 1)
        order = torch.argsort(tok * n + torch.arange(n), stable=True)
        st = tok[order]
        uniq, counts = torch.unique_consecutive(st, return_counts=True)
        offsets = torch.zeros(uniq.numel() + 1, dtype=torch.int64)
        offsets[1:] = torch.cumsum(counts, 0)
        dtable = self.zeros(vocab, d)
        u_dev = uniq.to(torch.int32).to("cuda", non_blocking=True)
        o_dev = offsets.to(torch.int32).to("cuda", non_blocking=True)
        p_dev = order.to(torch.int32).to("cuda", non_blocking=True)
        self.k.launch("embed_bwd_sparse_kernel", *_elems(uniq.numel() * d), dtable, u_dev, o_dev, p_dev, dout,
                      uniq.numel(), d, vocab)
        return dtable

    def cross_entropy_loss_grad_resident(self, logits, targets_host):
        rows, cols = logits.shape
        tgt = targets_host.to("cuda", non_blocking=True)
        loss_rows = torch.zeros(rows, dtype=torch.float32, device="cuda")
        d = self.zeros(rows, cols)
        self.k.launch("ce_loss_grad_kernel", rows, 256, loss_rows, d, logits, tgt, rows, cols)
        return loss_rows, d

    def global_grad_sumsq(self, grads):
        accum = torch.zeros(1, dtype=torch.float32, device="cuda")
        for g in grads:
            n = g.numel()
            grid = (n + 255) // 256
            partials = torch.zeros(grid, dtype=torch.float32, device="cuda")
            self.k.launch("sumsq_partials_kernel", grid, 256, g, n, partials)
            self.k.launch("sumsq_finish_kernel", 1, 256, partials, grid, accum)
        return accum

    def adamw_step_with_norm(self, p, m, v, grad, view, lr, betas, eps, wd, step, sumsq, max_norm):
        n = p.numel()
        b1, b2 = betas
        bc1, bc2 = 1.0 - b1 ** step, 1.0 - b2 ** step
        self.k.launch("adamw_norm_kernel", *_elems(n), p, m, v, grad, view, n, lr, b1, b2, eps, wd, bc1, bc2, sumsq,
                      max_norm)


# ------------------------------------------------------------------------------------------------
# CudaModel / CudaTrainer (scirust-sciagent/src/cuda_model.rs)
# ------------------------------------------------------------------------------------------------
class RefConfig:
    def __init__(self, vocab, d_model, n_layers, n_heads, n_kv_heads, d_ff, theta, eps=1e-5):
        self.vocab, self.d_model, self.n_layers = vocab, d_model, n_layers
        self.n_heads, self.n_kv_heads, self.d_ff, self.theta, self.eps = n_heads, n_kv_heads, d_ff, theta, eps


PRESETS = {
    "gqa_12l": RefConfig(32000, 1024, 12, 16, 4, 2816, 10000.0),
    "350m": RefConfig(32768, 1024, 24, 16, 4, 2816, 1_000_000.0),
    "llama3_8b": RefConfig(128256, 4096, 32, 32, 8, 14336, 500000.0),
    "tiny": RefConfig(512, 128, 2, 4, 2, 256, 10000.0),
}

BLOCK_KEYS = ("norm1", "wq", "wk", "wv", "wo", "norm2", "wg", "wu", "wd")


class RefModel:
    """bf16 weights in the reference's layout: matrices ``[in, out]``, tied embedding ``[vocab, d]``."""

    def __init__(self, cfg: RefConfig, chain: Chain, seed: int = 1234, std: float = 0.02, masters: bool = True):
        self.cfg, self.ch = cfg, chain
        g = torch.Generator(device="cuda").manual_seed(seed)
        d, kv, ff = cfg.d_model, cfg.n_kv_heads * (cfg.d_model // cfg.n_heads), cfg.d_ff

        def mat(r, c):
            return torch.randn((r, c), generator=g, device="cuda", dtype=torch.float32) * std

        def gain():
            return torch.ones((1, d), device="cuda", dtype=torch.float32)
        self.master = {"embedding": mat(cfg.vocab, d), "final_norm": gain()}
        for i in range(cfg.n_layers):
            self.master[f"b{i}"] = {"norm1": gain(), "wq": mat(d, d), "wk": mat(d, kv), "wv": mat(d, kv),
                                    "wo": mat(d, d), "norm2": gain(), "wg": mat(d, ff), "wu": mat(d, ff),
                                    "wd": mat(ff, d)}
        self.embedding = self.master["embedding"].to(BF)
        self.final_norm = self.master["final_norm"].to(BF)
        self.blocks = [{k: v.to(BF) for k, v in self.master[f"b{i}"].items()} for i in range(cfg.n_layers)]
        if not masters:
            self.master = None

    # -- attention (training form: cuBLAS scores, weights kept for the backward)
    def rope_heads(self, x, n_heads, seq, offset):
        return self.ch.rope_head_local(x, x.shape[1] // n_heads, seq, offset, self.cfg.theta)

    def rope_heads_backward(self, dy, n_heads, seq, offset):
        return self.ch.rope_head_local_backward(dy, dy.shape[1] // n_heads, seq, offset, self.cfg.theta)

    def attention_train_sequence(self, q, k, v):
        ch, cfg = self.ch, self.cfg
        dh = cfg.d_model // cfg.n_heads
        seq = q.shape[0]
        qr = self.rope_heads(q, cfg.n_heads, seq, 0)
        kr = self.rope_heads(k, cfg.n_kv_heads, seq, 0)
        repeat = cfg.n_heads // cfg.n_kv_heads
        scale = 1.0 / math.sqrt(dh)
        heads, weights_all = [], []
        for head in range(cfg.n_heads):
            kvh = head // repeat
            qs = ch.slice_cols(qr, head * dh, dh)
            ks = ch.slice_cols(kr, kvh * dh, dh)
            vs = ch.slice_cols(v, kvh * dh, dh)
            scores = ch.matmul_bt(qs, ks)
            scaled = ch.scale_causal_mask(scores, scale, True)
            weights = ch.softmax(scaled)
            heads.append(ch.matmul(weights, vs))
            weights_all.append(weights)
        return ch.concat_cols(heads), (qr, kr, weights_all)

    def attention_train_batched(self, q, k, v, B, S):
        ch = self.ch
        outs, seqs = [], []
        for b in range(B):
            row = b * S
            out, cache = self.attention_train_sequence(ch.slice_rows(q, row, S), ch.slice_rows(k, row, S),
                                                       ch.slice_rows(v, row, S))
            outs.append(out)
            seqs.append(cache)
        return ch.concat_rows(outs), seqs

    def block_train(self, x, b, B, S):
        ch, eps = self.ch, self.cfg.eps
        xn = ch.rms_norm(x, b["norm1"], eps)
        q, k, v = ch.matmul(xn, b["wq"]), ch.matmul(xn, b["wk"]), ch.matmul(xn, b["wv"])
        ctx, attention = self.attention_train_batched(q, k, v, B, S)
        attn_out = ch.matmul(ctx, b["wo"])
        h = ch.add(x, attn_out)
        hn = ch.rms_norm(h, b["norm2"], eps)
        gate, up = ch.matmul(hn, b["wg"]), ch.matmul(hn, b["wu"])
        act = ch.swiglu(gate, up)
        mlp = ch.matmul(act, b["wd"])
        out = ch.add(h, mlp)
        return out, dict(xn=xn, v=v, attention=attention, ctx=ctx, h=h, hn=hn, gate=gate, up=up, act=act)

    def forward_train(self, tokens_host, B, S):
        ch = self.ch
        xs = [ch.embed(tokens_host, self.embedding)]
        caches = []
        for b in self.blocks:
            out, cache = self.block_train(xs[-1], b, B, S)
            xs.append(out)
            caches.append(cache)
        normed = ch.rms_norm(xs[-1], self.final_norm, self.cfg.eps)
        logits = ch.matmul_bt(normed, self.embedding)
        return logits, dict(xs=xs, blocks=caches, normed=normed)

    def attention_backward_sequence_cached(self, v, dout, cache):
        ch, cfg = self.ch, self.cfg
        qr, kr, weights_all = cache
        dh = cfg.d_model // cfg.n_heads
        seq = qr.shape[0]
        repeat = cfg.n_heads // cfg.n_kv_heads
        scale = 1.0 / math.sqrt(dh)
        dq_heads = []
        dk_kv = [None] * cfg.n_kv_heads
        dv_kv = [None] * cfg.n_kv_heads
        for head in range(cfg.n_heads):
            kvh = head // repeat
            qs = ch.slice_cols(qr, head * dh, dh)
            ks = ch.slice_cols(kr, kvh * dh, dh)
            vs = ch.slice_cols(v, kvh * dh, dh)
            weights = weights_all[head]
            d_ctx = ch.slice_cols(dout, head * dh, dh)
            dweights = ch.matmul_bt(d_ctx, vs)
            dvs = ch.matmul_at(weights, d_ctx)
            dscaled = ch.softmax_backward(weights, dweights)
            dscores = ch.scale_causal_mask_backward(dscaled, scale, True)
            dqs = ch.matmul(dscores, ks)
            dks = ch.matmul_at(dscores, qs)
            dq_heads.append(dqs)
            dk_kv[kvh] = dks if dk_kv[kvh] is None else ch.add(dk_kv[kvh], dks)
            dv_kv[kvh] = dvs if dv_kv[kvh] is None else ch.add(dv_kv[kvh], dvs)
        dqr, dkr, dv = ch.concat_cols(dq_heads), ch.concat_cols(dk_kv), ch.concat_cols(dv_kv)
        return (self.rope_heads_backward(dqr, cfg.n_heads, seq, 0),
                self.rope_heads_backward(dkr, cfg.n_kv_heads, seq, 0), dv)

    def attention_backward_cached(self, v, dout, seqs, B, S):
        ch = self.ch
        dqs, dks, dvs = [], [], []
        for b in range(B):
            row = b * S
            dq, dk, dv = self.attention_backward_sequence_cached(ch.slice_rows(v, row, S),
                                                                 ch.slice_rows(dout, row, S), seqs[b])
            dqs.append(dq)
            dks.append(dk)
            dvs.append(dv)
        return ch.concat_rows(dqs), ch.concat_rows(dks), ch.concat_rows(dvs)

    def block_backward_cached(self, x, b, cache, dout, B, S):
        ch, eps = self.ch, self.cfg.eps
        dact = ch.matmul_bt(dout, b["wd"])
        dwd = ch.matmul_at(cache["act"], dout)
        dgate, dup = ch.swiglu_backward(cache["gate"], cache["up"], dact)
        dwg = ch.matmul_at(cache["hn"], dgate)
        dwu = ch.matmul_at(cache["hn"], dup)
        dhn = ch.add(ch.matmul_bt(dgate, b["wg"]), ch.matmul_bt(dup, b["wu"]))
        dnorm2 = ch.rms_norm_gain_backward(cache["h"], dhn, eps)
        dh = ch.add(dout, ch.rms_norm_backward(cache["h"], b["norm2"], dhn, eps))
        dwo = ch.matmul_at(cache["ctx"], dh)
        d_ctx = ch.matmul_bt(dh, b["wo"])
        dq, dk, dv = self.attention_backward_cached(cache["v"], d_ctx, cache["attention"], B, S)
        dwq = ch.matmul_at(cache["xn"], dq)
        dwk = ch.matmul_at(cache["xn"], dk)
        dwv = ch.matmul_at(cache["xn"], dv)
        dxn = ch.add(ch.add(ch.matmul_bt(dq, b["wq"]), ch.matmul_bt(dk, b["wk"])), ch.matmul_bt(dv, b["wv"]))
        dnorm1 = ch.rms_norm_gain_backward(x, dxn, eps)
        dx = ch.add(dh, ch.rms_norm_backward(x, b["norm1"], dxn, eps))
        return dx, dict(wq=dwq, wk=dwk, wv=dwv, wo=dwo, wg=dwg, wu=dwu, wd=dwd, norm1=dnorm1, norm2=dnorm2)

    def backward_cached(self, tokens_host, dlogits, cache, B, S):
        ch, eps = self.ch, self.cfg.eps
        trunk = cache["xs"][-1]
        d_normed = ch.matmul(dlogits, self.embedding)
        de_head = ch.matmul_at(dlogits, cache["normed"])
        d_final_norm = ch.rms_norm_gain_backward(trunk, d_normed, eps)
        d_cur = ch.rms_norm_backward(trunk, self.final_norm, d_normed, eps)
        block_grads = []
        for i in reversed(range(len(self.blocks))):
            d_cur, grads = self.block_backward_cached(cache["xs"][i], self.blocks[i], cache["blocks"][i], d_cur, B, S)
            block_grads.append(grads)
        block_grads.reverse()
        de_embed = ch.embed_backward(tokens_host, d_cur, self.cfg.vocab)
        return dict(embedding=ch.add(de_head, de_embed), blocks=block_grads, final_norm=d_final_norm)

    # -- cached decoder (deterministic left-to-right score/context kernels)
    def cached_attention_ltr(self, q, k, v):
        ch, cfg = self.ch, self.cfg
        dh = cfg.d_model // cfg.n_heads
        seq = q.shape[0]
        qr = self.rope_heads(q, cfg.n_heads, seq, 0)
        kr = self.rope_heads(k, cfg.n_kv_heads, seq, 0)
        repeat = cfg.n_heads // cfg.n_kv_heads
        scale = 1.0 / math.sqrt(dh)
        heads = []
        for head in range(cfg.n_heads):
            kvh = head // repeat
            qs = ch.slice_cols(qr, head * dh, dh)
            ks = ch.slice_cols(kr, kvh * dh, dh)
            vs = ch.slice_cols(v, kvh * dh, dh)
            scores = ch.attention_scores_ltr(qs, ks)
            scaled = ch.scale_causal_mask(scores, scale, True)
            weights = ch.softmax(scaled)
            heads.append(ch.attention_context(weights, vs))
        return ch.concat_cols(heads)

    def incremental_attention(self, qr, kcache, vcache):
        ch, cfg = self.ch, self.cfg
        dh = cfg.d_model // cfg.n_heads
        repeat = cfg.n_heads // cfg.n_kv_heads
        scale = 1.0 / math.sqrt(dh)
        heads = []
        for head in range(cfg.n_heads):
            kvh = head // repeat
            qs = ch.slice_cols(qr, head * dh, dh)
            ks = ch.slice_cols(kcache, kvh * dh, dh)
            vs = ch.slice_cols(vcache, kvh * dh, dh)
            scores = ch.attention_scores_ltr(qs, ks)
            scaled = ch.scale_causal_mask(scores, scale, False)
            weights = ch.softmax(scaled)
            heads.append(ch.attention_context(weights, vs))
        return ch.concat_cols(heads)

    def _mlp(self, x, attn_ctx, b):
        ch, eps = self.ch, self.cfg.eps
        attn_out = ch.matmul(attn_ctx, b["wo"])
        h = ch.add(x, attn_out)
        hn = ch.rms_norm(h, b["norm2"], eps)
        gate, up = ch.matmul(hn, b["wg"]), ch.matmul(hn, b["wu"])
        act = ch.swiglu(gate, up)
        return ch.add(h, ch.matmul(act, b["wd"]))

    def prefill_cached(self, prompt_host, kcache, vcache):
        ch, cfg = self.ch, self.cfg
        p = prompt_host.numel()
        x = ch.embed(prompt_host, self.embedding)
        for layer, b in enumerate(self.blocks):
            xn = ch.rms_norm(x, b["norm1"], cfg.eps)
            q, k, v = ch.matmul(xn, b["wq"]), ch.matmul(xn, b["wk"]), ch.matmul(xn, b["wv"])
            ctx = self.cached_attention_ltr(q, k, v)
            kcache[layer] = self.rope_heads(k, cfg.n_kv_heads, p, 0)
            vcache[layer] = v
            x = self._mlp(x, ctx, b)
        normed = ch.rms_norm(x, self.final_norm, cfg.eps)
        logits = ch.matmul_bt(normed, self.embedding)
        last = ch.slice_rows(logits, p - 1, 1)
        return last.float().cpu()          # download of the last row (bf16 -> f32 on the host in the reference)

    def decode_step_cached(self, token: int, pos: int, kcache, vcache):
        ch, cfg = self.ch, self.cfg
        x = ch.embed(torch.tensor([token], dtype=torch.int32), self.embedding)
        for layer, b in enumerate(self.blocks):
            xn = ch.rms_norm(x, b["norm1"], cfg.eps)
            q, k, v = ch.matmul(xn, b["wq"]), ch.matmul(xn, b["wk"]), ch.matmul(xn, b["wv"])
            qr = self.rope_heads(q, cfg.n_heads, 1, pos)
            kr = self.rope_heads(k, cfg.n_kv_heads, 1, pos)
            kcache[layer] = kr if kcache[layer] is None else ch.concat_rows([kcache[layer], kr])
            vcache[layer] = v if vcache[layer] is None else ch.concat_rows([vcache[layer], v])
            ctx = self.incremental_attention(qr, kcache[layer], vcache[layer])
            x = self._mlp(x, ctx, b)
        normed = ch.rms_norm(x, self.final_norm, cfg.eps)
        logits = ch.matmul_bt(normed, self.embedding)
        return logits.float().cpu()

    @staticmethod
    def greedy(row) -> int:
        """``sample_row`` at temperature 0: first maximum wins, ``best = row[0]; if v > best``."""
        r = row.reshape(-1)
        if torch.isnan(r[0]):
            return 0
        r = torch.where(torch.isnan(r), torch.full_like(r, float("-inf")), r)
        return int(torch.argmax(r))      # torch.argmax returns the first maximum on CPU tensors

    def generate_cached(self, prompt_host, max_new, on_first=None):
        L = len(self.blocks)
        kcache, vcache = [None] * L, [None] * L
        tokens = prompt_host.tolist()
        logits = self.prefill_cached(prompt_host, kcache, vcache)
        for i in range(max_new):
            nxt = self.greedy(logits)
            if i == 0 and on_first is not None:
                on_first()
            pos = len(tokens)
            tokens.append(nxt)
            if i + 1 == max_new:        # (the reference also stops on token 0; the workload here is a fixed length)
                break
            logits = self.decode_step_cached(nxt, pos, kcache, vcache)
        return tokens


class RefTrainer:
    def __init__(self, model: RefModel, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=1.0):
        self.model = model
        self.lr, self.betas, self.eps, self.wd, self.max_norm = lr, betas, eps, weight_decay, max_grad_norm
        self.step = 0
        z = torch.zeros_like
        ms = model.master
        self.m = {"embedding": z(ms["embedding"]), "final_norm": z(ms["final_norm"])}
        self.v = {"embedding": z(ms["embedding"]), "final_norm": z(ms["final_norm"])}
        for i in range(model.cfg.n_layers):
            self.m[f"b{i}"] = {k: z(t) for k, t in ms[f"b{i}"].items()}
            self.v[f"b{i}"] = {k: z(t) for k, t in ms[f"b{i}"].items()}

    def train_step_batch_deferred(self, tokens_host, targets_host, B, S):
        md, ch = self.model, self.model.ch
        self.step += 1
        logits, cache = md.forward_train(tokens_host, B, S)
        loss_rows, dlogits = ch.cross_entropy_loss_grad_resident(logits, targets_host)
        grads = md.backward_cached(tokens_host, dlogits, cache, B, S)
        refs = [grads["embedding"], grads["final_norm"]]
        for bg in grads["blocks"]:
            refs += [bg[k] for k in BLOCK_KEYS]
        sumsq = ch.global_grad_sumsq(refs)
        ms = md.master
        args = (self.lr, self.betas, self.eps, self.wd, self.step, sumsq, self.max_norm)
        ch.adamw_step_with_norm(ms["embedding"], self.m["embedding"], self.v["embedding"], grads["embedding"],
                                md.embedding, *args)
        ch.adamw_step_with_norm(ms["final_norm"], self.m["final_norm"], self.v["final_norm"], grads["final_norm"],
                                md.final_norm, *args)
        for i, bg in enumerate(grads["blocks"]):
            key = f"b{i}"
            for k in BLOCK_KEYS:
                ch.adamw_step_with_norm(ms[key][k], self.m[key][k], self.v[key][k], bg[k], md.blocks[i][k], *args)
        return loss_rows, sumsq

    @staticmethod
    def finish_step_diagnostics(loss_rows) -> float:
        return float(loss_rows.cpu().double().mean())      # mean_f32: download the rows, mean on the host


# ------------------------------------------------------------------------------------------------
# bench entry point (same JSON line as the framework's own arm)
# ------------------------------------------------------------------------------------------------
def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main(args, ClockSampler=None) -> int:
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device visible; the replay of the reference's CUDA route needs one")
    if not (REF_ROOT / "scirust-cuda" / "src" / "chain.rs").exists():
        return _unavailable("baseline/_ref does not hold the reference's scirust-cuda sources")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.gpus > 1 or world > 1:
        # the reference has no multi-GPU path (scirust/src/lib.rs:133); one rank says so, the others stay silent
        if rank == 0:
            return _unavailable("the reference is single-device (no NCCL/MPI path); it has no number at N > 1")
        return 0
    torch.cuda.set_device(0)
    try:
        chain = Chain()
    except Exception as exc:
        return _unavailable(f"NVRTC/driver set-up of the reference kernels failed: {exc}"[:300])

    out = {"impl": "reference",
           "reference_class": "replay of the reference's NVRTC kernels + cuBLAS bf16 GEMMs in the reference's call "
                              "order (no cargo/rustc on this image)",
           "host_side": "PyTorch caching allocator for alloc_zeros, ctypes launches on libcuda",
           "n_gpus": 1, "dtype": "bf16", "higher_is_better": True,
           "data": "synthetic token ids ~U{0..V-1}, random-init N(0,0.02) weights"}
    mode = getattr(args, "mode", "all")
    if mode in ("all", "train"):
        cfg = PRESETS[args.model]
        B, S = args.batch_per_gpu, args.seq_len
        model = RefModel(cfg, chain, seed=1234)
        trainer = RefTrainer(model)
        g = torch.Generator().manual_seed(1000)
        host = [torch.randint(0, cfg.vocab, (B, S + 1), generator=g, dtype=torch.int64) for _ in range(4)]
        toks = [h[:, :-1].reshape(-1).to(torch.int32).pin_memory() for h in host]
        tgts = [h[:, 1:].reshape(-1).to(torch.int32).pin_memory() for h in host]
        for i in range(args.warmup):
            trainer.train_step_batch_deferred(toks[i % 4], tgts[i % 4], B, S)
        torch.cuda.synchronize()
        sampler = ClockSampler(0) if ClockSampler is not None else None
        if sampler is not None:
            sampler.start()
        l0, g0 = chain.k.launches, chain.gemms
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            loss_rows, _ = trainer.train_step_batch_deferred(toks[i % 4], tgts[i % 4], B, S)
        e1.record()
        torch.cuda.synchronize()
        ms_dev = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
        launches = chain.k.launches - l0 + chain.gemms - g0
        # end to end: the loss is read back every step (finish_step_diagnostics)
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e2.record()
        last = 0.0
        for i in range(args.steps):
            loss_rows, _ = trainer.train_step_batch_deferred(toks[i % 4], tgts[i % 4], B, S)
            last = trainer.finish_step_diagnostics(loss_rows)
        e3.record()
        torch.cuda.synchronize()
        ms_e2e = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3)
        clocks = sampler.stop() if sampler is not None else None
        tokens = B * S * args.steps
        out.update({
            "metric": "GQA decoder train tok/s & decode tok/s, p50 TTFT",
            "value": tokens / (ms_dev / 1e3), "unit": "tokens/s", "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_dev / args.steps, "scaling": "weak", "vs_baseline": None,
            "config": {"model": f"{args.model}: {cfg.n_layers}L d{cfg.d_model} {cfg.n_heads}q/{cfg.n_kv_heads}kv "
                                f"dh{cfg.d_model // cfg.n_heads} ff{cfg.d_ff} V{cfg.vocab} (tied embedding)",
                       "global_batch": B, "seq_len": S, "parallelism": "dp1",
                       "optimizer": "AdamW lr 3e-4 wd 0.1 clip 1.0, fp32 master weights",
                       "l2": "per-step working set exceeds the 126 MB L2; no flush needed"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * B * S * 4 + 3 * B * S * 4, "d2h_bytes_per_step": B * S * 4,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches, "clocks": clocks, "final_loss": last})
        del trainer, model
        torch.cuda.empty_cache()
    if mode in ("all", "infer"):
        try:
            cfg = PRESETS[args.infer_model]
            model = RefModel(cfg, chain, seed=7, masters=False)
            g = torch.Generator().manual_seed(0)
            prompt = torch.randint(0, cfg.vocab, (args.prompt,), generator=g, dtype=torch.int64).to(torch.int32)
            L = cfg.n_layers
            ttft = []
            for i in range(3):
                kc, vc = [None] * L, [None] * L
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                logits = model.prefill_cached(prompt, kc, vc)
                model.greedy(logits)
                ttft.append((time.perf_counter() - t0) * 1e3)
            del kc, vc
            mark = {}
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            toks = model.generate_cached(prompt, args.new, on_first=lambda: mark.setdefault("t", time.perf_counter()))
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            decode_ms = (t1 - mark["t"]) * 1e3
            p50 = statistics.median(ttft[1:])
            row = {"batch": 1, "weights": "bf16", "tp": 1, "ttft_ms_p50": p50,
                   "decode_tok_s": (args.new - 1) / (decode_ms / 1e3), "decode_ms_per_step": decode_ms / (args.new - 1),
                   "e2e_request_tok_s": args.new / (t1 - t0), "first_tokens": toks[args.prompt:args.prompt + 2],
                   "timing": "host clock around synchronising calls (every step downloads its logits row)"}
            out.update({"decode_tok_s": row["decode_tok_s"], "ttft_ms_p50": p50,
                        "inference": {"model": f"{args.infer_model} shape, tied embedding, random-init",
                                      "prompt": args.prompt, "new_tokens": args.new,
                                      "kv_cache": "contiguous bf16, re-allocated every token (concat_rows)",
                                      "parallelism": "tp1", "rows": [row],
                                      "note": "the reference decodes one sequence at a time and has no int8 CUDA "
                                              "path; only the batch-1 bf16 row exists"}})
            if "value" not in out:
                out.update({"metric": "GQA decoder decode tok/s, p50 TTFT", "value": row["decode_tok_s"],
                            "unit": "tokens/s", "vs_baseline": None, "gpu_launches": chain.k.launches + chain.gemms})
        except Exception as exc:
            out["inference"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    print(json.dumps(out))
    return 0

"""Micro-benchmarks of single native kernels (CUDA-event timing, warm-up, L2 flush between
iterations). Also the small fixed workloads that the committed profiler summaries were taken on.

    python -m scirust_b200.ops.bench_kernels gemm --form nt --m 8192 --n 8192 --k 8192
    python -m scirust_b200.ops.bench_kernels attention --batch 8 --seq 2048 --heads 16 --kv-heads 4 --dh 64
    python -m scirust_b200.ops.bench_kernels attention_bwd --batch 1 --seq 2048
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib, attention as att, basic, gemm

BF = torch.bfloat16


def _time(fn, iters: int, warmup: int, flush: bool = True) -> float:
    """Mean milliseconds per call; a 256 MiB buffer is rewritten between calls to evict L2."""
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            scratch.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    _lib.check_status()
    return total / iters


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(BF)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_model", "attention", "attention_bwd", "rmsnorm", "ce", "adamw", "gemv",
                                      "decode_attn", "sampler", "gemm_w8", "conv"])
    ap.add_argument("--int8", action="store_true", help="gemv: per-channel int8 weights")
    ap.add_argument("--ctx", type=int, default=4096, help="decode_attn: cached positions per sequence")
    ap.add_argument("--library", action="store_true", help="gemm_model: also time torch.matmul (cuBLAS)")
    ap.add_argument("--form", default="nt", choices=["nn", "nt", "tn"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--dh", type=int, default=64)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args(argv)
    out = {"kernel": a.kernel}
    flush = not a.no_flush
    if a.kernel == "gemm":
        M, N, K = a.m, a.n, a.k
        if a.form == "nn":
            x, w = _rand((M, K), 1), _rand((K, N), 2)
            fn = lambda: gemm.matmul_nn(x, w)  # noqa: E731
        elif a.form == "nt":
            x, w = _rand((M, K), 1), _rand((N, K), 2)
            fn = lambda: gemm.matmul_nt(x, w)  # noqa: E731
        else:
            x, w = _rand((K, M), 1), _rand((K, N), 2)
            fn = lambda: gemm.matmul_tn(x, w)  # noqa: E731
        ms = _time(fn, a.iters, a.warmup, flush)
        out.update(form=a.form, m=M, n=N, k=K, ms=ms, tflops=2.0 * M * N * K / ms / 1e9)
    elif a.kernel == "gemm_model":
        # every GEMM of one training step of the 12-layer d1024 decoder at 16384 tokens, all three forms
        T = a.rows
        shapes = [("qkv", 1024, 1536), ("wo", 1024, 1024), ("gate_up", 1024, 5632), ("down", 2816, 1024),
                  ("lm_head_chunk", 1024, 32000)]
        rows = []
        for name, K, N in shapes:
            Tm = 4096 if name == "lm_head_chunk" else T
            x, w, dy = _rand((Tm, K), 1), _rand((K, N), 2), _rand((Tm, N), 3)
            wt = w.t().contiguous()
            forms = [("fwd x.W", lambda: gemm.matmul_nn(x, w), lambda: torch.matmul(x, w)),
                     ("dgrad dy.W^T", lambda: gemm.matmul_nt(dy, w), lambda: torch.matmul(dy, w.t())),
                     ("wgrad x^T.dy", lambda: gemm.matmul_tn(x, dy), lambda: torch.matmul(x.t(), dy))]
            if name == "lm_head_chunk":   # tied head: logits = h.E^T, dh = dlogits.E, dE = dlogits^T.h
                forms = [("fwd h.E^T", lambda: gemm.matmul_nt(x, wt), lambda: torch.matmul(x, wt.t())),
                         ("dgrad dl.E", lambda: gemm.matmul_nn(dy, wt), lambda: torch.matmul(dy, wt)),
                         ("wgrad dl^T.h", lambda: gemm.matmul_tn(dy, x), lambda: torch.matmul(dy.t(), x))]
            for fname, ours, lib in forms:
                fl = 2.0 * Tm * K * N
                ms = _time(ours, a.iters, a.warmup, flush)
                row = {"gemm": name, "form": fname, "tokens": Tm, "k": K, "n": N, "ms": round(ms, 4),
                       "tflops": round(fl / ms / 1e9, 1)}
                if a.library:
                    ml = _time(lib, a.iters, a.warmup, flush)
                    row.update(cublas_ms=round(ml, 4), cublas_tflops=round(fl / ml / 1e9, 1))
                rows.append(row)
        out["rows"] = rows
    elif a.kernel == "gemv":
        # batch-1 decode product: W [K, N] streamed once (default 14336 x 4096 bf16 = 117 MB, larger than L2)
        from . import decode
        K, N, M = a.k, a.n, a.batch
        w = _rand((K, N), 11)
        x = _rand((M, K), 12)
        wq = decode.quantize_per_channel(w) if a.int8 else w
        ms = _time(lambda: decode.gemv(x, wq), a.iters, a.warmup, flush)
        nbytes = K * N * (1 if a.int8 else 2)
        out.update(m=M, k=K, n=N, int8=bool(a.int8), ms=ms, gbs=nbytes / ms / 1e6)
    elif a.kernel == "gemm_w8":
        # batched decode product on the dequant-fused tcgen05 GEMM: x [batch, K] bf16, W [K, N] int8 + column scales
        from . import decode
        K, N, M = a.k, a.n, a.batch
        w = _rand((K, N), 11)
        x = _rand((M, K), 12)
        wq = decode.quantize_per_channel(w)
        ms = _time(lambda: decode.matmul_w8(x, wq), a.iters, a.warmup, flush)
        wq.transposed()
        m8 = _time(lambda: decode.matmul_w8a8(x, wq), a.iters, a.warmup, flush)
        xq, sx = decode.quantize_rows(x)
        mq = _time(lambda: decode.quantize_rows(x), a.iters, a.warmup, flush)
        mb = _time(lambda: gemm.matmul_nn(x, w), a.iters, a.warmup, flush)
        if M <= decode.SKINNY_MAX_ROWS:
            out.update(skinny_bf16_ms=_time(lambda: decode.matmul_skinny(x, w), a.iters, a.warmup, flush),
                       skinny_w8a8_ms=_time(lambda: decode.matmul_skinny(x, wq), a.iters, a.warmup, flush))
            out.update(skinny_bf16_gbs=2 * K * N / out["skinny_bf16_ms"] / 1e6, skinny_w8a8_gbs=K * N / out["skinny_w8a8_ms"] / 1e6)
        out.update(m=M, k=K, n=N, w8a16_ms=ms, w8a16_gbs=K * N / ms / 1e6, w8a8_ms=m8, w8a8_gbs=K * N / m8 / 1e6,
                   quantize_rows_ms=mq, bf16_ms=mb, bf16_gbs=2 * K * N / mb / 1e6)
    elif a.kernel == "conv":
        # 3x3 stride-1 convolution, NHWC rows: batch x seq x seq image of `heads` channels -> `cols` channels
        from . import conv
        B, Hs, Cin, Cout = a.batch, a.seq, a.heads, a.cols
        geom = conv.ConvGeom(B, Hs, Hs, Cin)
        x = _rand((geom.rows, Cin), 21)
        wp = conv.pack_conv_weight(_rand((Cout, Cin, 3, 3), 22).float(), Cin, 3).to(torch.bfloat16).cuda()
        ms = _time(lambda: conv.conv2d(x, wp, geom, 3, 1, 1), a.iters, a.warmup, flush)
        fl = 2.0 * geom.rows * Cout * 9 * Cin
        out.update(batch=B, hw=Hs, cin=Cin, cout=Cout, ms=ms, tflops=fl / ms / 1e9)
    elif a.kernel == "sampler":
        # top-k / top-p / temperature sampling of `batch` rows of `cols` fp32 logits (default: a 128256-word vocabulary)
        from ..generate import SamplingParams
        from .sampling import DeviceSampler
        rows, V = a.batch, a.cols if a.cols > 4096 else 128256
        logits = torch.randn((rows, V), device="cuda", generator=torch.Generator(device="cuda").manual_seed(15)) * 3
        sp = DeviceSampler(SamplingParams(temperature=0.8, top_k=50, top_p=0.95), rows, V, list(range(1, rows + 1)), "cuda")
        ms = _time(lambda: sp.sample(logits), a.iters, a.warmup, flush)
        out.update(rows=rows, vocab=V, ms=ms, gbs=rows * V * 4 / ms / 1e6)
    elif a.kernel == "decode_attn":
        from . import decode
        B, H, Hkv, dh, page, L = a.batch, a.heads, a.kv_heads, a.dh, 16, a.ctx
        blocks = (L + page - 1) // page
        pool = _rand((B * blocks, 2, Hkv, page, dh), 13)
        table = torch.randperm(B * blocks, device="cuda").to(torch.int32).reshape(B, blocks)
        lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
        q = _rand((B, H * dh), 14)
        ms = _time(lambda: decode.decode_attention(q, pool, table, page, lens, H, Hkv, dh), a.iters, a.warmup, flush)
        nbytes = B * L * 2 * Hkv * dh * 2
        out.update(batch=B, heads=H, kv_heads=Hkv, dh=dh, ctx=L, ms=ms, gbs=nbytes / ms / 1e6)
    elif a.kernel in ("attention", "attention_bwd"):
        B, S, H, Hkv, dh = a.batch, a.seq, a.heads, a.kv_heads, a.dh
        qkv = _rand((B * S, (H + 2 * Hkv) * dh), 3)
        flops = 4.0 * B * H * S * S * dh / 2
        if a.kernel == "attention":
            ms = _time(lambda: att.attention_fwd(qkv, B, S, H, Hkv, dh), a.iters, a.warmup, flush)
        else:
            o, lse = att.attention_fwd(qkv, B, S, H, Hkv, dh)
            do = _rand((B * S, H * dh), 4)
            ms = _time(lambda: att.attention_bwd(qkv, o, lse, do, B, S, H, Hkv, dh), a.iters, a.warmup, flush)
            flops *= 2.5
        out.update(batch=B, seq=S, heads=H, kv_heads=Hkv, dh=dh, causal=True, ms=ms, tflops=flops / ms / 1e9)
    elif a.kernel == "rmsnorm":
        x, w = _rand((a.rows, a.cols), 5), _rand((a.cols,), 6)
        ms = _time(lambda: basic.rmsnorm_fwd(x, w), a.iters, a.warmup, flush)
        out.update(rows=a.rows, cols=a.cols, ms=ms, gbs=2 * x.numel() * 2 / ms / 1e6)
    elif a.kernel == "ce":
        x = _rand((a.rows, a.cols), 7)
        t = torch.randint(0, a.cols, (a.rows,), device="cuda")
        ms = _time(lambda: basic.ce_fwd_bwd(x, t, 1.0 / a.rows), a.iters, a.warmup, flush)
        out.update(rows=a.rows, cols=a.cols, ms=ms, gbs=3 * x.numel() * 2 / ms / 1e6)
    elif a.kernel == "adamw":
        n = a.rows * a.cols
        p = torch.randn(n, device="cuda")
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        g, pb = _rand((n,), 8), torch.empty(n, dtype=BF, device="cuda")
        ms = _time(lambda: basic.optim_step(p, m, v, g, pb, lr=1e-3, step=1), a.iters, a.warmup, flush)
        out.update(n=n, ms=ms, gbs=n * (12 + 12 + 2 + 2) / ms / 1e6)
    print(json.dumps(out))


if __name__ == "__main__":
    main()

"""Inference engine for the SciAgent / Llama-shaped GQA decoder: batched flash prefill, paged bf16
KV cache, split-KV flash-decode, bf16 or int8 per-output-channel weights, device-side greedy
feedback (no per-token device->host copy) and CUDA-graph replay of the decode step.

Counterparts in the reference: ``CudaModel::prefill_cached`` / ``decode_step_cached`` /
``generate_cached`` (scirust-sciagent/src/cuda_model.rs:450-581), the batch-1 latency decoder with
fused QKV and gate/up, fixed-capacity KV and device feedback (scirust-sciagent/src/cuda_decode.rs:
17-470), ``PagedKvCache`` (scirust-core/src/nn/paged_attention.rs:21-147) and per-channel int8
weights (scirust-core/src/quantization.rs:95-190). Differences by design: prefill is one batched
causal pass (the reference's latency decoder feeds the prompt token by token), the cache is paged
and pre-sized (the reference's general path re-allocates the cache every token), any batch size
decodes in one step, and sampling other than greedy uses the shared ``sample_row`` policy on a
logits row copied to the host.
"""
from __future__ import annotations

import os

import ctypes as C
import math

import torch

from .. import ops
from ..generate import SamplingParams
from ..ops.sampling import DeviceSampler
from ..ops import _lib, attention as att, decode as D
from .sciagent import BF, GQADecoder, SciAgentConfig


class BlockAllocator:
    """Host-side page allocator (native: csrc/rt_alloc.cpp)."""

    def __init__(self, n_blocks: int):
        lib = _lib.rt()
        lib.sbrt_balloc_new.restype = C.c_void_p
        lib.sbrt_balloc_new.argtypes = [C.c_int32]
        lib.sbrt_balloc_delete.argtypes = [C.c_void_p]
        lib.sbrt_balloc_num_free.argtypes = [C.c_void_p]
        lib.sbrt_balloc_num_free.restype = C.c_int32
        lib.sbrt_balloc_alloc.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
        lib.sbrt_balloc_alloc.restype = C.c_int32
        lib.sbrt_balloc_free.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
        lib.sbrt_balloc_free.restype = C.c_int32
        self._lib = lib
        self._h = lib.sbrt_balloc_new(n_blocks)
        if not self._h:
            raise ValueError("n_blocks must be positive")
        self.n_blocks = n_blocks

    def num_free(self) -> int:
        return int(self._lib.sbrt_balloc_num_free(self._h))

    def alloc(self, n: int) -> list:
        buf = (C.c_int32 * max(n, 1))()
        if self._lib.sbrt_balloc_alloc(self._h, n, buf) != 0:
            raise MemoryError(f"KV cache exhausted: {n} pages requested, {self.num_free()} free")
        return list(buf[:n])

    def free(self, ids) -> None:
        ids = list(ids)
        buf = (C.c_int32 * max(len(ids), 1))(*ids)
        if self._lib.sbrt_balloc_free(self._h, buf, len(ids)) != 0:
            raise ValueError("invalid page ids returned to the allocator")

    def __del__(self):
        try:
            if self._h:
                self._lib.sbrt_balloc_delete(self._h)
                self._h = None
        except Exception:
            pass


class PagedKVCache:
    """Pools ``[n_layers][n_blocks, 2, Hkv, page, dh]`` (bf16) + block table + lengths."""

    def __init__(self, n_layers, n_blocks, Hkv, dh, page, max_batch, max_seq, device):
        self.page, self.max_batch = page, max_batch
        self.max_blocks = (max_seq + page - 1) // page
        self.pools = [torch.zeros((n_blocks, 2, Hkv, page, dh), dtype=BF, device=device) for _ in range(n_layers)]
        self.alloc = BlockAllocator(n_blocks)
        self.table_host = torch.zeros((max_batch, self.max_blocks), dtype=torch.int32)
        self.block_table = torch.zeros((max_batch, self.max_blocks), dtype=torch.int32, device=device)
        self.seq_len = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self.owned = [[] for _ in range(max_batch)]

    def reserve(self, seq: int, n_tokens: int) -> None:
        """Make sure sequence ``seq`` owns pages for positions < n_tokens."""
        need = (n_tokens + self.page - 1) // self.page
        if need > self.max_blocks:
            raise ValueError("sequence longer than the cache was sized for")
        have = len(self.owned[seq])
        if need > have:
            new = self.alloc.alloc(need - have)
            self.table_host[seq, have:need] = torch.tensor(new, dtype=torch.int32)
            self.owned[seq] += new

    def commit(self) -> None:
        self.block_table.copy_(self.table_host, non_blocking=True)

    def release(self, seq: int) -> None:
        self.alloc.free(self.owned[seq])
        self.owned[seq] = []
        self.table_host[seq].zero_()


class InferenceEngine:
    def __init__(self, model: GQADecoder, quant: str | None = None, max_batch: int = 1, max_seq: int = 4096,
                 page: int = 64, use_graph: bool = True):
        cfg = model.cfg
        self.cfg, self.quant = cfg, quant
        dev = model.flat.device
        self.dev = dev
        self.max_batch, self.max_seq = max_batch, max_seq
        self.use_graph = use_graph and dev.type == "cuda"

        self.H, self.Hkv = cfg.n_heads, cfg.n_kv_heads      # heads held by this rank
        self._load_weights(model)
        n_blocks = max_batch * ((max_seq + page - 1) // page)
        self.cache = PagedKVCache(cfg.n_layers, n_blocks, self.Hkv, cfg.head_dim, page, max_batch, max_seq, dev)
        self.cos, self.sin = ops.rope_table(max(cfg.max_seq_len, max_seq), cfg.head_dim, cfg.rope_theta, dev)
        self.tokens = torch.zeros(max_batch, dtype=torch.int64, device=dev)     # device feedback buffer
        self.logits = torch.zeros((max_batch, cfg.vocab_size), dtype=torch.float32, device=dev)
        self._graph = None
        self._graph_batch = None
        self._generated = None
        # greedy decoding of up to 8 rows: the LM-head GEMV does its own arg-max (SB_FUSED_ARGMAX=0: three launches)
        self.fused_argmax = os.environ.get("SB_FUSED_ARGMAX", "1") != "0"

    def _prep(self, w):
        w = w.detach()
        return D.quantize_per_channel(w) if self.quant == "int8" else w

    def _load_weights(self, model: GQADecoder):
        prep = self._prep
        self.embed = model.embed.detach()
        self.layers = []
        for l in model.layers:
            self.layers.append({"rms1": l.rms_attn.detach(), "wqkv": prep(l.wqkv), "wo": prep(l.wo),
                                "rms2": l.rms_ffn.detach(), "wgu": prep(l.wgu), "wd": prep(l.wd)})
        self.rms_final = model.rms_final.detach()
        # LM head as [d, V] so the weight-streaming kernels read it row by row
        self.head_t = prep(model.head_weight().detach().t().contiguous())

    # ------------------------------------------------------------------ linear dispatch
    def _proj_out(self, a, w, x, swiglu=False, site="attn"):
        """x + f(a) @ w: the attention-output and MLP-down products (row-parallel under tensor
        parallelism, where a subclass adds the all-reduce). ``swiglu``: a is a fused [gate | up]."""
        if a.shape[0] <= D.gemv_max_rows(w):
            return D.gemv(a, w, residual=x, swiglu=swiglu)
        if swiglu:
            a = ops.swiglu_fwd(a)
        return self._linear(a, w, residual=x)

    def _linear(self, x, w, residual=None):
        M = x.shape[0]
        if M <= D.gemv_max_rows(w):
            return D.gemv(x, w, residual=residual)
        if D.skinny_ok(x, w):
            # 9..64 rows (batched decoding): still bound by the weight bytes; the weight-streaming tcgen05 kernel
            return D.matmul_skinny(x, w, residual=residual)
        if isinstance(w, D.QuantWeight):
            # few rows: the product is bound by the weight bytes, so the int8 matrix is streamed and
            # dequantised inside the GEMM; many rows (prefill): it is bound by the tensor cores, so the
            # layer's weights are expanded to bf16 once (a few percent of the GEMM's time) and the
            # plain bf16 kernel runs at full rate
            if M < 1024 and w.q.shape[1] % 16 == 0:
                return D.matmul_int8(x, w, residual=residual)
            w = w.dequantize()
        return ops.matmul_nn(x, w, residual=residual)

    # ------------------------------------------------------------------ prefill
    def prefill(self, tokens: torch.Tensor):
        """tokens [B, P] (all prompts the same length). Fills the cache, leaves the greedy next
        token of every sequence in ``self.tokens`` and returns the last-position logits [B, V]."""
        cfg, cache = self.cfg, self.cache
        B, P = tokens.shape
        H, Hkv, dh = self.H, self.Hkv, cfg.head_dim
        tok = tokens.to(self.dev)
        for b in range(B):
            if cache.owned[b]:
                cache.release(b)
            cache.reserve(b, min(self.max_seq, P + 1))
        cache.commit()
        seq_of = torch.arange(B, dtype=torch.int32, device=self.dev).repeat_interleave(P)
        pos = torch.arange(P, dtype=torch.int32, device=self.dev).repeat(B)
        x = ops.embed_fwd(self.embed, tok.reshape(-1))
        for li, l in enumerate(self.layers):
            h, _ = ops.rmsnorm_fwd(x, l["rms1"], cfg.eps, want_inv=False)
            qkv = self._linear(h, l["wqkv"])
            ops.rope_(qkv, H + Hkv, dh, P, self.cos, self.sin)
            D.kv_append(qkv, H, Hkv, dh, cache.pools[li], cache.block_table, cache.page, seq_of, pos)
            a, _ = att.attention_fwd(qkv, B, P, H, Hkv, dh, causal=True, want_lse=False)
            x = self._proj_out(a, l["wo"], x, site="attn")
            h, _ = ops.rmsnorm_fwd(x, l["rms2"], cfg.eps, want_inv=False)
            gu = self._linear(h, l["wgu"])
            x = self._proj_out(gu, l["wd"], x, swiglu=True, site="mlp")
        last = x.view(B, P, -1)[:, -1, :].contiguous()
        logits = self.logits[:B]
        self._head(last, logits, rms_weight=self.rms_final)
        D.argmax_rows(logits, out_tokens=self.tokens[:B])
        cache.seq_len[:B] = P
        return logits

    def _head(self, hn, logits, rms_weight=None):
        """logits[M, V] (fp32) = norm(hn) @ head; ``rms_weight`` asks for the final RMSNorm to be
        applied here (fused into the weight-streaming kernel when M <= 8)."""
        self._head_local(hn, logits, rms_weight)

    def _head_local(self, hn, logits, rms_weight=None):
        M = hn.shape[0]
        if M <= D.gemv_max_rows(self.head_t):
            D.gemv(hn, self.head_t, out_f32=logits, rms_weight=rms_weight, eps=self.cfg.eps)
            return
        if rms_weight is not None:
            hn, _ = ops.rmsnorm_fwd(hn, rms_weight, self.cfg.eps, want_inv=False)
        if D.skinny_ok(hn, self.head_t):
            logits.copy_(D.matmul_skinny(hn, self.head_t).float())
            return
        if isinstance(self.head_t, D.QuantWeight):
            logits.copy_(D.matmul_int8(hn, self.head_t).float())
        else:
            logits.copy_(ops.matmul_nn(hn, self.head_t).float())

    # ------------------------------------------------------------------ decode
    def _decode_body(self, B: int, max_len: int, greedy: bool = False):
        cfg, cache = self.cfg, self.cache
        H, Hkv, dh = self.H, self.Hkv, cfg.head_dim
        seq_of = self._seq_of[:B]
        pos = cache.seq_len[:B]
        x = ops.embed_fwd(self.embed, self.tokens[:B])
        # weight-streaming path: norms and SwiGLU are fused into the GEMV loads
        small = B <= D.gemv_max_rows(self.layers[0]["wqkv"])
        for li, l in enumerate(self.layers):
            if small:
                qkv = D.gemv(x, l["wqkv"], rms_weight=l["rms1"], eps=cfg.eps)
            else:
                h, _ = ops.rmsnorm_fwd(x, l["rms1"], cfg.eps, want_inv=False)
                qkv = self._linear(h, l["wqkv"])
            D.rope_kv_append(qkv, H, Hkv, dh, self.cos, self.sin, cache.pools[li], cache.block_table, cache.page,
                             seq_of, pos)
            a = D.decode_attention(qkv, cache.pools[li], cache.block_table, cache.page, self._len_plus1[:B], H, Hkv,
                                   dh, max_len=max_len)
            x = self._proj_out(a, l["wo"], x, site="attn")
            if small:
                gu = D.gemv(x, l["wgu"], rms_weight=l["rms2"], eps=cfg.eps)
            else:
                h, _ = ops.rmsnorm_fwd(x, l["rms2"], cfg.eps, want_inv=False)
                gu = self._linear(h, l["wgu"])
            x = self._proj_out(gu, l["wd"], x, swiglu=True, site="mlp")
        if greedy and self._fused_argmax_ok(B):
            self._head_argmax(x, B)          # LM head and arg-max in one launch; the logits are not written
            return True
        self._head(x, self.logits[:B], rms_weight=self.rms_final)
        return False

    def _fused_argmax_ok(self, B: int) -> bool:
        return (self.dev.type == "cuda" and self.fused_argmax and B <= min(8, D.gemv_max_rows(self.head_t))
                and os.environ.get("SB_GEMV_FMA") != "1")

    def _head_argmax(self, x, B: int, logits=None):
        D.gemv_argmax(x, self.head_t, out_tokens=self.tokens[:B], rms_weight=self.rms_final, eps=self.cfg.eps,
                      logits=logits, generated=self._generated, step=0)

    def _step_eager(self, B, max_len, sampler=None, want_logits=False):
        torch.add(self.cache.seq_len[:B], 1, out=self._len_plus1[:B])
        with D.dependent_launch(self.dev.type == "cuda"):
            done = self._decode_body(B, max_len, greedy=sampler is None and not want_logits)
        if done:
            pass
        elif sampler is None:
            D.argmax_rows(self.logits[:B], out_tokens=self.tokens[:B], generated=self._generated, step=0)
        else:
            sampler.sample(self.logits[:B], out_tokens=self.tokens[:B])
            sampler.push(self.tokens[:B])
        self.cache.seq_len[:B] += 1

    def generate(self, prompts: torch.Tensor, max_new: int, params: SamplingParams | None = None, seed: int = 0,
                 stop_on_zero: bool = False):
        """Greedy or sampled generation; the token never leaves the device between steps (arg-max or
        the device sampler write the feedback buffer) and the step is replayed from a CUDA graph.
        Sequence ``b`` samples from the stream seeded with ``seed + b``. Returns int64 [B, max_new]."""
        params = params or SamplingParams()
        B, P = prompts.shape
        if B > self.max_batch or P + max_new > self.max_seq:
            raise ValueError("request exceeds the engine's max_batch / max_seq")
        greedy = params.temperature <= 0.0 and params.repetition_penalty <= 1.0
        for b in range(B):
            if self.cache.owned[b]:
                self.cache.release(b)
        logits = self.prefill(prompts)
        if self.dev.type == "cuda":
            # benchmarks time the decode steps from here (prefill and its arg-max are behind this event)
            self.prefill_done = torch.cuda.Event(enable_timing=True)
            self.prefill_done.record()
        for b in range(B):
            self.cache.reserve(b, P + max_new)
        self.cache.commit()
        out = torch.zeros((B, max_new), dtype=torch.int64, device=self.dev)
        self._seq_of = torch.arange(self.max_batch, dtype=torch.int32, device=self.dev)
        self._len_plus1 = torch.zeros(self.max_batch, dtype=torch.int32, device=self.dev)
        self._generated = None
        sampler = None
        if not greedy:
            sampler = DeviceSampler(params, B, self.cfg.vocab_size, [seed + b for b in range(B)], self.dev,
                                    history_len=P + max_new)
            sampler.set_history(prompts)
            sampler.sample(logits[:B], out_tokens=self.tokens[:B])
            sampler.push(self.tokens[:B])
        out[:, 0] = self.tokens[:B]
        max_len = P + max_new
        if self.use_graph and max_new > 2:
            # one eager step on the capture stream warms every workspace (they are kept per stream, and nothing may be
            # allocated or cleared inside the capture), then the step is captured once and replayed
            g = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream(device=self.dev)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._step_eager(B, max_len, sampler)
                out[:, 1] = self.tokens[:B]
                with torch.cuda.graph(g, stream=s):
                    self._step_eager(B, max_len, sampler)
            torch.cuda.current_stream().wait_stream(s)
            # capture only records; run the recorded step for positions 2 .. max_new-1
            for i in range(2, max_new):
                g.replay()
                out[:, i] = self.tokens[:B]
        else:
            for i in range(1, max_new):
                self._step_eager(B, max_len, sampler)
                out[:, i] = self.tokens[:B]
        _lib.check_status(self.dev) if self.dev.type == "cuda" else None
        return out


def teacher_forced_logits(engine: "InferenceEngine", prompts: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Logits ``[B, n, V]`` (fp32) of ``engine`` when it is FED ``tokens [B, n]`` after ``prompts`` instead of its own
    arg-max: step i sees the prompt and tokens[:, :i+1]. Two engines given the same tokens can then be compared
    step by step, which greedy generation does not allow once one near-tie flips a token (eager steps, no graph)."""
    B, P = prompts.shape
    n = tokens.shape[1]
    for b in range(B):
        if engine.cache.owned[b]:
            engine.cache.release(b)
    engine.prefill(prompts)
    for b in range(B):
        engine.cache.reserve(b, P + n + 1)
    engine.cache.commit()
    engine._seq_of = torch.arange(engine.max_batch, dtype=torch.int32, device=engine.dev)
    engine._len_plus1 = torch.zeros(engine.max_batch, dtype=torch.int32, device=engine.dev)
    engine._generated = None
    out = []
    tok = tokens.to(engine.dev)
    for i in range(n):
        engine.tokens[:B] = tok[:, i]
        engine._step_eager(B, P + n + 1, want_logits=True)
        out.append(engine.logits[:B].float().clone())
    return torch.stack(out, 1)


def reference_generate(model: GQADecoder, prompts: torch.Tensor, max_new: int) -> torch.Tensor:
    """Full-recompute greedy decoding through the training forward (the naive path the cached
    decoder must agree with token for token: scirust-sciagent/tests/cuda_parity.rs:184)."""
    toks = prompts.clone()
    out = []
    with torch.no_grad():
        for _ in range(max_new):
            logits = model(toks)
            nxt = torch.stack([torch.tensor(D._nan_safe_argmax(r.float().cpu())) for r in logits]).to(toks.device)
            out.append(nxt)
            toks = torch.cat([toks, nxt[:, None]], 1)
    return torch.stack(out, 1)

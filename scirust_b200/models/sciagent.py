"""SciAgent: the GQA / RoPE / RMSNorm / SwiGLU decoder-only language model.

Architecture and checkpoint naming follow the reference model
(scirust-sciagent/src/model.rs:14-236, block.rs:20-70, attention.rs:9-331, swiglu.rs:10-99,
norm.rs:45-75, config.rs:2-80): tied embedding -> N x [RMSNorm -> GQA(RoPE, causal) -> +res ->
RMSNorm -> SwiGLU -> +res] -> RMSNorm -> tied head.

The B200 design differs from the reference's op-chain (scirust-sciagent/src/cuda_model.rs:874-946):

* q/k/v and gate/up projections are single fused GEMMs over ``[in, out]`` weights
  (``wqkv = [wq | wk | wv]``, ``wgu = [gate | up]``); checkpoints still carry the
  reference's separate tensors, split/joined on save/load.
* every parameter lives in one flat bf16 buffer with matching flat fp32 master, gradient and
  Adam-moment buffers, so the optimizer and the data-parallel gradient reduction are each one
  launch per bucket; weight-gradient GEMMs write straight into the flat gradient buffer.
* each decoder block is one autograd node with a hand-scheduled backward that reuses saved
  activations and fuses the residual-stream gradient into the RMSNorm backward.
* the LM head never materialises the whole [T, V] logits matrix: it walks row chunks, and in
  training computes loss and gradient of a chunk in the same pass (as the reference's
  ce_loss_grad does, scirust-cuda/src/chain.rs:637).
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass

import torch
import torch.nn as nn

from .. import ops
from ..ops import attention as att

BF = torch.bfloat16


@dataclass
class SciAgentConfig:
    vocab_size: int = 32768
    d_model: int = 1024
    n_layers: int = 24
    n_heads: int = 16
    n_kv_heads: int = 4
    d_ff: int = 2816
    max_seq_len: int = 8192
    rope_theta: float = 1_000_000.0
    tie_embeddings: bool = True
    use_bias: bool = False
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim

    def to_dict(self) -> dict:
        return asdict(self)

    def validate(self) -> None:
        if self.d_model % self.n_heads or self.n_heads % self.n_kv_heads:
            raise ValueError("d_model must divide by n_heads and n_heads by n_kv_heads")
        if self.head_dim % 8 or self.d_ff % 8 or self.d_model % 8 or self.vocab_size % 8:
            raise ValueError("dimensions must be multiples of 8 (16-byte rows)")

    # presets: scirust-sciagent/src/config.rs:16-80
    @staticmethod
    def sciagent_7b():
        return SciAgentConfig(32768, 4096, 40, 32, 8, 11008, 8192, 1_000_000.0)

    @staticmethod
    def sciagent_350m():
        return SciAgentConfig(32768, 1024, 24, 16, 4, 2816, 8192, 1_000_000.0)

    @staticmethod
    def small():
        return SciAgentConfig(8192, 128, 4, 4, 2, 256, 256, 10000.0)

    @staticmethod
    def debug():
        return SciAgentConfig(256, 64, 2, 4, 2, 128, 128, 10000.0, tie_embeddings=False)

    # pretraining harness presets (scirust-sciagent/examples/cuda_pretrain.rs:64-120)
    @staticmethod
    def byte():
        """Tied, vocabulary 256: raw bytes, no tokenizer."""
        return SciAgentConfig(256, 256, 6, 8, 2, 512, 512, 10000.0)

    @staticmethod
    def demo():
        return SciAgentConfig(512, 256, 6, 8, 2, 512, 256, 10000.0)

    @staticmethod
    def code350m():
        """The 350M trunk on raw bytes (about 270M parameters)."""
        return SciAgentConfig(256, 1024, 24, 16, 4, 2816, 2048, 1_000_000.0)

    # benchmark shapes
    @staticmethod
    def gqa_12l():
        """12-layer training benchmark model: d1024, 16q/4kv, dh64, ff2816, V32000, theta 1e4."""
        return SciAgentConfig(32000, 1024, 12, 16, 4, 2816, 2048, 10000.0)

    @staticmethod
    def llama3_8b():
        return SciAgentConfig(128256, 4096, 32, 32, 8, 14336, 8192, 500000.0, tie_embeddings=False)

    @staticmethod
    def preset(name: str) -> "SciAgentConfig":
        table = {"7b": SciAgentConfig.sciagent_7b, "350m": SciAgentConfig.sciagent_350m,
                 "small": SciAgentConfig.small, "debug": SciAgentConfig.debug,
                 "gqa_12l": SciAgentConfig.gqa_12l, "llama3_8b": SciAgentConfig.llama3_8b, "byte": SciAgentConfig.byte,
                 "demo": SciAgentConfig.demo, "code350m": SciAgentConfig.code350m, "large": SciAgentConfig.code350m,
                 "byte-large": SciAgentConfig.code350m}
        if name not in table:
            raise KeyError(f"unknown model preset {name!r}; known: {sorted(table)}")
        return table[name]()


def _wgrad(param, a, dy):
    """Weight gradient aᵀ·dy. With a flat gradient buffer attached (``param.main_grad``) the GEMM
    writes (or accumulates) there and autograd receives None."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return ops.matmul_tn(a, dy)
    acc = getattr(param, "grad_started", False)
    ops.matmul_tn(a, dy, out=mg, residual=mg if acc else None)
    param.grad_started = True
    return None


def _vgrad(param, compute):
    """Vector (norm gain) gradient; ``compute(out)`` fills/returns it."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        return compute(None)
    if getattr(param, "grad_started", False):
        mg.add_(compute(None).to(mg.dtype))
    else:
        compute(mg)
        param.grad_started = True
    return None


class _BlockFn(torch.autograd.Function):
    """One decoder block, forward and hand-scheduled backward."""

    @staticmethod
    def _run(x, rms1, wqkv, wo, rms2, wgu, wd, blk):
        cfg, B, S = blk.cfg, blk.B, blk.S
        H, Hkv, dh = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        h1, inv1 = ops.rmsnorm_fwd(x, rms1, cfg.eps)
        qkv = ops.matmul_nn(h1, wqkv)
        ops.rope_(qkv, H + Hkv, dh, S, blk.cos, blk.sin)
        a, lse = att.attention_fwd(qkv, B, S, H, Hkv, dh, causal=True)
        x2 = ops.matmul_nn(a, wo, residual=x)
        h2, inv2 = ops.rmsnorm_fwd(x2, rms2, cfg.eps)
        gu, hm = ops.matmul_nn_swiglu(h2, wgu)      # SwiGLU in the GEMM epilogue on CUDA
        return (x, inv1, h1, qkv, a, lse, x2, inv2, h2, gu, hm)

    @staticmethod
    def forward(ctx, x, rms1, wqkv, wo, rms2, wgu, wd, blk):
        saved = _BlockFn._run(x, rms1, wqkv, wo, rms2, wgu, wd, blk)
        x3 = ops.matmul_nn(saved[10], wd, residual=saved[6])
        if blk.recompute:
            # activation recompute: keep only the block input; backward re-runs the forward kernels (fixed
            # reduction orders, so the recomputed activations are the bits of the first pass)
            ctx.save_for_backward(x)
        else:
            ctx.save_for_backward(*saved)
        ctx.blk = blk
        ctx.params = (rms1, wqkv, wo, rms2, wgu, wd)
        return x3

    @staticmethod
    def backward(ctx, dx3):
        rms1, wqkv, wo, rms2, wgu, wd = ctx.params
        blk = ctx.blk
        if blk.recompute:
            with torch.no_grad():
                saved = _BlockFn._run(ctx.saved_tensors[0], rms1, wqkv, wo, rms2, wgu, wd, blk)
        else:
            saved = ctx.saved_tensors
        x, inv1, h1, qkv, a, lse, x2, inv2, h2, gu, hm = saved
        cfg, B, S = blk.cfg, blk.B, blk.S
        H, Hkv, dh = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        dx3 = dx3.contiguous()
        # FFN
        g_wd = _wgrad(wd, hm, dx3)
        dgu = ops.matmul_nt_swiglu_bwd(dx3, wd, gu)     # dhm = dx3 @ wd^T never leaves the GEMM epilogue
        dh2 = ops.matmul_nt(dgu, wgu)
        g_wgu = _wgrad(wgu, h2, dgu)
        res = {}

        def _n2(out):
            dx, dw = ops.rmsnorm_bwd(dh2, x2, rms2, inv2, dres=dx3, dw_out=out)
            res["dx2"] = dx
            return dw
        g_rms2 = _vgrad(rms2, _n2)
        dx2 = res["dx2"]
        # attention
        da = ops.matmul_nt(dx2, wo)
        g_wo = _wgrad(wo, a, dx2)
        if blk.on_attention_bwd is not None:
            blk.on_attention_bwd(blk.index)
        dqkv = att.attention_bwd(qkv, a, lse, da, B, S, H, Hkv, dh, causal=True)
        ops.rope_(dqkv, H + Hkv, dh, S, blk.cos, blk.sin, backward=True)
        dh1 = ops.matmul_nt(dqkv, wqkv)
        g_wqkv = _wgrad(wqkv, h1, dqkv)

        def _n1(out):
            dx, dw = ops.rmsnorm_bwd(dh1, x, rms1, inv1, dres=dx2, dw_out=out)
            res["dx"] = dx
            return dw
        g_rms1 = _vgrad(rms1, _n1)
        if blk.on_grads_ready is not None:
            blk.on_grads_ready(blk.index)
        return res["dx"], g_rms1, g_wqkv, g_wo, g_rms2, g_wgu, g_wd, None


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, tokens):
        ctx.tokens = tokens
        ctx.table = table
        return ops.embed_fwd(table, tokens)

    @staticmethod
    def backward(ctx, dy):
        table = ctx.table
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            ops.embed_bwd(dy.contiguous(), ctx.tokens, mg, accumulate=getattr(table, "grad_started", False))
            table.grad_started = True
            cb = getattr(table, "on_grad_ready", None)
            if cb is not None:
                cb()
            return None, None
        g = torch.zeros_like(table)
        ops.embed_bwd(dy.contiguous(), ctx.tokens, g, accumulate=False)
        return g, None


class _HeadLossFn(torch.autograd.Function):
    """Final RMSNorm + LM head + mean cross-entropy. The gradient of each row chunk is produced
    in the same pass as its loss, so only ``chunk x V`` logits exist at a time. The backward
    seed is assumed to be 1 (a plain ``loss.backward()``)."""

    @staticmethod
    def forward(ctx, x, rmsf, head_w, targets, eps, chunk):
        T = x.shape[0]
        hn, inv = ops.rmsnorm_fwd(x, rmsf, eps)
        need_grad = any(ctx.needs_input_grad[:3])
        loss_rows = torch.empty(T, dtype=torch.float32, device=x.device)
        dhn = torch.empty_like(hn) if need_grad else None
        mg = getattr(head_w, "main_grad", None)
        g_head = None
        if need_grad and mg is None:
            g_head = torch.zeros_like(head_w)
        tgt = targets.reshape(-1)
        for r0 in range(0, T, chunk):
            r1 = min(T, r0 + chunk)
            logits = ops.matmul_nt(hn[r0:r1], head_w)
            if need_grad:
                lr, dl = ops.ce_fwd_bwd(logits, tgt[r0:r1], 1.0 / T)
                loss_rows[r0:r1] = lr
                ops.matmul_nn(dl, head_w, out=dhn[r0:r1])
                dst = mg if mg is not None else g_head
                started = (r0 > 0) or (mg is not None and getattr(head_w, "grad_started", False))
                ops.matmul_tn(dl, hn[r0:r1], out=dst, residual=dst if started else None)
            else:
                loss_rows[r0:r1] = ops.ce_loss_only(logits, tgt[r0:r1])
        if need_grad and mg is not None:
            head_w.grad_started = True
        ctx.save_for_backward(x, inv, dhn if dhn is not None else x)
        ctx.params = (rmsf, head_w)
        ctx.g_head = g_head
        ctx.need_grad = need_grad
        return loss_rows.sum() / T

    @staticmethod
    def backward(ctx, dloss):
        x, inv, dhn = ctx.saved_tensors
        rmsf, head_w = ctx.params
        res = {}

        def _nf(out):
            dx, dw = ops.rmsnorm_bwd(dhn, x, rmsf, inv, dw_out=out)
            res["dx"] = dx
            return dw
        g_rmsf = _vgrad(rmsf, _nf)
        return res["dx"], g_rmsf, ctx.g_head, None, None, None


class _BlockState:
    """Per-call constants shared by the blocks of one forward pass."""

    def __init__(self, cfg, B, S, cos, sin, index, on_grads_ready, on_attention_bwd=None, recompute=False):
        self.cfg, self.B, self.S, self.cos, self.sin = cfg, B, S, cos, sin
        self.index = index
        self.on_grads_ready = on_grads_ready
        self.on_attention_bwd = on_attention_bwd
        self.recompute = recompute


class DecoderLayer(nn.Module):
    def __init__(self, cfg: SciAgentConfig):
        super().__init__()
        d, ff = cfg.d_model, cfg.d_ff
        self.rms_attn = nn.Parameter(torch.empty(d, dtype=BF))
        self.wqkv = nn.Parameter(torch.empty(d, cfg.qkv_dim, dtype=BF))
        self.wo = nn.Parameter(torch.empty(cfg.n_heads * cfg.head_dim, d, dtype=BF))
        self.rms_ffn = nn.Parameter(torch.empty(d, dtype=BF))
        self.wgu = nn.Parameter(torch.empty(d, 2 * ff, dtype=BF))
        self.wd = nn.Parameter(torch.empty(ff, d, dtype=BF))

    def matrices(self):
        return [("wqkv", self.wqkv), ("wo", self.wo), ("wgu", self.wgu), ("wd", self.wd)]

    def gains(self):
        return [("rms_attn", self.rms_attn), ("rms_ffn", self.rms_ffn)]


class GQADecoder(nn.Module):
    """The SciAgent decoder. ``forward(tokens, targets)`` returns the mean next-token loss;
    ``forward(tokens)`` returns logits of the last position of every sequence."""

    def __init__(self, cfg: SciAgentConfig, device="cpu", seed: int = 0, init_std: float = 0.02,
                 head_chunk: int = 16384):
        super().__init__()
        cfg.validate()
        self.cfg = cfg
        self.head_chunk = head_chunk
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=BF))
        self.layers = nn.ModuleList([DecoderLayer(cfg) for _ in range(cfg.n_layers)])
        self.rms_final = nn.Parameter(torch.empty(cfg.d_model, dtype=BF))
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=BF))
        self.on_grads_ready = None  # callback(layer_index) used by data-parallel overlap
        # callback(layer_index) just before a layer's attention backward is launched: the stretch of backward whose
        # kernels are many short CTAs, not persistent GEMMs, so a collective started here takes SMs without stalling
        self.on_attention_bwd = None
        # long contexts: keep one activation (the block input) per layer and re-run the block's forward kernels in
        # backward, 1/15 of the saved bytes for about a third more compute
        self.activation_recompute = False
        self.to(device)
        self._flatten()
        self.reset_parameters(seed, init_std)

    # ------------------------------------------------------------------ flat storage
    def ordered_params(self):
        """(name, parameter, decays) in flat-buffer order: matrices layer by layer (last layer
        first is *not* used; buckets are addressed by name), then the no-decay gains."""
        out = [("embed", self.embed, True)]
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", p, True) for n, p in l.matrices()]
        if self.lm_head is not None:
            out.append(("lm_head", self.lm_head, True))
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", p, False) for n, p in l.gains()]
        out.append(("rms_final", self.rms_final, False))
        return out

    def _flatten(self):
        plist = self.ordered_params()
        # every tensor starts on a 16-byte boundary (8 bf16) so TMA descriptors stay valid
        offs, off = [], 0
        for _, p, _ in plist:
            offs.append(off)
            off += (p.numel() + 7) // 8 * 8
        dev = self.embed.device
        self.flat = torch.zeros(off, dtype=BF, device=dev)
        self.flat_grad = torch.zeros(off, dtype=BF, device=dev)
        self.segments = {}
        self.decay_end = 0
        for (name, p, decays), o in zip(plist, offs):
            n = p.numel()
            p.data = self.flat[o:o + n].view(p.shape)
            p.main_grad = self.flat_grad[o:o + n].view(p.shape)
            p.grad_started = False
            self.segments[name] = (o, n)
            if decays:
                self.decay_end = o + (n + 7) // 8 * 8

    def rebind_grad_buffer(self, new_grad: torch.Tensor) -> None:
        """Re-home the flat gradient buffer (e.g. into peer-mapped symmetric memory)."""
        if new_grad.numel() != self.flat_grad.numel() or new_grad.dtype != self.flat_grad.dtype:
            raise ValueError("gradient buffer must match the flat parameter buffer")
        new_grad.zero_()
        self.flat_grad = new_grad
        for name, p, _ in self.ordered_params():
            o, n = self.segments[name]
            p.main_grad = new_grad[o:o + n].view(p.shape)

    def layer_buckets(self):
        """(start, length) of each decoder layer's matrices inside the flat buffers."""
        out = []
        for i, _ in enumerate(self.layers):
            o0, _ = self.segments[f"layers.{i}.wqkv"]
            o1, n1 = self.segments[f"layers.{i}.wd"]
            out.append((o0, (o1 + n1 + 7) // 8 * 8 - o0))
        return out

    def zero_grad_flags(self):
        for _, p, _ in self.ordered_params():
            p.grad_started = False

    def reset_parameters(self, seed: int = 0, std: float = 0.02):
        dev = self.flat.device
        g = torch.Generator(device=dev).manual_seed(seed)
        with torch.no_grad():
            for name, p, decays in self.ordered_params():
                if decays:
                    p.copy_((torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * std).to(BF))
                else:
                    p.fill_(1.0)

    def num_params(self) -> int:
        return sum(p.numel() for _, p, _ in self.ordered_params())

    # ------------------------------------------------------------------ forward
    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    def hidden(self, tokens):
        B, S = tokens.shape
        cfg = self.cfg
        cos, sin = ops.rope_table(max(cfg.max_seq_len, S), cfg.head_dim, cfg.rope_theta, self.flat.device)
        x = _EmbedFn.apply(self.embed, tokens.reshape(-1))
        for i, l in enumerate(self.layers):
            blk = _BlockState(cfg, B, S, cos, sin, i, self.on_grads_ready, self.on_attention_bwd,
                              self.activation_recompute and torch.is_grad_enabled())
            x = _BlockFn.apply(x, l.rms_attn, l.wqkv, l.wo, l.rms_ffn, l.wgu, l.wd, blk)
        return x

    def forward(self, tokens, targets=None):
        x = self.hidden(tokens)
        if targets is not None:
            return _HeadLossFn.apply(x, self.rms_final, self.head_weight(), targets, self.cfg.eps, self.head_chunk)
        B, S = tokens.shape
        last = x.view(B, S, -1)[:, -1, :].contiguous()
        hn, _ = ops.rmsnorm_fwd(last, self.rms_final, self.cfg.eps, want_inv=False)
        return ops.matmul_nt(hn, self.head_weight())

    def logits_all(self, tokens):
        """Logits for every position [B*S, V] (small inputs / tests)."""
        x = self.hidden(tokens)
        hn, _ = ops.rmsnorm_fwd(x, self.rms_final, self.cfg.eps, want_inv=False)
        return ops.matmul_nt(hn, self.head_weight())

    # ------------------------------------------------------------------ reference checkpoints
    def reference_state_dict(self) -> dict:
        """fp32 tensors under the reference's key names and ``[in, out]`` layout
        (scirust-sciagent/src/attention.rs:312-315, swiglu.rs:58-60, norm.rs:75)."""
        cfg = self.cfg
        qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
        sd = {"sciagent.embed.weight": self.embed.detach().float().cpu()}
        for i, l in enumerate(self.layers):
            p = f"sciagent.layer{i}"
            w = l.wqkv.detach().float().cpu()
            sd[f"{p}.attn.wq.weight"] = w[:, :qd].contiguous()
            sd[f"{p}.attn.wk.weight"] = w[:, qd:qd + kd].contiguous()
            sd[f"{p}.attn.wv.weight"] = w[:, qd + kd:].contiguous()
            sd[f"{p}.attn.wo.weight"] = l.wo.detach().float().cpu()
            gu = l.wgu.detach().float().cpu()
            sd[f"{p}.ffn.gate.weight"] = gu[:, :cfg.d_ff].contiguous()
            sd[f"{p}.ffn.up.weight"] = gu[:, cfg.d_ff:].contiguous()
            sd[f"{p}.ffn.down.weight"] = l.wd.detach().float().cpu()
            sd[f"{p}.rms_attn/weight"] = l.rms_attn.detach().float().cpu().reshape(1, -1)
            sd[f"{p}.rms_ffn/weight"] = l.rms_ffn.detach().float().cpu().reshape(1, -1)
        sd["sciagent.rms_final/weight"] = self.rms_final.detach().float().cpu().reshape(1, -1)
        if self.lm_head is not None:
            # the reference's untied head is a Linear with [in, out] weight and a bias row
            sd["weight"] = self.lm_head.detach().float().cpu().t().contiguous()
            sd["bias"] = torch.zeros(1, cfg.vocab_size)
        return sd

    def load_reference_state_dict(self, sd: dict) -> None:
        cfg = self.cfg

        def get(k):
            if k not in sd:
                raise KeyError(f"missing {k}")
            return torch.as_tensor(sd[k]).float()
        with torch.no_grad():
            self.embed.copy_(get("sciagent.embed.weight").to(BF))
            for i, l in enumerate(self.layers):
                p = f"sciagent.layer{i}"
                l.wqkv.copy_(torch.cat([get(f"{p}.attn.wq.weight"), get(f"{p}.attn.wk.weight"),
                                        get(f"{p}.attn.wv.weight")], 1).to(BF))
                l.wo.copy_(get(f"{p}.attn.wo.weight").to(BF))
                l.wgu.copy_(torch.cat([get(f"{p}.ffn.gate.weight"), get(f"{p}.ffn.up.weight")], 1).to(BF))
                l.wd.copy_(get(f"{p}.ffn.down.weight").to(BF))
                l.rms_attn.copy_(get(f"{p}.rms_attn/weight").reshape(-1).to(BF))
                l.rms_ffn.copy_(get(f"{p}.rms_ffn/weight").reshape(-1).to(BF))
            self.rms_final.copy_(get("sciagent.rms_final/weight").reshape(-1).to(BF))
            if self.lm_head is not None and "weight" in sd:
                self.lm_head.copy_(get("weight").t().to(BF))

"""Tensor-parallel SciAgent decoder (sequence-parallel activations).

Every rank holds ``1/W`` of each block's projection weights (query heads and FFN columns are split;
KV heads are split when ``n_kv_heads >= W`` and otherwise each KV head is replicated on the
``W / n_kv_heads`` ranks whose query heads use it) and a full copy of the embedding and the norm
gains. Between blocks the residual stream is sharded over tokens. The four block boundaries are
the fused all-gather->GEMM / GEMM->reduce-scatter kernels of ``parallel/tensor_parallel.py``; with
``backend="nccl"`` the same model runs on NCCL collectives and library GEMMs (the baseline).

Gradients of replicated parameters (embedding, gains, replicated KV projections) are summed over
the ranks that hold a copy after backward, so all copies stay bitwise identical.
The single-GPU model this shards is ``models/sciagent.py`` (reference architecture:
scirust-sciagent/src/model.rs, block.rs, attention.rs, swiglu.rs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import attention as att
from .sciagent import BF, GQADecoder, SciAgentConfig, _EmbedFn, _HeadLossFn, _vgrad


def _acc_into(param, fn):
    """Run ``fn(out, residual)`` writing the weight gradient into the flat gradient view."""
    mg = param.main_grad
    started = getattr(param, "grad_started", False)
    fn(mg, mg if started else None)
    param.grad_started = True


class _TPBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rms1, wqkv, wo, rms2, wgu, wd, blk):
        cfg, tp, B, S, i = blk.cfg, blk.tp, blk.B, blk.S, blk.index
        Hq, Hkv, dh = blk.hq, blk.hkv, cfg.head_dim
        Tl, d = x.shape
        h1 = tp.buffer(f"h1.{i}", (Tl, d))
        _, inv1 = ops.rmsnorm_fwd(x, rms1, cfg.eps, out=h1)
        qkv = tp.ag_matmul_nn(h1, wqkv, keep=f"h1.{i}")
        ops.rope_(qkv, Hq + Hkv, dh, S, blk.cos, blk.sin)
        a, lse = att.attention_fwd(qkv, B, S, Hq, Hkv, dh, causal=True)
        x2 = tp.matmul_nn_rs(a, wo, residual_shard=x)
        h2 = tp.buffer(f"h2.{i}", (Tl, d))
        _, inv2 = ops.rmsnorm_fwd(x2, rms2, cfg.eps, out=h2)
        gu = tp.ag_matmul_nn(h2, wgu, keep=f"h2.{i}")
        hm = ops.swiglu_fwd(gu)
        x3 = tp.matmul_nn_rs(hm, wd, residual_shard=x2)
        ctx.save_for_backward(x, inv1, h1, qkv, a, lse, x2, inv2, h2, gu, hm)
        ctx.blk = blk
        ctx.params = (rms1, wqkv, wo, rms2, wgu, wd)
        return x3

    @staticmethod
    def backward(ctx, dx3):
        x, inv1, h1, qkv, a, lse, x2, inv2, h2, gu, hm = ctx.saved_tensors
        rms1, wqkv, wo, rms2, wgu, wd = ctx.params
        blk = ctx.blk
        cfg, tp, B, S = blk.cfg, blk.tp, blk.B, blk.S
        Hq, Hkv, dh = blk.hq, blk.hkv, cfg.head_dim
        Tl, d = x.shape
        # the incoming gradient shard must be peer-visible: the next two products gather it
        g3 = tp.buffer("dy.a", (Tl, d))
        g3.copy_(dx3)
        i = blk.index
        dhm = tp.ag_matmul_nt(g3, wd, keep="dy.a")
        # the gathered gradient is already in local memory: the weight gradient needs no second gather
        _acc_into(wd, lambda out, res: tp.matmul_tn_ag(hm, g3, out=out, residual=res, keep="dy.a"))
        dgu = ops.swiglu_bwd(gu, dhm)
        dh2 = tp.matmul_nt_rs(dgu, wgu)
        _acc_into(wgu, lambda out, res: tp.ag_matmul_tn(h2, dgu, out=out, residual=res, keep=f"h2.{i}"))
        res = {}

        def _n2(out):
            dx, dw = ops.rmsnorm_bwd(dh2, x2, rms2, inv2, dres=g3, dw_out=out)
            res["dx2"] = dx
            return dw
        g_rms2 = _vgrad(rms2, _n2)
        g2 = tp.buffer("dy.b", (Tl, d))
        g2.copy_(res["dx2"])
        da = tp.ag_matmul_nt(g2, wo, keep="dy.b")
        _acc_into(wo, lambda out, r: tp.matmul_tn_ag(a, g2, out=out, residual=r, keep="dy.b"))
        dqkv = att.attention_bwd(qkv, a, lse, da, B, S, Hq, Hkv, dh, causal=True)
        ops.rope_(dqkv, Hq + Hkv, dh, S, blk.cos, blk.sin, backward=True)
        dh1 = tp.matmul_nt_rs(dqkv, wqkv)
        _acc_into(wqkv, lambda out, r: tp.ag_matmul_tn(h1, dqkv, out=out, residual=r, keep=f"h1.{i}"))

        def _n1(out):
            dx, dw = ops.rmsnorm_bwd(dh1, x, rms1, inv1, dres=g2, dw_out=out)
            res["dx"] = dx
            return dw
        g_rms1 = _vgrad(rms1, _n1)
        return res["dx"], g_rms1, None, None, g_rms2, None, None, None


class _TPBlockState:
    def __init__(self, cfg, tp, B, S, cos, sin, index, hq, hkv):
        self.cfg, self.tp, self.B, self.S, self.cos, self.sin = cfg, tp, B, S, cos, sin
        self.index, self.hq, self.hkv = index, hq, hkv


class TPDecoderLayer(nn.Module):
    def __init__(self, cfg, hq, hkv, ffr):
        super().__init__()
        d, dh = cfg.d_model, cfg.head_dim
        self.rms_attn = nn.Parameter(torch.empty(d, dtype=BF))
        self.wqkv = nn.Parameter(torch.empty(d, (hq + 2 * hkv) * dh, dtype=BF))
        self.wo = nn.Parameter(torch.empty(hq * dh, d, dtype=BF))
        self.rms_ffn = nn.Parameter(torch.empty(d, dtype=BF))
        self.wgu = nn.Parameter(torch.empty(d, 2 * ffr, dtype=BF))
        self.wd = nn.Parameter(torch.empty(ffr, d, dtype=BF))


class TPDecoder(nn.Module):
    """Rank-local shard of a ``GQADecoder``. Tokens ``[B, S]`` are the *same* on every rank of the
    group; the returned loss is the mean over all ``B*S`` positions (identical on every rank)."""

    def __init__(self, cfg: SciAgentConfig, tp, seed: int = 0, head_chunk: int = 4096):
        super().__init__()
        cfg.validate()
        self.cfg, self.tp = cfg, tp
        W, r = tp.world, tp.rank
        if cfg.n_heads % W or cfg.d_ff % (W * 8):
            raise ValueError("n_heads and d_ff/8 must divide by the tensor-parallel size")
        self.hq = cfg.n_heads // W
        if cfg.n_kv_heads >= W:
            if cfg.n_kv_heads % W:
                raise ValueError("n_kv_heads must divide by the tensor-parallel size")
            self.hkv, self.kv_rep = cfg.n_kv_heads // W, 1
            self.kv0 = r * self.hkv
        else:
            if W % cfg.n_kv_heads:
                raise ValueError("tensor-parallel size must be a multiple of n_kv_heads")
            self.hkv, self.kv_rep = 1, W // cfg.n_kv_heads
            self.kv0 = r // self.kv_rep
        self.ffr = cfg.d_ff // W
        self.head_chunk = head_chunk
        dev = tp.dev
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=BF))
        self.layers = nn.ModuleList([TPDecoderLayer(cfg, self.hq, self.hkv, self.ffr) for _ in range(cfg.n_layers)])
        self.rms_final = nn.Parameter(torch.empty(cfg.d_model, dtype=BF))
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=BF))
        self.on_grads_ready = None
        self.to(dev)
        self._flatten()
        self._kv_group = None
        if self.kv_rep > 1:
            glob = dist.get_process_group_ranks(tp.group)
            whole_job = len(glob) == dist.get_world_size()
            for g in range(cfg.n_kv_heads):
                ranks = list(range(g * self.kv_rep, (g + 1) * self.kv_rep))
                if whole_job:
                    grp = dist.new_group(ranks)
                    if r in ranks:
                        self._kv_group = grp
                elif r in ranks:
                    # the tensor-parallel group is one of several (a mesh axis): only its own members can take part
                    self._kv_group = dist.new_group([glob[i] for i in ranks], use_local_synchronization=True)
        self.load_from_full(GQADecoder(cfg, device=dev, seed=seed))

    # ---------------------------------------------------------------- flat storage
    def ordered_params(self):
        out = []
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", getattr(l, n), True, False) for n in ("wqkv", "wo", "wgu", "wd")]
        # replicated parameters last: decayed matrices first, then gains
        out.append(("embed", self.embed, True, True))
        if self.lm_head is not None:
            out.append(("lm_head", self.lm_head, True, True))
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", getattr(l, n), False, True) for n in ("rms_attn", "rms_ffn")]
        out.append(("rms_final", self.rms_final, False, True))
        return out

    def _flatten(self):
        plist = self.ordered_params()
        offs, off = [], 0
        for _, p, _, _ in plist:
            offs.append(off)
            off += (p.numel() + 7) // 8 * 8
        dev = self.embed.device
        self.flat = torch.zeros(off, dtype=BF, device=dev)
        self.flat_grad = torch.zeros(off, dtype=BF, device=dev)
        self.segments, self.decay_end, self.replicated_start = {}, 0, None
        for (name, p, decays, repl), o in zip(plist, offs):
            n = p.numel()
            p.data = self.flat[o:o + n].view(p.shape)
            p.main_grad = self.flat_grad[o:o + n].view(p.shape)
            p.grad_started = False
            self.segments[name] = (o, n)
            if decays:
                self.decay_end = o + (n + 7) // 8 * 8
            if repl and self.replicated_start is None:
                self.replicated_start = o

    def zero_grad_flags(self):
        for _, p, _, _ in self.ordered_params():
            p.grad_started = False

    def num_params(self):
        return sum(p.numel() for _, p, _, _ in self.ordered_params())

    def load_from_full(self, full: GQADecoder) -> None:
        """Copy this rank's shard out of a full single-GPU model."""
        cfg, r = self.cfg, self.tp.rank
        dh, H, Hkv, ff = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        q0 = r * self.hq
        with torch.no_grad():
            self.embed.copy_(full.embed)
            self.rms_final.copy_(full.rms_final)
            if self.lm_head is not None:
                self.lm_head.copy_(full.lm_head)
            for l, fl in zip(self.layers, full.layers):
                w = fl.wqkv
                q = w[:, q0 * dh:(q0 + self.hq) * dh]
                k = w[:, (H + self.kv0) * dh:(H + self.kv0 + self.hkv) * dh]
                v = w[:, (H + Hkv + self.kv0) * dh:(H + Hkv + self.kv0 + self.hkv) * dh]
                l.wqkv.copy_(torch.cat([q, k, v], 1))
                l.wo.copy_(fl.wo[q0 * dh:(q0 + self.hq) * dh, :])
                g = fl.wgu[:, r * self.ffr:(r + 1) * self.ffr]
                u = fl.wgu[:, ff + r * self.ffr:ff + (r + 1) * self.ffr]
                l.wgu.copy_(torch.cat([g, u], 1))
                l.wd.copy_(fl.wd[r * self.ffr:(r + 1) * self.ffr, :])
                l.rms_attn.copy_(fl.rms_attn)
                l.rms_ffn.copy_(fl.rms_ffn)

    # ---------------------------------------------------------------- forward / loss
    def head_weight(self):
        return self.embed if self.lm_head is None else self.lm_head

    def forward(self, tokens, targets):
        cfg, tp = self.cfg, self.tp
        B, S = tokens.shape
        T = B * S
        W, r = tp.world, tp.rank
        if T % (W * 128):
            raise ValueError("B*S must be a multiple of 128 * tensor-parallel size")
        Tl = T // W
        cos, sin = ops.rope_table(max(cfg.max_seq_len, S), cfg.head_dim, cfg.rope_theta, self.flat.device)
        tok_l = tokens.reshape(-1)[r * Tl:(r + 1) * Tl].contiguous()
        tgt_l = targets.reshape(-1)[r * Tl:(r + 1) * Tl].contiguous()
        x = _EmbedFn.apply(self.embed, tok_l)
        for i, l in enumerate(self.layers):
            blk = _TPBlockState(cfg, tp, B, S, cos, sin, i, self.hq, self.hkv)
            x = _TPBlockFn.apply(x, l.rms_attn, l.wqkv, l.wo, l.rms_ffn, l.wgu, l.wd, blk)
        # local mean over Tl rows; gradients inside are scaled by 1/Tl, fixed up in finish_grads
        return _HeadLossFn.apply(x, self.rms_final, self.head_weight(), tgt_l, cfg.eps, self.head_chunk)

    # ---------------------------------------------------------------- after backward
    def finish_grads(self):
        """Sum the gradients of replicated parameters over the ranks holding a copy and apply the
        1/W that turns per-shard means into the global mean. Returns the gradient scale the
        optimizer still has to apply to every element."""
        tp = self.tp
        W = tp.world
        rs = self.replicated_start
        dist.all_reduce(self.flat_grad[rs:], op=dist.ReduceOp.SUM, group=tp.group)
        if self._kv_group is not None:
            dh, hq, hkv = self.cfg.head_dim, self.hq, self.hkv
            for l in self.layers:
                kvg = l.wqkv.main_grad[:, hq * dh:].contiguous()
                dist.all_reduce(kvg, op=dist.ReduceOp.SUM, group=self._kv_group)
                l.wqkv.main_grad[:, hq * dh:].copy_(kvg)
        return 1.0 / W

    def global_grad_sumsq(self, out: torch.Tensor, grad_scale: float) -> torch.Tensor:
        """Sum of squares of the whole (unsharded) model's gradient: sharded part summed over
        ranks, replicated part counted once (replicated KV copies are divided by their count)."""
        rs = self.replicated_start
        ops.sumsq(self.flat_grad[:rs], out=out)
        if self._kv_group is not None:
            dh, hq = self.cfg.head_dim, self.hq
            extra = torch.zeros(1, dtype=torch.float32, device=out.device)
            for l in self.layers:
                extra += l.wqkv.main_grad[:, hq * dh:].float().pow(2).sum()
            out -= extra * (1.0 - 1.0 / self.kv_rep)
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.tp.group)
        out += ops.sumsq(self.flat_grad[rs:])
        return out


# ------------------------------------------------------------------------------------------------------------------
# Vocabulary-parallel variant: the embedding table and the LM head are sharded over the vocabulary axis as well, so no
# rank holds the whole table, a [tokens, V] logit matrix or a full-vocabulary gradient.
# ------------------------------------------------------------------------------------------------------------------
class _VPEmbedFn(torch.autograd.Function):
    """Sequence-parallel embedding from a vocabulary shard: every rank looks ALL tokens up in its own slice (zero rows
    for ids it does not own) and a reduce-scatter over rows leaves each rank with its token shard: exactly one rank
    contributes a non-zero row, so the bf16 sum is exact. Backward gathers the row shards and scatters into the local
    slice only."""

    @staticmethod
    def forward(ctx, table, tokens, v0, group, world):
        per = table.shape[0]
        loc = tokens.reshape(-1) - v0
        own = (loc >= 0) & (loc < per)
        loc = loc.clamp(0, per - 1)
        full = ops.embed_fwd(table, loc) * own[:, None].to(table.dtype)
        T, d = full.shape
        out = torch.empty((T // world, d), dtype=table.dtype, device=table.device)
        dist.reduce_scatter_tensor(out, full.contiguous(), group=group)
        ctx.table, ctx.loc, ctx.own, ctx.group, ctx.T = table, loc, own, group, T
        return out

    @staticmethod
    def backward(ctx, dy):
        table = ctx.table
        full = torch.empty((ctx.T, dy.shape[1]), dtype=dy.dtype, device=dy.device)
        dist.all_gather_into_tensor(full, dy.contiguous(), group=ctx.group)
        full = full * ctx.own[:, None].to(full.dtype)
        ops.embed_bwd(full, ctx.loc, table.main_grad, accumulate=getattr(table, "grad_started", False))
        table.grad_started = True
        return None, None, None, None, None


class _VPHeadLossFn(torch.autograd.Function):
    """Final RMSNorm (on the token shard) -> all-gather of the normalised rows -> logits of THIS rank's vocabulary
    slice, chunk of rows by chunk -> vocabulary-parallel cross-entropy (three numbers per row exchanged, combined in
    rank order) -> partial d(hidden) = dlogits_local @ head_slice, summed over ranks by a reduce-scatter over rows.
    The head-slice gradient is complete locally (all tokens, own vocabulary rows). Gradients are produced in the forward
    pass, as in the single-device head, scaled by 1 / (tokens per rank) like every other shard of this model."""

    @staticmethod
    def forward(ctx, x, rmsf, head_w, targets, eps, chunk, v0, group, world):
        from ..parallel import vocab_parallel as VP
        Tl, d = x.shape
        T = Tl * world
        hn_l, inv = ops.rmsnorm_fwd(x, rmsf, eps)
        hn = torch.empty((T, d), dtype=hn_l.dtype, device=x.device)
        dist.all_gather_into_tensor(hn, hn_l.contiguous(), group=group)
        tgt = targets.reshape(-1)
        need_grad = any(ctx.needs_input_grad[:3])
        loss_rows = torch.empty(T, dtype=torch.float32, device=x.device)
        dhn = torch.empty_like(hn) if need_grad else None
        mg = head_w.main_grad
        for r0 in range(0, T, chunk):
            r1 = min(T, r0 + chunk)
            logits = ops.matmul_nt(hn[r0:r1], head_w)
            lr, dl = VP.vocab_parallel_ce(logits, tgt[r0:r1], v0, 1.0 / Tl, group=group)
            loss_rows[r0:r1] = lr
            if need_grad:
                ops.matmul_nn(dl, head_w, out=dhn[r0:r1])
                started = (r0 > 0) or getattr(head_w, "grad_started", False)
                ops.matmul_tn(dl, hn[r0:r1], out=mg, residual=mg if started else None)
        dhn_l = None
        if need_grad:
            head_w.grad_started = True
            dhn_l = torch.empty((Tl, d), dtype=dhn.dtype, device=x.device)
            dist.reduce_scatter_tensor(dhn_l, dhn, group=group)
        ctx.save_for_backward(x, inv, dhn_l if dhn_l is not None else x)
        ctx.rmsf = rmsf
        return loss_rows.sum() / T

    @staticmethod
    def backward(ctx, dloss):
        x, inv, dhn_l = ctx.saved_tensors
        rmsf = ctx.rmsf
        res = {}

        def _nf(out):
            dx, dw = ops.rmsnorm_bwd(dhn_l, x, rmsf, inv, dw_out=out)
            res["dx"] = dx
            return dw
        g = _vgrad(rmsf, _nf)
        return res["dx"], g, None, None, None, None, None, None, None


class TPDecoderVocabParallel(TPDecoder):
    """``TPDecoder`` whose embedding table and LM head hold only the vocabulary ids ``[r V / W, (r + 1) V / W)``.
    The replicated segment shrinks to the norm gains; per-rank memory for the table, its two optimizer moments and the
    logits falls by ``W``. The returned loss is the mean over ALL ``B * S`` positions and is identical on every rank."""

    def __init__(self, cfg: SciAgentConfig, tp, seed: int = 0, head_chunk: int = 4096):
        if cfg.vocab_size % (tp.world * 8):
            raise ValueError("vocab_size / 8 must divide by the tensor-parallel size")
        self.vper = cfg.vocab_size // tp.world
        self.v0 = tp.rank * self.vper
        super().__init__(cfg, tp, seed=seed, head_chunk=head_chunk)

    def _vocab_shard(self, full_table):
        return full_table[self.v0:self.v0 + self.vper]

    def ordered_params(self):
        out = []
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", getattr(l, n), True, False) for n in ("wqkv", "wo", "wgu", "wd")]
        out.append(("embed", self.embed, True, False))                 # sharded over the vocabulary: not replicated
        if self.lm_head is not None:
            out.append(("lm_head", self.lm_head, True, False))
        for i, l in enumerate(self.layers):
            out += [(f"layers.{i}.{n}", getattr(l, n), False, True) for n in ("rms_attn", "rms_ffn")]
        out.append(("rms_final", self.rms_final, False, True))
        return out

    def _flatten(self):
        # the parent allocated full tables; keep only this rank's slice before the flat storage is laid out
        dev = self.embed.device
        self.embed = nn.Parameter(torch.empty(self.vper, self.cfg.d_model, dtype=BF, device=dev))
        if self.lm_head is not None:
            self.lm_head = nn.Parameter(torch.empty(self.vper, self.cfg.d_model, dtype=BF, device=dev))
        super()._flatten()

    def load_from_full(self, full: GQADecoder) -> None:
        class _View:                                                   # the parent copies whole tables: hand it slices
            pass
        view = _View()
        view.embed = self._vocab_shard(full.embed)
        view.lm_head = None if full.lm_head is None else self._vocab_shard(full.lm_head)
        view.rms_final, view.layers = full.rms_final, full.layers
        super().load_from_full(view)

    def forward(self, tokens, targets):
        cfg, tp = self.cfg, self.tp
        B, S = tokens.shape
        T = B * S
        W = tp.world
        if T % (W * 128):
            raise ValueError("B*S must be a multiple of 128 * tensor-parallel size")
        cos, sin = ops.rope_table(max(cfg.max_seq_len, S), cfg.head_dim, cfg.rope_theta, self.flat.device)
        x = _VPEmbedFn.apply(self.embed, tokens.reshape(-1).contiguous(), self.v0, tp.group, W)
        for i, l in enumerate(self.layers):
            blk = _TPBlockState(cfg, tp, B, S, cos, sin, i, self.hq, self.hkv)
            x = _TPBlockFn.apply(x, l.rms_attn, l.wqkv, l.wo, l.rms_ffn, l.wgu, l.wd, blk)
        return _VPHeadLossFn.apply(x, self.rms_final, self.head_weight(), targets.reshape(-1).contiguous(), cfg.eps,
                                   self.head_chunk, self.v0, tp.group, W)

"""Tensor-parallel inference engine (TP = 2/4/8 over NVLink): the Llama-shape serving configuration.

Sharding (Megatron style): every rank holds ``H / W`` query heads and ``max(1, Hkv / W)`` KV heads
of the fused QKV matrix, the matching rows of the attention output matrix, ``ff / W`` columns of
gate and up and the matching rows of down, and ``V / W`` columns of the LM head; embedding, norm
gains and the residual stream are replicated. Per layer there are two reductions of the ``[B, d]``
partial products (attention output, MLP down) and one gather of the logits per step.

Decode steps use ``SmallCollectives`` (one peer-memory kernel per reduction, device-resident epoch,
graph-replayable); prefill-sized partials use the bandwidth-oriented ``FusedAllReduce``. With
``backend="nccl"`` everything goes through ``torch.distributed`` instead: the baseline, and the
path that runs on CPU under gloo.

The reference decodes on one device only (scirust-sciagent/src/cuda_model.rs:450-581,
cuda_decode.rs:17-470); this engine keeps its greedy/tie rules and KV-cache semantics per rank.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops import decode as D
from ..parallel.small_collectives import SmallCollectives
from .infer import InferenceEngine
from .sciagent import BF, GQADecoder

SMALL_BYTES = 1 << 20      # partials up to this size (summed over ranks) take the latency path


def _cols(w, parts):
    """Concatenate column ranges [(start, stop), ...] of a [K, N] matrix into a contiguous shard."""
    return torch.cat([w[:, a:b] for a, b in parts], dim=1).contiguous()


class TPInferenceEngine(InferenceEngine):
    def __init__(self, model: GQADecoder, group=None, quant: str | None = None, max_batch: int = 1,
                 max_seq: int = 4096, page: int = 64, use_graph: bool = True, backend: str = "fused"):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        cfg = model.cfg
        W = self.world
        if cfg.n_heads % W or cfg.d_ff % W or cfg.vocab_size % W:
            raise ValueError("tensor parallel size must divide n_heads, d_ff and vocab_size")
        if cfg.n_kv_heads % W and W % cfg.n_kv_heads:
            raise ValueError("tensor parallel size and n_kv_heads must divide one another")
        if (cfg.vocab_size // W) % 8:
            raise ValueError("vocab_size / tensor parallel size must be a multiple of 8")
        dev = model.flat.device
        self.backend = backend if dev.type == "cuda" else "nccl"
        self.region = None
        self.big = None
        self._small_rows = max(8, min(max_batch * max_seq, SMALL_BYTES // (2 * W * cfg.d_model)))
        if self.backend != "fused":
            self._small_rows = max_batch * max_seq
        if self.backend == "fused":
            from ..parallel.fused_allreduce import FusedAllReduce
            from ..parallel.symm import SymmetricRegion
            d = cfg.d_model
            big_rows = max_batch * max_seq
            self._big_elems = big_rows * d if big_rows * d * 2 * W > SMALL_BYTES else 0
            nbytes = (2 * self._big_elems * 2 + 2 * self._small_rows * d * 4
                      + max_batch * (cfg.vocab_size // W) * 4 + 2 * W * 8 * d * 4 + (1 << 17))
            self.region = SymmetricRegion(self.group, nbytes, device=dev)
            if self._big_elems:
                self.big_src = self.region.tensor((self._big_elems,), BF)
                self.big_dst = self.region.tensor((self._big_elems,), BF)
                self.big = FusedAllReduce(self.region, self.big_src, self.big_dst, n_ctas=64)
        self.coll = SmallCollectives(self.group, self.region, backend=self.backend)
        # decode steps of up to 8 rows: the row-parallel GEMV performs its own all-reduce (one launch instead of two);
        # SB_TP_FUSED_GEMV=0 keeps the GEMV + stand-alone collective pair
        self.gemv_chan = None
        if self.backend == "fused" and os.environ.get("SB_TP_FUSED_GEMV", "1") != "0":
            from ..parallel.small_collectives import GemvAllReduceChannel
            self.gemv_chan = GemvAllReduceChannel(self.region, rows=8, n_max=cfg.d_model)
        self.amax_chan = None
        if self.backend == "fused" and self.region is not None and W > 1:
            from ..parallel.small_collectives import ArgmaxChannel
            self.amax_chan = ArgmaxChannel(self.region)
        super().__init__(model, quant=quant, max_batch=max_batch, max_seq=max_seq, page=page,
                         use_graph=use_graph and self.backend == "fused")
        self.vocab_local = cfg.vocab_size // W
        self.logits_local = self.coll.source("logits", (max_batch, self.vocab_local), torch.float32, device=dev)

    # ------------------------------------------------------------------ weights
    def _load_weights(self, model: GQADecoder):
        cfg, W, r = self.cfg, self.world, self.rank
        dh, H, Hkv, ff = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        hq = H // W
        hkv = max(1, Hkv // W)
        kv0 = (r * Hkv) // W              # first KV head of this rank (replicated when Hkv < W)
        self.H, self.Hkv = hq, hkv
        q_cols = (r * hq * dh, (r + 1) * hq * dh)
        k_cols = (H * dh + kv0 * dh, H * dh + (kv0 + hkv) * dh)
        v_cols = ((H + Hkv) * dh + kv0 * dh, (H + Hkv) * dh + (kv0 + hkv) * dh)
        fl = ff // W
        prep = self._prep
        # copies, so that the caller may drop the full model (its flat parameter buffer) afterwards
        self.embed = model.embed.detach().clone()
        self.layers = []
        for l in model.layers:
            wqkv = _cols(l.wqkv.detach(), [q_cols, k_cols, v_cols])
            wo = l.wo.detach()[r * hq * dh:(r + 1) * hq * dh].contiguous()
            wgu = _cols(l.wgu.detach(), [(r * fl, (r + 1) * fl), (ff + r * fl, ff + (r + 1) * fl)])
            wd = l.wd.detach()[r * fl:(r + 1) * fl].contiguous()
            self.layers.append({"rms1": l.rms_attn.detach().clone(), "wqkv": prep(wqkv), "wo": prep(wo),
                                "rms2": l.rms_ffn.detach().clone(), "wgu": prep(wgu), "wd": prep(wd)})
        self.rms_final = model.rms_final.detach().clone()
        vl = cfg.vocab_size // W
        self.head_t = prep(model.head_weight().detach()[r * vl:(r + 1) * vl].t().contiguous())

    # ------------------------------------------------------------------ row-parallel products
    def _proj_out(self, a, w, x, swiglu=False, site="attn"):
        M, d = x.shape
        coll = self.coll
        if self.backend != "fused" or M * d * 2 * self.world <= SMALL_BYTES:
            if self.gemv_chan is not None and M <= D.gemv_max_rows(w) and os.environ.get("SB_GEMV_FMA") != "1":
                return D.gemv_allreduce(a, w, self.gemv_chan, residual=x, swiglu=swiglu)
            full = coll.source(site, (self._small_rows, d), torch.float32, device=x.device)
            if M <= D.gemv_max_rows(w):
                src = full[:M]
                D.gemv(a, w, out_f32=src, swiglu=swiglu)
            else:
                src = full.view(-1).view(BF)[:M * d].view(M, d)     # same base address, bf16 partial
                if swiglu:
                    a = ops.swiglu_fwd(a)
                self._linear_into(a, w, src)
            return coll.all_reduce(src, residual=x)
        # prefill-sized partial: bandwidth-oriented all-reduce, then the residual add
        if swiglu:
            a = ops.swiglu_fwd(a)
        n = M * d
        src = self.big_src[:n].view(M, d)
        self._linear_into(a, w, src)
        epoch = self.big.next_epoch()
        self.big.reduce(0, n, 1.0, epoch)
        return ops.add(x, self.big_dst[:n].view(M, d))

    def _linear_into(self, a, w, out):
        if not a.is_cuda:
            out.copy_(self._linear(a, w))
            return out
        if D.skinny_ok(a, w):
            return D.matmul_skinny(a, w, out=out)
        if isinstance(w, D.QuantWeight):
            if a.shape[0] < 1024 and w.q.shape[1] % 16 == 0:
                return D.matmul_int8(a, w, out=out)
            w = w.dequantize()
        return ops.matmul_nn(a, w, out=out)

    # ------------------------------------------------------------------ vocabulary-parallel head
    def _head(self, hn, logits, rms_weight=None):
        M = hn.shape[0]
        local = self.logits_local[:M]
        self._head_local(hn, local, rms_weight)
        self.coll.gather_rows(local, logits)

    def _fused_argmax_ok(self, B: int) -> bool:
        return self.amax_chan is not None and super()._fused_argmax_ok(B)

    def _head_argmax(self, x, B: int, logits=None):
        D.gemv_argmax(x, self.head_t, out_tokens=self.tokens[:B], rms_weight=self.rms_final, eps=self.cfg.eps,
                      logits=logits, chan=self.amax_chan, col_offset=self.rank * self.vocab_local,
                      generated=self._generated, step=0)

    def close(self):
        """Collective: unmaps the peers' symmetric memory."""
        if self.region is not None:
            self.region.close()
            self.region = None

"""Pipeline parallelism for the GQA decoder: contiguous groups of layers on consecutive ranks, micro-batches in a
one-forward-one-backward (1F1B) schedule, activations and their gradients exchanged with point-to-point
``torch.distributed`` transfers (NCCL between GPUs, gloo between CPU ranks).

Stage ``s`` of ``P`` owns layers ``[lo, hi)``; stage 0 also owns the embedding, stage ``P - 1`` the final norm, the
LM head and the loss. Every stage keeps its parameters, gradients and optimizer state in the same flat buffers as
the single-device model (``models/sciagent.py``), so ``train.Trainer`` drives a ``PipelineModel`` unchanged: one call
of the model runs the whole schedule (forward and backward of every micro-batch), ``loss.backward()`` is then a
no-op, and the gradient norm is the sum over the stages.

Semantics kept from the reference's data-parallel trainer (scirust-core/src/distributed.rs:96-167): the loss is the
mean over the micro-batches, gradients accumulate in micro-batch order, so a run equals the single-process run that
accumulates the same micro-batches, bit for bit while gradient clipping is inactive (asserted on CPU ranks; the
squared gradient norm is added stage by stage, so an active clip factor may differ in its last bit). With tied embeddings the first and last
stage both hold the table; their gradients are summed between the two before the optimizer, and counted once in
the gradient norm.

Sends are asynchronous and receives blocking, which is what makes the schedule free of send/send deadlocks on both
backends; on CUDA every transfer is issued on the stage's current stream (NCCL orders them with the kernels).
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist

from .. import ops
from ..models.sciagent import BF, GQADecoder, SciAgentConfig, _BlockFn, _BlockState, _EmbedFn, _HeadLossFn


def split_layers(n_layers: int, stages: int) -> list[tuple[int, int]]:
    """Contiguous ``[lo, hi)`` per stage; the first ``n_layers % stages`` stages take one layer more."""
    if stages < 1 or n_layers < stages:
        raise ValueError("need at least one layer per pipeline stage")
    base, extra = divmod(n_layers, stages)
    out, lo = [], 0
    for s in range(stages):
        hi = lo + base + (1 if s < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


class PipelineModel:
    """One pipeline stage behind the interface ``train.Trainer`` expects from a model."""

    def __init__(self, cfg: SciAgentConfig, group=None, device=None, micro_batches: int = 4, seed: int = 0):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.cfg_full = cfg
        self.lo, self.hi = split_layers(cfg.n_layers, self.world)[self.rank]
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.micro_batches = micro_batches
        local = dataclasses.replace(cfg, n_layers=self.hi - self.lo)
        self.stage = GQADecoder(local, device=device, seed=seed + 1000 * self.rank)
        self.device = self.stage.flat.device
        self.flat, self.flat_grad, self.decay_end = self.stage.flat, self.stage.flat_grad, self.stage.decay_end
        self.tied = cfg.tie_embeddings and self.world > 1
        # created by every rank (a collective), used by the two end stages only
        self.tie_group = dist.new_group([self._global(0), self._global(self.world - 1)]) if self.tied else None
        self._sends = []
        self.last_losses = None

    def _global(self, r):
        return dist.get_global_rank(self.group, r) if self.group is not dist.group.WORLD else r

    # ------------------------------------------------------------------ weights
    def load_from_full(self, full: GQADecoder) -> None:
        """Copy this stage's parameters out of a complete model (tests, conversion of a single-device checkpoint)."""
        with torch.no_grad():
            for i in range(self.lo, self.hi):
                src, dst = full.layers[i], self.stage.layers[i - self.lo]
                for name in ("rms_attn", "wqkv", "wo", "rms_ffn", "wgu", "wd"):
                    getattr(dst, name).copy_(getattr(src, name))
            self.stage.embed.copy_(full.embed)
            self.stage.rms_final.copy_(full.rms_final)
            if full.lm_head is not None:
                self.stage.lm_head.copy_(full.lm_head)

    def zero_grad_flags(self):
        self.stage.zero_grad_flags()

    def parameters(self):
        return self.stage.parameters()

    # ------------------------------------------------------------------ transfers
    def _send(self, t, dst):
        self._sends.append((dist.isend(t.contiguous(), self._global(dst), group=self.group), t))

    def _recv(self, shape, src, dtype=BF):
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, self._global(src), group=self.group)
        return t

    def _drain(self):
        for w, _ in self._sends:
            w.wait()
        self._sends = []

    # ------------------------------------------------------------------ one micro-batch
    def _forward(self, inp, tgt, scale):
        st, cfg = self.stage, self.stage.cfg
        B, S = inp.shape
        cos, sin = ops.rope_table(max(cfg.max_seq_len, S), cfg.head_dim, cfg.rope_theta, self.device)
        if self.first:
            x_in = None
            x = _EmbedFn.apply(st.embed, inp.reshape(-1))
        else:
            x_in = self._recv((B * S, cfg.d_model), self.rank - 1).requires_grad_()
            x = x_in
        for i, l in enumerate(st.layers):
            blk = _BlockState(cfg, B, S, cos, sin, i, None, None, st.activation_recompute)
            x = _BlockFn.apply(x, l.rms_attn, l.wqkv, l.wo, l.rms_ffn, l.wgu, l.wd, blk)
        if self.last:
            loss = _HeadLossFn.apply(x, st.rms_final, st.head_weight(), tgt, cfg.eps, st.head_chunk)
            return x_in, loss * scale, loss.detach()
        self._send(x.detach(), self.rank + 1)
        return x_in, x, None

    def _backward(self, x_in, out):
        if self.last:
            out.backward()
        else:
            out.backward(self._recv(tuple(out.shape), self.rank + 1))
        if not self.first:
            self._send(x_in.grad, self.rank - 1)

    # ------------------------------------------------------------------ the schedule
    def __call__(self, inp, tgt):
        M = self.micro_batches
        B = inp.shape[0]
        if B % M:
            raise ValueError("batch size must be a multiple of the number of micro-batches")
        mb = B // M
        warm = min(self.world - self.rank - 1, M)
        live, losses = [], []
        nf = nb = 0

        def fwd():
            nonlocal nf
            sl = slice(nf * mb, (nf + 1) * mb)
            x_in, out, lv = self._forward(inp[sl], tgt[sl] if self.last else None, 1.0 / M)
            live.append((x_in, out))
            if lv is not None:
                losses.append(lv)
            nf += 1

        def bwd():
            nonlocal nb
            self._backward(*live.pop(0))
            nb += 1
        for _ in range(warm):
            fwd()
        for _ in range(M - warm):
            fwd()
            bwd()
        for _ in range(warm):
            bwd()
        self._drain()
        if self.tied and (self.first or self.last):
            g = self.stage.embed.main_grad if hasattr(self.stage.embed, "main_grad") else self.stage.embed.grad
            dist.all_reduce(g, group=self.tie_group)
        # the mean loss is known on the last stage; every stage reports it
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.last:
            total += torch.stack(losses).float().sum() / M
        dist.broadcast(total, self._global(self.world - 1), group=self.group)
        self.last_losses = losses
        return total[0].detach().requires_grad_()      # Trainer calls .backward() on it: nothing is left to do

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, directory, step: int, loss: float, lr: float, trainer=None):
        """Every stage writes ``directory/step_N/stage_K`` (its layers, under their LOCAL indices, with the optimizer
        state and fp32 masters when a trainer is given; atomic per stage); rank 0 writes ``pipeline.json`` with the
        layer split once all stages are done, which is what marks the checkpoint complete."""
        import json
        from pathlib import Path
        from ..io.checkpoint import save_sciagent_checkpoint
        root = Path(directory) / f"step_{int(step)}"
        root.mkdir(parents=True, exist_ok=True)
        save_sciagent_checkpoint(self.stage, root / f"stage_{self.rank}", step, loss, lr, trainer=trainer,
                                 extra_opt={"pipeline_stage": self.rank, "layers": [self.lo, self.hi]})
        dist.barrier(group=self.group)
        if self.rank == 0:
            info = {"stages": self.world, "n_layers": self.cfg_full.n_layers, "micro_batches": self.micro_batches,
                    "split": split_layers(self.cfg_full.n_layers, self.world), "step": int(step)}
            (root / "pipeline.json").write_text(json.dumps(info, indent=2, sort_keys=True))
        dist.barrier(group=self.group)
        return root

    def load_checkpoint(self, root, trainer=None) -> dict:
        """Resume this stage from ``root`` (a ``step_N`` directory written by the same layer split)."""
        import json
        from pathlib import Path
        from ..io.checkpoint import load_optimizer_state, load_sciagent_checkpoint
        root = Path(root)
        info = json.loads((root / "pipeline.json").read_text())
        if info["stages"] != self.world or info["n_layers"] != self.cfg_full.n_layers:
            raise ValueError(f"checkpoint was written by {info['stages']} stages over {info['n_layers']} layers")
        _, meta = load_sciagent_checkpoint(root / f"stage_{self.rank}", model=self.stage)
        if trainer is not None:
            load_optimizer_state(self.stage, trainer, root / f"stage_{self.rank}")
        return meta

    @staticmethod
    def latest(directory):
        """Newest ``step_N`` directory that holds a complete pipeline checkpoint, or None."""
        from pathlib import Path
        d = Path(directory)
        if not d.exists():
            return None
        done = [p for p in d.iterdir() if p.name.startswith("step_") and p.name[5:].isdigit() and (p / "pipeline.json").exists()]
        return max(done, key=lambda p: int(p.name[5:])) if done else None

    # ------------------------------------------------------------------ hooks used by Trainer
    def global_grad_sumsq(self, out: torch.Tensor, scale: float = 1.0) -> None:
        ops.sumsq(self.flat_grad, out=out)
        if self.tied and self.last:
            # the tied table's gradient is also held (and counted) by stage 0
            g = self.stage.embed.main_grad
            out -= g.float().pow(2).sum()
        dist.all_reduce(out, group=self.group)     # the optimizer applies `scale` to the gradient and its norm


# ----------------------------------------------------------------------------------------------------------------------
# Interleaved (virtual-stage) schedule
# ----------------------------------------------------------------------------------------------------------------------
def interleaved_schedule(stages: int, virtual: int, micro_batches: int, rank: int) -> list[tuple[str, int, int]]:
    """Order of work on one rank as ``(kind, chunk, micro_batch)`` with kind ``"F"`` or ``"B"``.

    Every rank owns ``virtual`` chunks of layers; chunk ``v`` of rank ``r`` is global stage ``v * stages + r``, so a
    micro-batch crosses every rank ``virtual`` times and the pipeline bubble shrinks by that factor. Forward step ``k``
    works on chunk ``(k mod (stages * virtual)) // stages`` and micro-batch ``(k // (stages * virtual)) * stages + k mod
    stages``; backward steps walk the chunks in the opposite order. A rank runs ``2 (stages - rank - 1) + (virtual - 1)
    stages`` forward steps ahead, then alternates one forward with one backward, then drains. For each chunk the
    micro-batches appear in increasing order in both directions, so gradients accumulate in the order of the
    single-process run."""
    P, V, M = stages, virtual, micro_batches
    if M % P:
        raise ValueError("the interleaved schedule needs a number of micro-batches that is a multiple of the stages")
    if not 0 <= rank < P or V < 1:
        raise ValueError("bad rank or virtual-stage count")
    total = M * V

    def item(k, forward):
        in_group = k % (P * V)
        chunk = in_group // P
        return ("F" if forward else "B", chunk if forward else V - 1 - chunk, (k // (P * V)) * P + in_group % P)
    warm = min(total, 2 * (P - rank - 1) + (V - 1) * P)
    out = [item(k, True) for k in range(warm)]
    for i in range(total - warm):
        out.append(item(warm + i, True))
        out.append(item(i, False))
    out += [item(k, False) for k in range(total - warm, total)]
    return out


def check_schedule(stages: int, virtual: int, micro_batches: int) -> int:
    """Replay the schedules of all ranks with asynchronous sends, blocking receives and first-in-first-out matching
    per (sender, receiver, direction): raises on a deadlock or on a message that would be received out of order;
    returns the number of scheduling rounds (a rank advances at most one item per round), a proxy for the makespan."""
    P, V = stages, virtual
    plans = [interleaved_schedule(P, V, micro_batches, r) for r in range(P)]
    pos = [0] * P
    queues: dict = {}
    rounds = 0
    while any(pos[r] < len(plans[r]) for r in range(P)):
        progressed = False
        sends = []
        for r in range(P):
            if pos[r] >= len(plans[r]):
                continue
            kind, v, m = plans[r][pos[r]]
            g = v * P + r
            first, last = g == 0, g == P * V - 1
            if kind == "F" and not first:
                q = queues.get(((r - 1) % P, r, "F"), [])
                want = (v if r > 0 else v - 1, m)
                if not q:
                    continue
                if q[0] != want:
                    raise AssertionError(f"rank {r} expects activation {want}, the channel delivers {q[0]} first")
                q.pop(0)
            if kind == "B" and not last:
                q = queues.get(((r + 1) % P, r, "B"), [])
                want = (v if r < P - 1 else v + 1, m)
                if not q:
                    continue
                if q[0] != want:
                    raise AssertionError(f"rank {r} expects gradient {want}, the channel delivers {q[0]} first")
                q.pop(0)
            if kind == "F" and not last:
                sends.append(((r, (r + 1) % P, "F"), (v, m)))
            if kind == "B" and not first:
                sends.append(((r, (r - 1) % P, "B"), (v, m)))
            pos[r] += 1
            progressed = True
        for key, msg in sends:                                               # visible from the next round on
            queues.setdefault(key, []).append(msg)
        rounds += 1
        if not progressed:
            raise AssertionError(f"deadlock at positions {pos}")
    return rounds


class InterleavedPipelineModel(PipelineModel):
    """``PipelineModel`` with ``virtual_stages`` chunks of layers per rank (global stage ``v * P + rank``), run in the
    interleaved one-forward-one-backward order of ``interleaved_schedule``. The chunks of a rank sit one after the other
    in ONE flat parameter / gradient buffer, so the trainer and the optimizer see a single stage. Activations and
    gradients travel in two separate process groups (one per direction): each keeps its own per-pair ordering, which
    the schedule respects (``check_schedule``), also when ``P = 2`` makes the next and the previous rank the same."""

    def __init__(self, cfg: SciAgentConfig, group=None, device=None, micro_batches: int = 4, virtual_stages: int = 2, seed: int = 0):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.virtual = virtual_stages
        self.cfg_full = cfg
        self.micro_batches = micro_batches
        self.split = split_layers(cfg.n_layers, self.world * virtual_stages)
        self.chunks, off = [], 0
        for v in range(virtual_stages):
            lo, hi = self.split[v * self.world + self.rank]
            self.chunks.append((lo, hi, off))                                 # global [lo, hi) sits at local offset off
            off += hi - lo
        self.lo, self.hi = self.chunks[0][0], self.chunks[-1][1]
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.stage = GQADecoder(dataclasses.replace(cfg, n_layers=off), device=device, seed=seed + 1000 * self.rank)
        self.device = self.stage.flat.device
        self.flat, self.flat_grad, self.decay_end = self.stage.flat, self.stage.flat_grad, self.stage.decay_end
        self.tied = cfg.tie_embeddings and self.world > 1
        self.tie_group = dist.new_group([self._global(0), self._global(self.world - 1)]) if self.tied else None
        members = [self._global(r) for r in range(self.world)]
        self.fwd_group, self.bwd_group = dist.new_group(members), dist.new_group(members)
        self._sends = []
        self.last_losses = None
        interleaved_schedule(self.world, virtual_stages, micro_batches, self.rank)      # validates M against P early

    def load_from_full(self, full: GQADecoder) -> None:
        with torch.no_grad():
            for lo, hi, off in self.chunks:
                for i in range(lo, hi):
                    src, dst = full.layers[i], self.stage.layers[off + i - lo]
                    for name in ("rms_attn", "wqkv", "wo", "rms_ffn", "wgu", "wd"):
                        getattr(dst, name).copy_(getattr(src, name))
            self.stage.embed.copy_(full.embed)
            self.stage.rms_final.copy_(full.rms_final)
            if full.lm_head is not None:
                self.stage.lm_head.copy_(full.lm_head)

    def local_layer(self, global_index: int):
        for lo, hi, off in self.chunks:
            if lo <= global_index < hi:
                return self.stage.layers[off + global_index - lo]
        raise IndexError(f"layer {global_index} is not on this rank")

    def _isend(self, t, dst, group):
        self._sends.append((dist.isend(t.contiguous(), self._global(dst), group=group), t))

    def _recv_from(self, shape, src, group, dtype=BF):
        t = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(t, self._global(src), group=group)
        return t

    def _forward_chunk(self, v, inp, tgt, scale):
        st, cfg = self.stage, self.stage.cfg
        B, S = inp.shape
        P = self.world
        g_first, g_last = self.first and v == 0, self.last and v == self.virtual - 1
        cos, sin = ops.rope_table(max(cfg.max_seq_len, S), cfg.head_dim, cfg.rope_theta, self.device)
        if g_first:
            x_in = None
            x = _EmbedFn.apply(st.embed, inp.reshape(-1))
        else:
            x_in = self._recv_from((B * S, cfg.d_model), (self.rank - 1) % P, self.fwd_group).requires_grad_()
            x = x_in
        lo, hi, off = self.chunks[v]
        for i in range(off, off + hi - lo):
            l = st.layers[i]
            blk = _BlockState(cfg, B, S, cos, sin, i, None, None, st.activation_recompute)
            x = _BlockFn.apply(x, l.rms_attn, l.wqkv, l.wo, l.rms_ffn, l.wgu, l.wd, blk)
        if g_last:
            loss = _HeadLossFn.apply(x, st.rms_final, st.head_weight(), tgt, cfg.eps, st.head_chunk)
            return x_in, loss * scale, loss.detach()
        self._isend(x.detach(), (self.rank + 1) % P, self.fwd_group)
        return x_in, x, None

    def _backward_chunk(self, v, x_in, out):
        P = self.world
        g_first, g_last = self.first and v == 0, self.last and v == self.virtual - 1
        if g_last:
            out.backward()
        else:
            out.backward(self._recv_from(tuple(out.shape), (self.rank + 1) % P, self.bwd_group))
        if not g_first:
            self._isend(x_in.grad, (self.rank - 1) % P, self.bwd_group)

    def __call__(self, inp, tgt):
        M = self.micro_batches
        B = inp.shape[0]
        if B % M:
            raise ValueError("batch size must be a multiple of the number of micro-batches")
        mb = B // M
        live, losses = {}, []
        for kind, v, m in interleaved_schedule(self.world, self.virtual, M, self.rank):
            if kind == "F":
                sl = slice(m * mb, (m + 1) * mb)
                needs_tgt = self.last and v == self.virtual - 1
                x_in, out, lv = self._forward_chunk(v, inp[sl], tgt[sl] if needs_tgt else None, 1.0 / M)
                live[(v, m)] = (x_in, out)
                if lv is not None:
                    losses.append(lv)
            else:
                self._backward_chunk(v, *live.pop((v, m)))
        self._drain()
        if self.tied and (self.first or self.last):
            g = self.stage.embed.main_grad if hasattr(self.stage.embed, "main_grad") else self.stage.embed.grad
            dist.all_reduce(g, group=self.tie_group)
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.last:
            total += torch.stack(losses).float().sum() / M
        dist.broadcast(total, self._global(self.world - 1), group=self.group)
        self.last_losses = losses
        return total[0].detach().requires_grad_()

    def save_checkpoint(self, directory, step: int, loss: float, lr: float, trainer=None):
        import json
        from pathlib import Path
        from ..io.checkpoint import save_sciagent_checkpoint
        root = Path(directory) / f"step_{int(step)}"
        root.mkdir(parents=True, exist_ok=True)
        save_sciagent_checkpoint(self.stage, root / f"stage_{self.rank}", step, loss, lr, trainer=trainer,
                                 extra_opt={"pipeline_stage": self.rank, "chunks": [[lo, hi] for lo, hi, _ in self.chunks]})
        dist.barrier(group=self.group)
        if self.rank == 0:
            info = {"stages": self.world, "virtual_stages": self.virtual, "n_layers": self.cfg_full.n_layers,
                    "micro_batches": self.micro_batches, "split": self.split, "step": int(step)}
            (root / "pipeline.json").write_text(json.dumps(info, indent=2, sort_keys=True))
        dist.barrier(group=self.group)
        return root

    def load_checkpoint(self, root, trainer=None) -> dict:
        import json
        from pathlib import Path
        root = Path(root)
        info = json.loads((root / "pipeline.json").read_text())
        if info.get("virtual_stages", 1) != self.virtual:
            raise ValueError(f"checkpoint was written with {info.get('virtual_stages', 1)} virtual stages per rank")
        return super().load_checkpoint(root, trainer=trainer)

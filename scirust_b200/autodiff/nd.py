"""N-D reverse-mode tape: ``NdTape`` / ``NdVar`` with the reference's operator surface.

The reference keeps a second tape for N-D tensors next to the 2-D one (scirust-core/src/autodiff/nd.rs:107-680):
``input`` / ``input_from_2d`` / ``value`` / ``backward`` on the tape, and on a variable ``add sub mul div``
(NumPy-style broadcasting), ``matmul`` (2-D), ``bmm`` (leading batch axes), ``softmax`` (last axis),
``transpose_last2``, ``reshape``, ``permute``, ``layernorm`` / ``rmsnorm`` (last axis, no affine), ``sigmoid``,
``exp``, ``relu``, ``sum``, ``rope`` (positions on the second-to-last axis, interleaved pairs, frequency
``base^(-2p/d)``), ``gather`` (rows by index: an embedding lookup), ``causal_conv`` (per-channel causal convolution
with a lag-indexed filter: Hyena's primitive), ``cat0`` and the fused ``cross_entropy``. ``backward(root)`` returns
one gradient per node, indexed like the nodes.

Here a node's value is a torch tensor and the backward pass is torch's; what this module adds is the surface, the
index-addressed node list, the op semantics where they differ from torch's defaults (un-affine norms, interleaved
RoPE, lag-ordered convolution sums) and the same run-time check that two operands belong to one tape.
On CUDA tensors ``rmsnorm`` / ``rope`` / ``cross_entropy`` go through the framework's native kernels when the shapes
allow (bf16, 16-byte rows); everything else is the fp32 torch statement.
"""
from __future__ import annotations

import torch


class NdTapeError(RuntimeError):
    pass


class NdTape:
    def __init__(self, device=None):
        self.device = torch.device(device) if device is not None else None
        self.nodes: list = []

    def _push(self, t: torch.Tensor) -> "NdVar":
        v = NdVar(self, len(self.nodes), t)
        self.nodes.append(v)
        return v

    def input(self, value, requires_grad: bool = True) -> "NdVar":
        t = value.t if hasattr(value, "t") and not isinstance(value, torch.Tensor) else value
        t = torch.as_tensor(t).detach().clone()
        if not t.is_floating_point():
            t = t.float()
        if self.device is not None:
            t = t.to(self.device)
        if requires_grad:
            t.requires_grad_(True)
        return self._push(t)

    def input_from_2d(self, t) -> "NdVar":
        """A 2-D tensor of the 2-D tape family as an N-D input (same data, shape ``[rows, cols]``)."""
        return self.input(t)

    def value(self, v: "NdVar") -> torch.Tensor:
        return self.nodes[v.idx].t.detach()

    def backward(self, root: "NdVar"):
        """Gradients of ``root`` (summed if it is not a scalar) with respect to every node, by node index; nodes
        that do not influence the root get zeros."""
        if root.tape is not self:
            raise NdTapeError("backward: variable belongs to another tape")
        wanted = [n.t for n in self.nodes if n.t.requires_grad]
        grads = torch.autograd.grad(root.t.sum(), wanted, allow_unused=True, retain_graph=True)
        it = iter(grads)
        out = []
        for n in self.nodes:
            g = next(it) if n.t.requires_grad else None
            out.append(torch.zeros_like(n.t) if g is None else g)
        return out


class NdVar:
    __slots__ = ("tape", "idx", "t")

    def __init__(self, tape: NdTape, idx: int, t: torch.Tensor):
        self.tape, self.idx, self.t = tape, idx, t

    # ---- plumbing
    def _other(self, other) -> torch.Tensor:
        if isinstance(other, NdVar):
            if other.tape is not self.tape:
                raise NdTapeError("operands belong to different tapes")
            return other.t
        return torch.as_tensor(other, dtype=self.t.dtype, device=self.t.device)

    def _new(self, t: torch.Tensor) -> "NdVar":
        return self.tape._push(t)

    def shape(self):
        return list(self.t.shape)

    # ---- arithmetic (broadcasting as NumPy / the reference's ew_broadcast)
    def add(self, other):
        return self._new(self.t + self._other(other))

    def sub(self, other):
        return self._new(self.t - self._other(other))

    def mul(self, other):
        return self._new(self.t * self._other(other))

    def div(self, other):
        return self._new(self.t / self._other(other))

    __add__, __sub__, __mul__, __truediv__ = add, sub, mul, div

    def matmul(self, other):
        b = self._other(other)
        if self.t.dim() != 2 or b.dim() != 2:
            raise NdTapeError("matmul: both operands must be 2-D (use bmm for batches)")
        return self._new(self.t @ b)

    def bmm(self, other):
        b = self._other(other)
        if self.t.dim() < 3 or b.dim() != self.t.dim():
            raise NdTapeError("bmm: operands need matching leading batch axes")
        return self._new(torch.matmul(self.t, b))

    # ---- shape
    def transpose_last2(self):
        return self._new(self.t.transpose(-1, -2))

    def reshape(self, shape):
        return self._new(self.t.reshape(*shape))

    def permute(self, perm):
        return self._new(self.t.permute(*perm))

    def cat0(self, rest):
        parts = [self.t] + [self._other(r) for r in rest]
        for p in parts[1:]:
            if tuple(p.shape[1:]) != tuple(self.t.shape[1:]):
                raise NdTapeError("cat0: trailing dims must match")
        return self._new(torch.cat(parts, 0))

    def gather(self, indices):
        """Rows ``indices`` of a 2-D table (an embedding lookup); the backward pass scatter-adds."""
        idx = torch.as_tensor(indices, dtype=torch.int64, device=self.t.device)
        if self.t.dim() != 2:
            raise NdTapeError("gather: the table must be 2-D")
        if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= self.t.shape[0]):
            raise NdTapeError("gather: index out of range")
        return self._new(self.t.index_select(0, idx))

    # ---- pointwise / reductions
    def relu(self):
        return self._new(torch.relu(self.t))

    def sigmoid(self):
        return self._new(torch.sigmoid(self.t))

    def exp(self):
        return self._new(torch.exp(self.t))

    def sum(self):
        return self._new(self.t.sum().reshape(1))

    def softmax(self):
        return self._new(torch.softmax(self.t, -1))

    # ---- normalisation without affine (gains are applied by a separate mul / add)
    def layernorm(self, eps: float = 1e-5):
        x = self.t
        mu = x.mean(-1, keepdim=True)
        var = (x - mu).pow(2).mean(-1, keepdim=True)
        return self._new((x - mu) * torch.rsqrt(var + eps))

    def rmsnorm(self, eps: float = 1e-5):
        x = self.t
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            from ..nn.functional_native import rmsnorm_unit_gain
            return self._new(rmsnorm_unit_gain(x, eps))
        return self._new(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))

    def rope(self, base: float = 10000.0):
        """Rotary embedding over ``(..., seq, d)``: pair ``(x[2p], x[2p+1])`` at position ``pos`` turns by
        ``pos * base^(-2p/d)``."""
        x = self.t
        d = x.shape[-1]
        if d % 2:
            raise NdTapeError("rope: last axis must be even")
        seq = x.shape[-2]
        pos = torch.arange(seq, dtype=torch.float32, device=x.device)
        freq = torch.pow(torch.tensor(float(base), device=x.device),
                         -2.0 * torch.arange(d // 2, dtype=torch.float32, device=x.device) / d)
        ang = pos[:, None] * freq[None, :]
        c, s = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out = torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).reshape(x.shape)
        return self._new(out)

    def causal_conv(self, h):
        """``y[t, c] = sum_{tau=0..t} h[tau, c] * u[t - tau, c]`` for ``(seq, d)`` signal and filter, the taps added in
        ascending ``tau`` (the reference's order, so a CPU fp32 result is bit-identical to its direct loop)."""
        u, hh = self.t, self._other(h)
        if u.dim() != 2 or tuple(u.shape) != tuple(hh.shape):
            raise NdTapeError("causal_conv: signal and filter must share shape (seq, d)")
        seq = u.shape[0]
        y = torch.zeros_like(u)
        for tau in range(seq):
            y = y + torch.cat([torch.zeros_like(u[:tau]), hh[tau:tau + 1] * u[:seq - tau]], 0)
        return self._new(y)

    def cross_entropy(self, targets):
        """Mean negative log-likelihood of ``(n, vocab)`` logits, log-sum-exp form; scalar of shape ``[1]``."""
        x = self.t
        if x.dim() != 2:
            raise NdTapeError("cross_entropy: logits must be 2-D (n, vocab)")
        tgt = torch.as_tensor(targets, dtype=torch.int64, device=x.device)
        if tgt.numel() != x.shape[0]:
            raise NdTapeError("cross_entropy: one target per row")
        if tgt.numel() and (int(tgt.min()) < 0 or int(tgt.max()) >= x.shape[1]):
            raise NdTapeError("cross_entropy: target out of range")
        xf = x.float()
        mx = xf.max(-1, keepdim=True).values
        lse = mx.squeeze(-1) + torch.log(torch.exp(xf - mx).sum(-1))
        loss = (lse - xf.gather(1, tgt[:, None]).squeeze(1)).sum() / x.shape[0]
        return self._new(loss.reshape(1))

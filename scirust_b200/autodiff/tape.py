"""Tape-style reverse-mode autodiff with SciRust's surface, executed by ``torch.autograd``.

The reference records nodes on a ``Tape`` (three parallel vectors: nodes / values / grads), hands
out ``Var`` handles tied to the tape, builds one fresh tape per step and walks it backwards in
``Tape::backward`` (scirust-core/src/autodiff/reverse.rs:1369-1385, 1559-1586, 1664-3433; ops
``impl Var`` :3451-5412). Here a ``Var`` wraps a torch tensor (2-D, like the reference's
``Tensor``), the tape keeps the node list so ``value(idx)`` / ``grad(idx)`` / ``set_value`` work by
index exactly as optimizers expect, and the backward pass is torch's. Using a ``Var`` with another
tape raises, as the reference does at run time (:3461).

Values may live on CPU (deterministic fp32) or CUDA; ``Tape(device=...)`` moves inputs there.
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.nn.functional as F

from ..tensor import Tensor


class TapeError(RuntimeError):
    pass


def _t(x):
    if isinstance(x, Tensor):
        return x.t
    return torch.as_tensor(x, dtype=torch.float32)


class Tape:
    def __init__(self, device=None):
        self.device = torch.device(device) if device is not None else None
        self.vars: list = []
        self._no_grad = False
        self._gen = torch.Generator()
        self._gen.manual_seed(0)
        self.training = True

    # ---- registration
    def _push(self, t: torch.Tensor, leaf: bool = False) -> "Var":
        v = Var(self, len(self.vars), t)
        self.vars.append(v)
        return v

    def input(self, value, requires_grad: bool = True) -> "Var":
        t = _t(value).detach().clone()
        if self.device is not None:
            t = t.to(self.device)
        if t.dim() == 1:
            t = t.reshape(1, -1)
        if requires_grad and not self._no_grad and t.is_floating_point():
            t.requires_grad_(True)
        return self._push(t, leaf=True)

    def constant(self, value) -> "Var":
        return self.input(value, requires_grad=False)

    def __len__(self):
        return len(self.vars)

    # ---- access by node index
    def value(self, idx: int) -> Tensor:
        return Tensor(self.vars[idx].t.detach().cpu())

    def grad(self, idx: int) -> Tensor:
        v = self.vars[idx].t
        g = v.grad if v.grad is not None else torch.zeros_like(v)
        return Tensor(g.detach().cpu())

    def set_value(self, idx: int, value) -> None:
        with torch.no_grad():
            self.vars[idx].t.copy_(_t(value).to(self.vars[idx].t.device))

    # ---- differentiation
    def backward(self, loss) -> None:
        idx = loss.idx if isinstance(loss, Var) else int(loss)
        v = self.vars[idx]
        if v.t.numel() != 1:
            raise TapeError("backward expects a scalar (1x1) loss")
        if v.t.requires_grad:
            v.t.backward()

    @contextlib.contextmanager
    def no_grad(self):
        prev = self._no_grad
        self._no_grad = True
        try:
            with torch.no_grad():
                yield self
        finally:
            self._no_grad = prev

    def clip_grad_norm(self, indices, max_norm: float) -> float:
        """Scale the gradients of the given nodes so their joint L2 norm is at most ``max_norm``;
        returns the norm before clipping (reverse.rs:1624)."""
        sq = 0.0
        for i in indices:
            g = self.vars[i].t.grad
            if g is not None:
                sq += float((g.double() ** 2).sum())
        norm = math.sqrt(sq)
        if max_norm > 0 and norm > max_norm:
            k = max_norm / norm
            for i in indices:
                g = self.vars[i].t.grad
                if g is not None:
                    g.mul_(k)
        return norm

    def clip_grad_value(self, indices, max_value: float) -> None:
        """Clamp every gradient element of the given nodes to ``[-max_value, max_value]``."""
        for i in indices:
            g = self.vars[i].t.grad
            if g is not None:
                g.clamp_(-max_value, max_value)

    def zeros(self, rows: int, cols: int) -> "Var":
        return self.constant(torch.zeros(rows, cols))

    def ones(self, rows: int, cols: int) -> "Var":
        return self.constant(torch.ones(rows, cols))

    def set_seed(self, seed: int) -> None:
        """Seed of the dropout mask stream (reverse.rs:1406)."""
        self._gen.manual_seed(int(seed))

    def train(self, mode: bool = True):
        self.training = mode


class Var:
    __slots__ = ("tape", "idx", "t")

    def __init__(self, tape: Tape, idx: int, t: torch.Tensor):
        self.tape, self.idx, self.t = tape, idx, t

    # ---- helpers
    def _same(self, o: "Var") -> None:
        if o.tape is not self.tape:
            raise TapeError("variables belong to different tapes")

    def _new(self, t: torch.Tensor) -> "Var":
        return self.tape._push(t)

    def _shape_eq(self, o: "Var", what: str) -> None:
        if self.t.shape != o.t.shape:
            raise TapeError(f"{what}: shape mismatch {tuple(self.t.shape)} vs {tuple(o.t.shape)}")

    def value(self) -> Tensor:
        return Tensor(self.t.detach().cpu())

    def shape(self):
        return tuple(self.t.shape)

    def item(self) -> float:
        return float(self.t.detach().reshape(-1)[0])

    # ---- arithmetic
    def add(self, o):
        self._same(o); self._shape_eq(o, "add")
        return self._new(self.t + o.t)

    def sub(self, o):
        self._same(o); self._shape_eq(o, "sub")
        return self._new(self.t - o.t)

    def mul(self, o):
        self._same(o); self._shape_eq(o, "mul")
        return self._new(self.t * o.t)
    hadamard = mul

    def div(self, o):
        self._same(o); self._shape_eq(o, "div")
        return self._new(self.t / o.t)

    def add_bias(self, b):
        """(rows, cols) + (1, cols)."""
        self._same(b)
        if b.t.shape[0] != 1 or b.t.shape[1] != self.t.shape[1]:
            raise TapeError("add_bias expects a (1, cols) bias")
        return self._new(self.t + b.t)
    add_broadcast = add_bias

    def sub_broadcast(self, b): self._same(b); return self._new(self.t - b.t)
    def mul_broadcast(self, b): self._same(b); return self._new(self.t * b.t)
    def div_broadcast(self, b): self._same(b); return self._new(self.t / b.t)
    def scale(self, k: float): return self._new(self.t * float(k))
    def neg(self): return self._new(-self.t)
    def exp(self): return self._new(torch.exp(self.t))
    def log(self): return self._new(torch.log(self.t))
    ln = log
    def sqrt(self): return self._new(torch.sqrt(self.t))
    def reciprocal(self): return self._new(torch.reciprocal(self.t))
    def pow(self, p: float): return self._new(torch.pow(self.t, float(p)))
    def sin(self): return self._new(torch.sin(self.t))
    def cos(self): return self._new(torch.cos(self.t))
    def tan(self): return self._new(torch.tan(self.t))
    def asin(self): return self._new(torch.asin(self.t))
    def acos(self): return self._new(torch.acos(self.t))
    def atan(self): return self._new(torch.atan(self.t))
    def atan2(self, o): self._same(o); return self._new(torch.atan2(self.t, o.t))
    def abs(self): return self._new(torch.abs(self.t))
    def relu(self): return self._new(torch.relu(self.t))
    def sigmoid(self): return self._new(torch.sigmoid(self.t))
    def tanh(self): return self._new(torch.tanh(self.t))
    def gelu(self): return self._new(F.gelu(self.t))
    def gelu_tanh(self): return self._new(F.gelu(self.t, approximate="tanh"))   # the form of tensor/parity.rs:136 and of the fused kernels

    def lgamma(self): return self._new(torch.lgamma(self.t))
    def digamma(self): return self._new(torch.digamma(self.t))

    def gather(self, axis: int, indices):
        """``out[i][j] = x[indices[i][j]][j]`` (axis 0) or ``x[i][indices[i][j]]`` (axis 1); gradients scatter-add back."""
        idx = torch.as_tensor(indices, dtype=torch.long, device=self.t.device).reshape(self.t.shape)
        return self._new(torch.gather(self.t, axis, idx))

    def unfold(self, axis: int, size: int, step: int):
        """Sliding windows along ``axis``, flattened to 2-D: rows = (kept axis, window index), columns = window."""
        u = self.t.unfold(axis, size, step)                                   # [.., windows, size] with the window axis last
        return self._new(u.reshape(-1, size))

    def conv1d(self, w, b, in_c: int, length: int, k: int, stride: int = 1):
        """Input ``(B, C * L)`` flattened like the 2-D convolution, weight ``(out_c, in_c * K)``, bias ``(1, out_c)``."""
        if k > length:
            raise TapeError(f"conv1d: kernel {k} is larger than the input length {length}")
        x = self.t.reshape(-1, in_c, length)
        y = F.conv1d(x, w.t.reshape(w.t.shape[0], in_c, k), b.t.reshape(-1) if b is not None else None, stride=stride)
        return self._new(y.reshape(y.shape[0], -1))

    def cholesky(self):
        """Lower-triangular factor of a symmetric positive-definite matrix."""
        if self.t.dim() != 2 or self.t.shape[0] != self.t.shape[1]:
            raise TapeError(f"cholesky: the matrix must be square, got {tuple(self.t.shape)}")
        l, info = torch.linalg.cholesky_ex(self.t)
        if int(info):
            raise TapeError(f"cholesky: the matrix is not positive-definite (leading minor {int(info)})")
        return self._new(l)
    def silu(self): return self._new(F.silu(self.t))
    __add__, __sub__, __mul__, __truediv__, __neg__ = add, sub, mul, div, neg

    # ---- matrix products
    def matmul(self, o):
        self._same(o)
        if self.t.shape[1] != o.t.shape[0]:
            raise TapeError(f"matmul: inner dimensions differ ({self.t.shape[1]} vs {o.t.shape[0]})")
        return self._new(self.t @ o.t)
    try_matmul = matmul

    def matmul_bt(self, o):
        self._same(o)
        return self._new(self.t @ o.t.t())

    def bmm2d(self, o, batch: int):
        """Batched matmul over tensors flattened to 2-D: (batch*m, k) x (batch*k, n) -> (batch*m, n)."""
        self._same(o)
        m, k = self.t.shape[0] // batch, self.t.shape[1]
        n = o.t.shape[1]
        r = torch.bmm(self.t.reshape(batch, m, k), o.t.reshape(batch, k, n))
        return self._new(r.reshape(batch * m, n))

    def linear(self, w, b=None):
        """x.W (+ b) with W (in, out), b (1, out)  (reverse.rs:4697)."""
        y = self.matmul(w)
        return y.add_bias(b) if b is not None else y
    try_linear = linear

    def transpose(self): return self._new(self.t.t())
    def reshape(self, rows: int, cols: int): return self._new(self.t.reshape(rows, cols))

    # ---- reductions
    def sum(self): return self._new(self.t.sum().reshape(1, 1))
    def mean(self): return self._new(self.t.mean().reshape(1, 1))
    def sum_axis(self, axis: int): return self._new(self.t.sum(axis, keepdim=True))
    def mean_axis(self, axis: int): return self._new(self.t.mean(axis, keepdim=True))
    def var_axis(self, axis: int): return self._new(self.t.var(axis, unbiased=False, keepdim=True))
    def max_axis(self, axis: int): return self._new(self.t.amax(axis, keepdim=True))

    def broadcast(self, rows: int, cols: int):
        return self._new(self.t.expand(rows, cols))

    def softmax(self): return self._new(torch.softmax(self.t, 1))
    def log_softmax(self): return self._new(torch.log_softmax(self.t, 1))

    # ---- structure
    @staticmethod
    def concat_rows(vs):
        if len({v.t.shape[1] for v in vs}) != 1:
            raise TapeError(f"concat_rows: column counts differ: {[v.t.shape[1] for v in vs]}")
        return vs[0]._new(torch.cat([v.t for v in vs], 0))

    @staticmethod
    def concat_cols(vs):
        if len({v.t.shape[0] for v in vs}) != 1:
            raise TapeError(f"concat_cols: row counts differ: {[v.t.shape[0] for v in vs]}")
        return vs[0]._new(torch.cat([v.t for v in vs], 1))

    def slice_rows(self, a: int, b: int): return self._new(self.t[a:b])
    def slice_cols(self, a: int, b: int): return self._new(self.t[:, a:b])

    def embedding(self, indices):
        """Rows of this table selected by ``indices`` (reverse.rs embedding op)."""
        idx = torch.as_tensor(indices, dtype=torch.long, device=self.t.device)
        if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= self.t.shape[0]):
            raise TapeError("embedding index out of range")
        return self._new(self.t[idx])

    def causal_mask(self, seq: int = None):
        """Adds -1e30-style masking of j > i for square score blocks (reverse.rs:4838)."""
        n = self.t.shape[1]
        rows = self.t.shape[0]
        i = torch.arange(rows, device=self.t.device) % n
        mask = torch.arange(n, device=self.t.device)[None, :] > i[:, None]
        return self._new(self.t.masked_fill(mask, -1.0e9))

    def dropout(self, p: float):
        if not self.tape.training or p <= 0.0:
            return self
        keep = (torch.rand(self.t.shape, generator=self.tape._gen) >= p).to(self.t.device, self.t.dtype)
        return self._new(self.t * keep / (1.0 - p))

    def layer_norm(self, gamma, beta, eps: float = 1e-5):
        self._same(gamma); self._same(beta)
        return self._new(F.layer_norm(self.t, (self.t.shape[1],), gamma.t.reshape(-1), beta.t.reshape(-1), eps))
    try_layer_norm = layer_norm

    def rms_norm(self, gamma, eps: float = 1e-5):
        self._same(gamma)
        inv = torch.rsqrt(self.t.pow(2).mean(1, keepdim=True) + eps)
        return self._new(self.t * inv * gamma.t.reshape(1, -1))

    def l2_normalize(self, eps: float = 1e-12):
        return self._new(self.t / (self.t.norm(dim=1, keepdim=True) + eps))

    def cosine_sim_matrix(self, o):
        self._same(o)
        a = self.t / (self.t.norm(dim=1, keepdim=True) + 1e-12)
        b = o.t / (o.t.norm(dim=1, keepdim=True) + 1e-12)
        return self._new(a @ b.t())

    # ---- convolution family: NCHW flattened to (B, C*H*W); weight (out_c, in_c*K*K)
    def conv2d(self, w, b, in_c: int, h: int, wd: int, k: int, stride: int = 1, same: bool = False):
        if not same and (k > h or k > wd):
            raise TapeError(f"conv2d: kernel {k} is larger than the {h} x {wd} input")
        self._same(w)
        B = self.t.shape[0]
        out_c = w.t.shape[0]
        pad = (k - 1) // 2 if same else 0
        y = F.conv2d(self.t.reshape(B, in_c, h, wd), w.t.reshape(out_c, in_c, k, k),
                     b.t.reshape(-1) if b is not None else None, stride=stride, padding=pad)
        return self._new(y.reshape(B, -1))
    try_conv2d_forward = conv2d

    def conv2d_transpose(self, w, b, in_c: int, h: int, wd: int, k: int, stride: int = 1):
        B = self.t.shape[0]
        out_c = w.t.shape[0]
        y = F.conv_transpose2d(self.t.reshape(B, in_c, h, wd), w.t.reshape(out_c, in_c, k, k).transpose(0, 1),
                               b.t.reshape(-1) if b is not None else None, stride=stride)
        return self._new(y.reshape(B, -1))

    def max_pool2d(self, c: int, h: int, wd: int, k: int, stride: int):
        B = self.t.shape[0]
        y = F.max_pool2d(self.t.reshape(B, c, h, wd), k, stride)
        return self._new(y.reshape(B, -1))

    def avg_pool2d(self, c: int, h: int, wd: int, k: int, stride: int):
        B = self.t.shape[0]
        return self._new(F.avg_pool2d(self.t.reshape(B, c, h, wd), k, stride).reshape(B, -1))

    # ---- attention
    def flash_attention(self, k, v, causal: bool = False, scale: float = None):
        """softmax(q k^T * scale [+ causal mask]) v for one head, blockwise-equivalent result."""
        self._same(k); self._same(v)
        d = self.t.shape[1]
        scale = 1.0 / math.sqrt(d) if scale is None else scale
        s = (self.t @ k.t.t()) * scale
        if causal:
            n, m = s.shape
            s = s.masked_fill(torch.triu(torch.ones(n, m, dtype=torch.bool, device=s.device), 1), float("-inf"))
        return self._new(torch.softmax(s, 1) @ v.t)

    # ---- quantisation-aware training: fake-quantise with a straight-through gradient
    def fake_quantize(self, bits: int = 8):
        qmax = float(2 ** (bits - 1) - 1)
        mx = self.t.detach().abs().max()
        scale = torch.where(mx > 0, mx / qmax, torch.ones_like(mx))
        q = torch.clamp(torch.round(self.t / scale), -qmax - 1, qmax) * scale
        return self._new(self.t + (q - self.t).detach())

    # ---- portable (libm-free, bit-reproducible) variants
    def exp_portable(self):
        from ..numerics import portable
        return self._new(portable.PortableExp.apply(self.t))

    def matmul_portable(self, o):
        from ..numerics import portable
        return self._new(portable.PortableMatmul.apply(self.t, o.t))

    def ln_portable(self):
        from ..numerics import portable
        return self._new(portable.PortableLn.apply(self.t))

    def softmax_portable(self):
        from ..numerics import portable
        return self._new(portable.PortableSoftmax.apply(self.t))

    # ---- remaining elementwise / structural ops of the reference surface
    def sinh(self): return self._new(torch.sinh(self.t))
    def cosh(self): return self._new(torch.cosh(self.t))
    def log10(self): return self._new(torch.log10(self.t))

    def add_scaled(self, o, k: float):
        """self + k * o."""
        self._same(o); self._shape_eq(o, "add_scaled")
        return self._new(self.t + float(k) * o.t)

    def add_hadamard(self, a, b):
        """self + a * b (element-wise)."""
        self._same(a); self._same(b); self._shape_eq(a, "add_hadamard"); self._shape_eq(b, "add_hadamard")
        return self._new(torch.addcmul(self.t, a.t, b.t))

    def sub_hadamard(self, a, b):
        self._same(a); self._same(b); self._shape_eq(a, "sub_hadamard"); self._shape_eq(b, "sub_hadamard")
        return self._new(torch.addcmul(self.t, a.t, b.t, value=-1.0))

    def broadcast_to(self, rows: int, cols: int):
        r, c = self.t.shape
        if (r not in (1, rows)) or (c not in (1, cols)):
            raise TapeError(f"broadcast_to: cannot expand {(r, c)} to {(rows, cols)}")
        return self._new(self.t.expand(rows, cols))

    def detach(self):
        """The same values as a new leaf that stops the gradient."""
        return self.tape.constant(self.t.detach())

    def fake_quantize_ste_range(self, lo: float, hi: float, bits: int = 8):
        """Uniform quantiser over a FIXED range with a straight-through gradient inside it and zero outside."""
        if not hi > lo:
            raise TapeError("fake_quantize_ste_range needs hi > lo")
        levels = float(2 ** bits - 1)
        step = (hi - lo) / levels
        x = self.t.clamp(lo, hi)
        q = torch.round((x - lo) / step) * step + lo
        return self._new(x + (q - x).detach())

    def tt_contract(self, cores, bias, in_dims, out_dims, ranks):
        """``x [B, prod(in_dims)]`` through a tensor-train weight: core k is ``[r_k * in_k * out_k, r_{k+1}]``
        (row-major ``(r_k, in_k, out_k)``), ``ranks`` has ``d + 1`` entries starting and ending with 1. The product is
        contracted core by core, never forming the dense ``[in, out]`` matrix."""
        d = len(in_dims)
        if d == 0 or d > 8 or len(out_dims) != d or len(ranks) != d + 1 or len(cores) != d:
            raise TapeError("tt_contract: need 1..8 modes, matching out_dims, d + 1 ranks and d cores")
        if ranks[0] != 1 or ranks[-1] != 1:
            raise TapeError("tt_contract: boundary ranks must be 1")
        B = self.t.shape[0]
        if self.t.shape[1] != math.prod(in_dims):
            raise TapeError(f"tt_contract: input width {self.t.shape[1]} != prod(in_dims) {math.prod(in_dims)}")
        # state [B, r_k, remaining inputs..., produced outputs]
        state = self.t.reshape(B, 1, *in_dims, 1)
        for k, core in enumerate(cores):
            self._same(core)
            rk, ik, ok, rn = ranks[k], in_dims[k], out_dims[k], ranks[k + 1]
            if core.t.numel() != rk * ik * ok * rn:
                raise TapeError(f"tt_contract: core {k} has {core.t.numel()} elements, expected {rk * ik * ok * rn}")
            g = core.t.reshape(rk, ik, ok, rn)
            rest = state.shape[3:-1]
            st = state.reshape(B, rk, ik, -1, state.shape[-1])                 # [B, r, i, rest, outs]
            st = torch.einsum("brixo,ripn->bnxop", st, g)                      # -> [B, r', rest, outs, out_k]
            state = st.reshape(B, rn, *rest, st.shape[3] * ok)
        y = state.reshape(B, -1)
        if bias is not None:
            self._same(bias)
            y = y + bias.t.reshape(1, -1)
        return self._new(y)
    try_tt_contract = tt_contract

    def quantum_expectations(self, parameters, layer):
        """Rows of classical features through a ``quantum.QuantumLayer`` with shared trainable ``parameters [1, P]``:
        ``[batch, observables]``, differentiable in both."""
        self._same(parameters)
        return self._new(layer.forward(self.t, parameters.t))
    try_quantum_expectations = quantum_expectations

    def quantum_expectation(self, parameters, layer):
        from ..quantum import QuantumError
        if len(layer.observables) != 1:
            raise QuantumError("quantum_expectation needs a layer with exactly one observable")
        if self.t.shape[0] != 1:
            raise QuantumError("quantum_expectation takes one row of features")
        return self.quantum_expectations(parameters, layer)
    try_quantum_expectation = quantum_expectation

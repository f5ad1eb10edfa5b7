"""Dense tensors with SciRust's surface on top of ``torch.Tensor``.

``Tensor`` is the reference's row-major 2-D fp32 matrix (scirust-core/src/autodiff/reverse.rs:
291-1078): ``rows``, ``cols``, ``data``; element-wise ops, axis reductions, softmax / log-softmax,
transpose, matmul, broadcasting helpers. ``Tensor.sum`` adds left to right like the reference's
sequential ``iter().sum()`` (:681-683) so seeded CPU runs reproduce its bits.
``TensorND`` mirrors scirust-core/src/tensor/tensor_nd.rs:16-440 (shape + flat data, reshape,
transpose, slice, broadcast, 2-D bridge). Both hold a ``torch.Tensor`` in ``.t`` and move to CUDA
with ``.to(device)``.
"""
from __future__ import annotations

import ctypes as C

import torch


def _seq_sum(t: torch.Tensor) -> float:
    """Left-to-right fp32 sum (native loop; bit-identical to a sequential Rust ``iter().sum()``)."""
    from .ops import _lib
    lib = _lib.rt()
    lib.sbrt_sum_f32.argtypes = [C.c_void_p, C.c_int64]
    lib.sbrt_sum_f32.restype = C.c_float
    x = t.detach().to(torch.float32).cpu().contiguous()
    return float(lib.sbrt_sum_f32(x.data_ptr(), x.numel()))


class Tensor:
    __slots__ = ("t",)

    def __init__(self, t: torch.Tensor):
        if t.dim() != 2:
            raise ValueError(f"Tensor is 2-D; got shape {tuple(t.shape)}")
        self.t = t.to(torch.float32)

    # ---- construction
    @staticmethod
    def from_vec(data, rows: int, cols: int) -> "Tensor":
        t = torch.as_tensor(data, dtype=torch.float32)
        if t.numel() != rows * cols:
            raise ValueError(f"from_vec: {t.numel()} values for shape {rows}x{cols}")
        return Tensor(t.reshape(rows, cols).clone())

    @staticmethod
    def zeros(rows: int, cols: int) -> "Tensor":
        return Tensor(torch.zeros(rows, cols))

    @staticmethod
    def ones(rows: int, cols: int) -> "Tensor":
        return Tensor(torch.ones(rows, cols))

    @staticmethod
    def scalar(v: float) -> "Tensor":
        return Tensor(torch.full((1, 1), float(v)))

    @staticmethod
    def eye(n: int) -> "Tensor":
        return Tensor(torch.eye(n))

    # ---- views
    @property
    def rows(self) -> int:
        return self.t.shape[0]

    @property
    def cols(self) -> int:
        return self.t.shape[1]

    @property
    def data(self) -> list:
        return self.t.reshape(-1).tolist()

    def shape(self):
        return (self.rows, self.cols)

    def get(self, r: int, c: int) -> float:
        return float(self.t[r, c])

    def set(self, r: int, c: int, v: float) -> None:
        self.t[r, c] = v

    def clone(self) -> "Tensor":
        return Tensor(self.t.clone())

    def to(self, device) -> "Tensor":
        return Tensor(self.t.to(device))

    # ---- element-wise
    def _bin(self, other, fn):
        o = other.t if isinstance(other, Tensor) else other
        if isinstance(other, Tensor) and other.t.shape != self.t.shape:
            raise ValueError(f"shape mismatch {tuple(self.t.shape)} vs {tuple(other.t.shape)}")
        return Tensor(fn(self.t, o))

    def add(self, o): return self._bin(o, torch.add)
    def sub(self, o): return self._bin(o, torch.sub)
    def hadamard(self, o): return self._bin(o, torch.mul)
    def div(self, o): return self._bin(o, torch.div)
    def scale(self, k: float): return Tensor(self.t * float(k))
    def neg(self): return Tensor(-self.t)
    def exp(self): return Tensor(torch.exp(self.t))
    def ln(self): return Tensor(torch.log(self.t))
    def sqrt(self): return Tensor(torch.sqrt(self.t))
    def abs(self): return Tensor(torch.abs(self.t))
    def relu(self): return Tensor(torch.relu(self.t))
    def sigmoid(self): return Tensor(torch.sigmoid(self.t))
    def tanh(self): return Tensor(torch.tanh(self.t))
    def map(self, fn): return Tensor(torch.tensor([fn(v) for v in self.data], dtype=torch.float32).reshape(self.t.shape))
    __add__, __sub__, __mul__, __neg__ = add, sub, hadamard, neg

    # ---- broadcasting helpers
    def add_row_broadcast(self, row: "Tensor") -> "Tensor":
        if row.rows != 1 or row.cols != self.cols:
            raise ValueError("add_row_broadcast expects a (1, cols) tensor")
        return Tensor(self.t + row.t)

    def broadcast_rows(self, rows: int) -> "Tensor":
        if self.rows != 1:
            raise ValueError("broadcast_rows expects a (1, cols) tensor")
        return Tensor(self.t.expand(rows, self.cols).clone())

    def broadcast_cols(self, cols: int) -> "Tensor":
        if self.cols != 1:
            raise ValueError("broadcast_cols expects a (rows, 1) tensor")
        return Tensor(self.t.expand(self.rows, cols).clone())

    # ---- reductions
    def sum(self) -> float:
        if self.t.is_cuda:
            return float(self.t.sum())
        return _seq_sum(self.t)

    def mean(self) -> float:
        return self.sum() / float(self.t.numel())

    def sum_axis(self, axis: int) -> "Tensor":
        return Tensor(self.t.sum(axis, keepdim=True))

    def mean_axis(self, axis: int) -> "Tensor":
        return Tensor(self.t.mean(axis, keepdim=True))

    def max_axis(self, axis: int) -> "Tensor":
        return Tensor(self.t.amax(axis, keepdim=True))

    def argmax_rows(self) -> list:
        return self.t.argmax(1).tolist()

    def softmax(self) -> "Tensor":
        return Tensor(torch.softmax(self.t, 1))

    def log_softmax(self) -> "Tensor":
        return Tensor(torch.log_softmax(self.t, 1))

    # ---- linear algebra
    def transpose(self) -> "Tensor":
        return Tensor(self.t.t().contiguous())

    def matmul(self, o: "Tensor") -> "Tensor":
        if self.cols != o.rows:
            raise ValueError(f"matmul: inner dimensions differ ({self.cols} vs {o.rows})")
        return Tensor(self.t @ o.t)

    def matmul_bt(self, o: "Tensor") -> "Tensor":
        return Tensor(self.t @ o.t.t())

    def slice_rows(self, a: int, b: int) -> "Tensor":
        return Tensor(self.t[a:b].clone())

    def slice_cols(self, a: int, b: int) -> "Tensor":
        return Tensor(self.t[:, a:b].clone())

    @staticmethod
    def concat_rows(ts) -> "Tensor":
        return Tensor(torch.cat([x.t for x in ts], 0))

    @staticmethod
    def concat_cols(ts) -> "Tensor":
        return Tensor(torch.cat([x.t for x in ts], 1))

    def frobenius_norm(self) -> float:
        return float(torch.linalg.norm(self.t))

    def __eq__(self, o):
        return isinstance(o, Tensor) and torch.equal(self.t, o.t)

    def __repr__(self):
        return f"Tensor({self.rows}x{self.cols})"


class TensorND:
    """N-dimensional fp32 tensor (flat row-major data + shape)."""
    __slots__ = ("t",)

    def __init__(self, t: torch.Tensor):
        self.t = t.to(torch.float32)

    @staticmethod
    def from_vec(data, shape) -> "TensorND":
        t = torch.as_tensor(data, dtype=torch.float32)
        n = 1
        for s in shape:
            n *= s
        if t.numel() != n:
            raise ValueError(f"{t.numel()} values for shape {tuple(shape)}")
        return TensorND(t.reshape(tuple(shape)).clone())

    @staticmethod
    def zeros(shape) -> "TensorND":
        return TensorND(torch.zeros(tuple(shape)))

    @property
    def shape(self):
        return tuple(self.t.shape)

    @property
    def data(self):
        return self.t.reshape(-1).tolist()

    def ndim(self): return self.t.dim()
    def numel(self): return self.t.numel()
    def reshape(self, shape): return TensorND(self.t.reshape(tuple(shape)))
    def transpose(self, a: int, b: int): return TensorND(self.t.transpose(a, b).contiguous())
    def permute(self, dims): return TensorND(self.t.permute(*dims).contiguous())
    def slice(self, dim: int, a: int, b: int): return TensorND(self.t.narrow(dim, a, b - a).clone())
    def broadcast_to(self, shape): return TensorND(self.t.expand(tuple(shape)).clone())
    def add(self, o): return TensorND(self.t + o.t)
    def sub(self, o): return TensorND(self.t - o.t)
    def mul(self, o): return TensorND(self.t * o.t)
    def div(self, o): return TensorND(self.t / o.t)
    def matmul(self, o): return TensorND(self.t @ o.t)
    def sum_to(self, shape):
        """Sum broadcast dimensions back to ``shape`` (the adjoint of ``broadcast_to``)."""
        t = self.t
        while t.dim() > len(shape):
            t = t.sum(0)
        for i, s in enumerate(shape):
            if s == 1 and t.shape[i] != 1:
                t = t.sum(i, keepdim=True)
        return TensorND(t)

    def to_2d(self) -> Tensor:
        if self.t.dim() == 1:
            return Tensor(self.t.reshape(1, -1))
        return Tensor(self.t.reshape(-1, self.t.shape[-1]))

    @staticmethod
    def from_2d(t: Tensor, shape=None) -> "TensorND":
        return TensorND(t.t.reshape(tuple(shape)) if shape is not None else t.t)

    def to(self, device): return TensorND(self.t.to(device))
    def __repr__(self): return f"TensorND{self.shape}"


class Tensor3D:
    """A ``(batch, seq_len, d_model)`` view over a 2-D ``(batch * seq_len, d_model)`` tensor: the shape convention of
    the sequence layers (scirust-core/src/tensor/tensor3d.rs:7-80)."""

    def __init__(self, inner: Tensor, batch: int, seq_len: int, d_model: int):
        if inner.rows != batch * seq_len or inner.cols != d_model:
            raise ValueError(f"Tensor3D: a {inner.shape} matrix is not ({batch} * {seq_len}, {d_model})")
        self.inner, self.batch, self.seq_len, self.d_model = inner, batch, seq_len, d_model

    @staticmethod
    def zeros(batch: int, seq_len: int, d_model: int) -> "Tensor3D":
        return Tensor3D(Tensor.zeros(batch * seq_len, d_model), batch, seq_len, d_model)

    @property
    def shape(self):
        return self.batch, self.seq_len, self.d_model

    def as_nd(self) -> "TensorND":
        return TensorND(self.inner.t.reshape(self.batch, self.seq_len, self.d_model))


class Var3D:
    """The tape counterpart of ``Tensor3D``: a ``Var`` plus its 3-D interpretation."""

    def __init__(self, var, batch: int, seq_len: int, d_model: int):
        if tuple(var.t.shape) != (batch * seq_len, d_model):
            raise ValueError(f"Var3D: a {tuple(var.t.shape)} variable is not ({batch} * {seq_len}, {d_model})")
        self.var, self.batch, self.seq_len, self.d_model = var, batch, seq_len, d_model

    @staticmethod
    def input_3d(tape, t3d: Tensor3D) -> "Var3D":
        return Var3D(tape.input(t3d.inner), t3d.batch, t3d.seq_len, t3d.d_model)

    from_var = classmethod(lambda cls, var, b, s, d: cls(var, b, s, d))

    @property
    def shape(self):
        return self.batch, self.seq_len, self.d_model

    def as_var(self):
        return self.var


def broadcast_get(data, shape, idx) -> float:
    """Element of a row-major array read with broadcasting: axes of extent 1 ignore their index
    (scirust-core/src/tensor/broadcast.rs:23)."""
    off, stride = 0, 1
    for extent, i in zip(reversed(list(shape)), reversed(list(idx))):
        off += (0 if extent == 1 else i) * stride
        stride *= extent
    return float(data[off])


def unbroadcast(grad: "torch.Tensor", shape) -> "torch.Tensor":
    """Sum a gradient back to the shape it was broadcast from (leading axes and axes of extent 1)."""
    g = grad
    while g.dim() > len(shape):
        g = g.sum(0)
    for ax, extent in enumerate(shape):
        if extent == 1 and g.shape[ax] != 1:
            g = g.sum(ax, keepdim=True)
    return g

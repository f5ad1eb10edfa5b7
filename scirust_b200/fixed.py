"""Deterministic fixed-point arithmetic on integer tensors: every operation is integer-only (int32 storage, int64
intermediates), so results are bit-identical on any CPU and on the GPU, whatever the thread count, library version or
reduction order; the point of the format is reproducible inference and exactly reversible transforms, not speed.

A ``FixedTensor`` holds ``raw`` (int32) and ``frac`` (fractional bits): value = raw / 2^frac. Conventions:
* ``round_shift(wide, frac, mode)`` divides by 2^frac with one of four rounding modes (toward zero, floor, ceil, nearest
  with ties to even); ``narrow(wide, overflow)`` brings an int64 back to int32 by wrapping, saturating or raising.
* add / sub / neg are exact (then narrowed); mul takes the 64-bit product and rounds it once; div shifts the numerator.
* ``dot`` / ``matmul`` round EVERY product to the format (toward zero, wrapped) and add the rounded products exactly in
  64 bits before one final wrap: the result does not depend on the order of the sum, so a tiled or parallel reduction
  gives the same bits as a serial one.
* ``sqrt`` is the integer square root of ``raw << frac`` (floor); ``exp`` / ``exp2`` / ``ln`` / ``log2`` / ``sin`` / ``cos`` /
  ``sigmoid`` / ``tanh`` are evaluated in Q30 with integer series after range reduction and are within 2 units in the last
  place for ``frac <= 24``; arguments <= 0 of a logarithm give the minimum value; ``exp`` saturates.
* ``softmax``, ``rmsnorm``, ``layer_norm``, ``FixedLinear`` and ``FixedMlp`` build a whole integer forward pass.
Reference counterpart: scirust-simd/src/fixed/{types,rounding,overflow,rescale,ops,math,transcendental,reductions,linalg,
activation,norm,layer,model}.rs.
"""
from __future__ import annotations

import torch

I32_MIN, I32_MAX = -(1 << 31), (1 << 31) - 1
ROUNDINGS = ("toward_zero", "floor", "ceil", "nearest_even")
OVERFLOWS = ("wrap", "saturate", "checked")
Q = 30
_LN2_Q60 = 799144290325165979
_PI_Q60 = 3622009729038561421
_LN2_Q = (_LN2_Q60 + (1 << 29)) >> 30
_LOG2E_Q = ((1 << 90) + _LN2_Q60 // 2) // _LN2_Q60                      # 2^30 / ln 2
_HALF_PI_Q = (_PI_Q60 + (1 << 30)) >> 31
_TWO_OVER_PI_Q = ((1 << 91) + _PI_Q60 // 2) // _PI_Q60


class FixedOverflow(ArithmeticError):
    pass


def round_shift(wide: torch.Tensor, frac: int, mode: str = "toward_zero") -> torch.Tensor:
    if frac == 0:
        return wide
    floor = wide >> frac
    rem = wide - (floor << frac)
    if mode == "floor":
        return floor
    if mode == "toward_zero":
        return floor + ((wide < 0) & (rem != 0)).to(wide.dtype)
    if mode == "ceil":
        return floor + (rem != 0).to(wide.dtype)
    if mode == "nearest_even":
        half = 1 << (frac - 1)
        return floor + ((rem > half) | ((rem == half) & ((floor & 1) == 1))).to(wide.dtype)
    raise ValueError(f"unknown rounding mode {mode!r}")


def narrow(wide: torch.Tensor, overflow: str = "wrap") -> torch.Tensor:
    if overflow == "wrap":
        return (((wide + (1 << 31)) & 0xFFFFFFFF) - (1 << 31)).to(torch.int32)     # two's-complement truncation, spelled out
    if overflow == "saturate":
        return wide.clamp(I32_MIN, I32_MAX).to(torch.int32)
    if overflow == "checked":
        if bool(((wide < I32_MIN) | (wide > I32_MAX)).any()):
            raise FixedOverflow("result does not fit 32 bits")
        return wide.to(torch.int32)
    raise ValueError(f"unknown overflow mode {overflow!r}")


def _isqrt(v: torch.Tensor) -> torch.Tensor:
    """Floor of the square root of non-negative int64 values below 2^62, bit by bit."""
    res = torch.zeros_like(v)
    rem = v.clone()
    for shift in range(60, -1, -2):
        bit = 1 << shift
        trial = res + bit
        take = rem >= trial
        rem = torch.where(take, rem - trial, rem)
        res = torch.where(take, (res >> 1) + bit, res >> 1)
    return res


def _mul_q(a: torch.Tensor, b) -> torch.Tensor:
    return (a * b + (1 << (Q - 1))) >> Q


def _mul_qc(a: torch.Tensor, c: int) -> torch.Tensor:
    """``round(a * c / 2^30)`` (half up) for |a| below 2^46 and a Q30 constant below 2^31, without leaving 64 bits: the
    high and low 16-bit parts of ``a`` are multiplied separately and recombined exactly."""
    hi, lo = a >> 16, a & 0xFFFF
    t = hi * c
    sh = Q - 16
    return (t >> sh) + ((((t & ((1 << sh) - 1)) << 16) + lo * c + (1 << (Q - 1))) >> Q)


def _series_coeffs(base_q60: int, terms: int, only=None):
    """c_n = base^n / n! in Q30 from exact integer arithmetic."""
    out, fact = [], 1
    for n in range(terms):
        fact = fact * max(n, 1)
        num = base_q60 ** n
        c = (num * (1 << Q) + (fact << (60 * n)) // 2) // (fact << (60 * n)) if n else 1 << Q
        out.append(c)
    return out


_EXP2_C = _series_coeffs(_LN2_Q60, 12)
_FACT_INV = _series_coeffs(1 << 60, 14)                                   # 1 / n! in Q30


def _exp2_core(y: torch.Tensor) -> torch.Tensor:
    """``y`` Q30 int64 -> 2^y in Q30, saturated to the int64 range that the caller narrows."""
    k = (y + (1 << (Q - 1))) >> Q
    f = y - (k << Q)
    acc = torch.full_like(f, _EXP2_C[-1])
    for c in reversed(_EXP2_C[:-1]):
        acc = _mul_q(acc, f) + c
    big = k > 31
    kk = k.clamp(-62, 31)
    return torch.where(big, torch.full_like(acc, 1 << 62), torch.where(kk >= 0, acc << kk.clamp_min(0), acc >> (-kk).clamp_min(0)))


def _log2_core(x: torch.Tensor) -> torch.Tensor:
    """``x`` positive Q30 int64 (below 2^62) -> log2(x) in Q30 through 2 atanh((m-1)/(m+1)) / ln 2 on the mantissa."""
    msb = torch.zeros_like(x)
    v = x.clone()
    for s in (32, 16, 8, 4, 2, 1):
        big = v >= (1 << s)
        msb = msb + big.to(x.dtype) * s
        v = torch.where(big, v >> s, v)
    k = msb - Q
    m = torch.where(k >= 0, x >> k.clamp_min(0), x << (-k).clamp_min(0))      # [2^30, 2^31)
    t = ((m - (1 << Q)) << Q) // (m + (1 << Q))                              # (m-1)/(m+1) in [0, 1/3)
    t2 = _mul_q(t, t)
    acc = torch.zeros_like(t)
    for n in range(25, 0, -2):
        acc = _mul_q(acc, t2) + ((1 << Q) + n // 2) // n
    ln_m = _mul_q(acc, t) * 2
    return (k << Q) + _mul_qc(ln_m, _LOG2E_Q)


def _sincos_core(x: torch.Tensor):
    m = (_mul_qc(x, _TWO_OVER_PI_Q) + (1 << (Q - 1))) >> Q
    r = x - m * _HALF_PI_Q
    r2 = _mul_q(r, r)
    s = torch.zeros_like(r)
    c = torch.zeros_like(r)
    for n in range(13, 0, -2):                                               # sin: r - r^3/3! + ...
        s = _FACT_INV[n] * (1 if (n // 2) % 2 == 0 else -1) + _mul_q(s, r2)
    s = _mul_q(s, r)
    for n in range(12, -1, -2):
        c = _FACT_INV[n] * (1 if (n // 2) % 2 == 0 else -1) + _mul_q(c, r2)
    quad = m & 3
    sin = torch.where(quad == 0, s, torch.where(quad == 1, c, torch.where(quad == 2, -s, -c)))
    cos = torch.where(quad == 0, c, torch.where(quad == 1, -s, torch.where(quad == 2, -c, s)))
    return sin, cos


class FixedTensor:
    __slots__ = ("raw", "frac")

    def __init__(self, raw: torch.Tensor, frac: int):
        if raw.dtype != torch.int32:
            raise TypeError("raw storage is int32")
        if not 0 <= frac <= 30:
            raise ValueError("0 <= frac <= 30")
        self.raw, self.frac = raw, frac

    # ---- construction / conversion
    @staticmethod
    def from_float(x, frac: int, rounding: str = "nearest_even", overflow: str = "checked") -> "FixedTensor":
        x = torch.as_tensor(x, dtype=torch.float64)
        if not bool(torch.isfinite(x).all()):
            raise FixedOverflow("only finite values convert")
        s = x * float(1 << frac)
        r = {"toward_zero": torch.trunc, "floor": torch.floor, "ceil": torch.ceil, "nearest_even": torch.round}[rounding](s)
        return FixedTensor(narrow(r.to(torch.int64), overflow), frac)

    @staticmethod
    def from_int(v, frac: int, overflow: str = "saturate") -> "FixedTensor":
        return FixedTensor(narrow(torch.as_tensor(v, dtype=torch.int64) << frac, overflow), frac)

    def to_float(self, dtype=torch.float64) -> torch.Tensor:
        return (self.raw.to(torch.float64) / float(1 << self.frac)).to(dtype)

    def one(self) -> int:
        return 1 << self.frac

    @property
    def shape(self):
        return self.raw.shape

    def to(self, device) -> "FixedTensor":
        return FixedTensor(self.raw.to(device), self.frac)

    def _wide(self):
        return self.raw.to(torch.int64)

    def _same(self, o: "FixedTensor"):
        if self.frac != o.frac:
            raise ValueError(f"formats differ (Q{self.frac} vs Q{o.frac}); rescale first")

    def _new(self, wide, overflow="wrap"):
        return FixedTensor(narrow(wide, overflow), self.frac)

    def __getitem__(self, idx):
        return FixedTensor(self.raw[idx], self.frac)

    def __eq__(self, o):
        return isinstance(o, FixedTensor) and self.frac == o.frac and torch.equal(self.raw, o.raw)

    # ---- exact ring operations
    def add(self, o, overflow="wrap"):
        self._same(o)
        return self._new(self._wide() + o._wide(), overflow)

    def sub(self, o, overflow="wrap"):
        self._same(o)
        return self._new(self._wide() - o._wide(), overflow)

    def neg(self, overflow="wrap"):
        return self._new(-self._wide(), overflow)

    def abs(self, overflow="wrap"):
        return self._new(self._wide().abs(), overflow)

    __add__, __sub__, __neg__ = add, sub, neg

    def mul(self, o, rounding="toward_zero", overflow="wrap"):
        self._same(o)
        return self._new(round_shift(self._wide() * o._wide(), self.frac, rounding), overflow)

    __mul__ = mul

    def div(self, o, rounding="toward_zero", overflow="checked"):
        """(self << frac) / o with the chosen rounding of the exact quotient; division by zero raises."""
        self._same(o)
        den = o._wide()
        if bool((den == 0).any()):
            raise ZeroDivisionError("fixed-point division by zero")
        num = self._wide() << self.frac
        q = torch.div(num, den, rounding_mode="floor")
        rem = num - q * den                                                  # same sign as den, |rem| < |den|
        if rounding == "floor":
            pass
        elif rounding == "ceil":
            q = q + (rem != 0).to(q.dtype)
        elif rounding == "toward_zero":
            q = q + ((rem != 0) & ((num < 0) != (den < 0))).to(q.dtype)
        elif rounding == "nearest_even":
            twice, d = (rem * 2).abs(), den.abs()
            q = q + ((twice > d) | ((twice == d) & ((q & 1) == 1))).to(q.dtype)
        else:
            raise ValueError(f"unknown rounding mode {rounding!r}")
        return self._new(q, overflow)

    def rescale(self, frac: int, rounding="toward_zero", overflow="wrap") -> "FixedTensor":
        w = self._wide()
        w = w << (frac - self.frac) if frac >= self.frac else round_shift(w, self.frac - frac, rounding)
        return FixedTensor(narrow(w, overflow), frac)

    # ---- order-independent reductions
    def sum(self, dim=-1):
        return self._new(self._wide().sum(dim))

    def l1_norm(self, dim=-1):
        return self._new(self._wide().abs().sum(dim))

    def dot(self, o, dim=-1):
        self._same(o)
        p = narrow(round_shift(self._wide() * o._wide(), self.frac, "toward_zero")).to(torch.int64)
        return self._new(p.sum(dim))

    def matmul(self, o, chunk: int = 64):
        """``[.., M, K] @ [K, N]``: per-product rounding, exact 64-bit sum; K is walked in chunks to bound memory."""
        self._same(o)
        a, b = self._wide(), o._wide()
        acc = torch.zeros(*a.shape[:-1], b.shape[-1], dtype=torch.int64, device=a.device)
        for k0 in range(0, a.shape[-1], chunk):
            p = a[..., k0:k0 + chunk, None] * b[k0:k0 + chunk, :]
            acc += narrow(round_shift(p, self.frac, "toward_zero")).to(torch.int64).sum(-2)
        return self._new(acc)

    __matmul__ = matmul

    def max(self, dim=-1):
        return FixedTensor(self.raw.max(dim).values, self.frac)

    def argmax(self, dim=-1):
        return self.raw.argmax(dim)

    def mean(self, dim=-1):
        n = self.raw.shape[dim]
        s = self._wide().sum(dim)
        return self._new(torch.div(s.abs(), n, rounding_mode="floor") * s.sign())     # toward zero

    # ---- element-wise functions
    def relu(self):
        return FixedTensor(self.raw.clamp_min(0), self.frac)

    def clamp(self, lo: float, hi: float):
        f = float(1 << self.frac)
        return FixedTensor(self.raw.clamp(int(round(lo * f)), int(round(hi * f))), self.frac)

    def relu6(self):
        return self.clamp(0.0, 6.0)

    def hardsigmoid(self):
        """clamp(x / 6 + 1/2, 0, 1), the division rounded toward zero."""
        w = self._wide() + 3 * self.one()
        q = torch.div(w.abs(), 6, rounding_mode="floor") * w.sign()
        return FixedTensor(q.clamp(0, self.one()).to(torch.int32), self.frac)

    def sqrt(self):
        w = (self._wide().clamp_min(0)) << self.frac
        return self._new(_isqrt(w), "saturate")

    def reciprocal(self):
        return FixedTensor(torch.full_like(self.raw, self.one()), self.frac).div(self)

    def rsqrt(self):
        return self.sqrt().reciprocal()

    def _to_q(self):
        return self._wide() << (Q - self.frac)

    def _from_q(self, v):
        sh = Q - self.frac
        r = v if sh == 0 else (v + (1 << (sh - 1))) >> sh
        return self._new(r, "saturate")

    def exp2(self):
        return self._from_q(_exp2_core(self._to_q()))

    def exp(self):
        return self._from_q(_exp2_core(_mul_qc(self._to_q(), _LOG2E_Q)))

    def log2(self):
        pos = self.raw > 0
        v = _log2_core(torch.where(pos, self._to_q(), torch.full_like(self._wide(), 1 << Q)))
        out = self._from_q(v)
        return FixedTensor(torch.where(pos, out.raw, torch.full_like(out.raw, I32_MIN)), self.frac)

    def ln(self):
        pos = self.raw > 0
        v = _mul_qc(_log2_core(torch.where(pos, self._to_q(), torch.full_like(self._wide(), 1 << Q))), _LN2_Q)
        out = self._from_q(v)
        return FixedTensor(torch.where(pos, out.raw, torch.full_like(out.raw, I32_MIN)), self.frac)

    def sin(self):
        return self._from_q(_sincos_core(self._to_q())[0])

    def cos(self):
        return self._from_q(_sincos_core(self._to_q())[1])

    def sigmoid(self):
        """1 / (1 + exp(-|x|)) evaluated on the stable side and mirrored."""
        q = self._to_q()
        e = _exp2_core(_mul_qc(-q.abs(), _LOG2E_Q))                           # (0, 1]
        s = ((1 << (2 * Q)) + ((1 << Q) + e) // 2) // ((1 << Q) + e)          # 1 / (1 + e) in [1/2, 1)
        return self._from_q(torch.where(q >= 0, s, (1 << Q) - s))

    def tanh(self):
        q = (self._to_q() * 2).clamp(-(40 << Q), 40 << Q)
        e = _exp2_core(_mul_qc(-q.abs(), _LOG2E_Q))
        s = ((1 << (2 * Q)) + ((1 << Q) + e) // 2) // ((1 << Q) + e)
        s = torch.where(q >= 0, s, (1 << Q) - s)
        return self._from_q(2 * s - (1 << Q))

    def silu(self):
        return self.mul(self.sigmoid())

    def softmax(self, dim=-1):
        """exp of the max-shifted input (so every term is at most one), divided by the exact sum, nearest rounding."""
        q = self._to_q()
        e = _exp2_core(_mul_qc(q - q.max(dim, keepdim=True).values, _LOG2E_Q))
        total = e.sum(dim, keepdim=True)
        return self._from_q(((e << Q) + total // 2) // total)


# ------------------------------------------------------------------ normalisation and layers
def rmsnorm(x: FixedTensor, gamma: FixedTensor, eps: float = 1e-5) -> FixedTensor:
    ms = x.mul(x).mean(-1)
    inv = ms.add(FixedTensor.from_float(torch.full_like(ms.raw, eps, dtype=torch.float64), x.frac, "ceil")).rsqrt()
    return x.mul(FixedTensor(inv.raw[..., None].expand_as(x.raw).contiguous(), x.frac)).mul(_expand(gamma, x))


def layer_norm(x: FixedTensor, gamma: FixedTensor, beta: FixedTensor, eps: float = 1e-5) -> FixedTensor:
    mu = x.mean(-1)
    c = x.sub(FixedTensor(mu.raw[..., None].expand_as(x.raw).contiguous(), x.frac))
    var = c.mul(c).mean(-1)
    inv = var.add(FixedTensor.from_float(torch.full_like(var.raw, eps, dtype=torch.float64), x.frac, "ceil")).rsqrt()
    return c.mul(FixedTensor(inv.raw[..., None].expand_as(x.raw).contiguous(), x.frac)).mul(_expand(gamma, x)).add(_expand(beta, x))


def _expand(p: FixedTensor, like: FixedTensor) -> FixedTensor:
    return FixedTensor(p.raw.expand_as(like.raw).contiguous(), p.frac)


class FixedLinear:
    def __init__(self, weight: FixedTensor, bias: FixedTensor | None):
        self.weight, self.bias = weight, bias                                 # weight [in, out]

    @staticmethod
    def from_float(linear: torch.nn.Linear, frac: int) -> "FixedLinear":
        w = FixedTensor.from_float(linear.weight.detach().t().contiguous(), frac)
        b = FixedTensor.from_float(linear.bias.detach(), frac) if linear.bias is not None else None
        return FixedLinear(w, b)

    def __call__(self, x: FixedTensor) -> FixedTensor:
        y = x.matmul(self.weight)
        return y.add(_expand(self.bias, y)) if self.bias is not None else y


class FixedMlp:
    """Integer forward pass of a ``torch.nn.Sequential`` of Linear / ReLU / Sigmoid / Tanh / SiLU / Softmax layers."""

    _ACT = {torch.nn.ReLU: "relu", torch.nn.Sigmoid: "sigmoid", torch.nn.Tanh: "tanh", torch.nn.SiLU: "silu",
            torch.nn.Softmax: "softmax", torch.nn.ReLU6: "relu6", torch.nn.Hardsigmoid: "hardsigmoid"}

    def __init__(self, layers, frac: int):
        self.layers, self.frac = layers, frac

    @staticmethod
    def from_float(seq, frac: int = 16) -> "FixedMlp":
        layers = []
        for m in seq:
            if isinstance(m, torch.nn.Linear):
                layers.append(FixedLinear.from_float(m, frac))
            elif type(m) in FixedMlp._ACT:
                layers.append(FixedMlp._ACT[type(m)])
            else:
                raise ValueError(f"unsupported module {type(m).__name__}")
        return FixedMlp(layers, frac)

    def to(self, device):
        for l in self.layers:
            if isinstance(l, FixedLinear):
                l.weight = l.weight.to(device)
                l.bias = l.bias.to(device) if l.bias is not None else None
        return self

    def __call__(self, x) -> FixedTensor:
        h = x if isinstance(x, FixedTensor) else FixedTensor.from_float(x, self.frac, overflow="saturate")
        for l in self.layers:
            h = l(h) if isinstance(l, FixedLinear) else getattr(h, l)()
        return h

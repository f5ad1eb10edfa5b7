"""Order-independent, correctly rounded reductions (scirust-core/src/reproducible.rs:23-106 and the
Kulisch-style exact accumulator of scirust-core/src/exact_acc.rs:34-461).

``ExactAccumulator`` keeps the exact sum of fp32 (or fp64) values as an arbitrary-precision integer
scaled by 2^-1074 - the long-accumulator idea with Python integers as the register - so the result
does not depend on the order of insertion or on how partial accumulators were merged, and
``round_f32`` / ``round_f64`` return the correctly rounded value. This is the ``ExactSum`` combiner of
the tree all-reduce (topology-independent bits)."""
from __future__ import annotations

import math
import struct
from fractions import Fraction

import numpy as np

_SHIFT = 1074 + 64  # every finite double is an integer multiple of 2^-1074


class ExactAccumulator:
    __slots__ = ("acc", "nan", "pos_inf", "neg_inf")

    def __init__(self):
        self.acc, self.nan, self.pos_inf, self.neg_inf = 0, False, False, False

    def add(self, x: float) -> None:
        x = float(x)
        if math.isnan(x):
            self.nan = True
        elif math.isinf(x):
            if x > 0:
                self.pos_inf = True
            else:
                self.neg_inf = True
        elif x != 0.0:
            m, e = math.frexp(x)                      # x = m * 2^e, 0.5 <= |m| < 1
            self.acc += int(m * (1 << 53)) << (e - 53 + _SHIFT) if e - 53 + _SHIFT >= 0 else 0

    def add_all(self, xs) -> "ExactAccumulator":
        for v in np.asarray(xs, dtype=np.float64).reshape(-1).tolist():
            self.add(v)
        return self

    def add_product(self, a: float, b: float) -> None:
        """Exact a*b of two fp32 values (the product of two 24-bit significands fits a double)."""
        self.add(float(np.float32(a)) * float(np.float32(b)))

    def merge(self, other: "ExactAccumulator") -> None:
        self.acc += other.acc
        self.nan |= other.nan
        self.pos_inf |= other.pos_inf
        self.neg_inf |= other.neg_inf

    def _special(self):
        if self.nan or (self.pos_inf and self.neg_inf):
            return float("nan")
        if self.pos_inf:
            return float("inf")
        if self.neg_inf:
            return float("-inf")
        return None

    def round_f64(self) -> float:
        s = self._special()
        if s is not None:
            return s
        return float(Fraction(self.acc, 1 << _SHIFT))   # Fraction -> float is correctly rounded

    def round_f32(self) -> float:
        s = self._special()
        if s is not None:
            return s
        fr = Fraction(self.acc, 1 << _SHIFT)
        if fr == 0:
            return 0.0
        d = float(fr)
        f = np.float32(d)
        # double rounding guard: if d sits exactly between two floats, decide with the exact value
        lo, hi = np.nextafter(f, np.float32(-np.inf)), np.nextafter(f, np.float32(np.inf))
        best = min((lo, f, hi), key=lambda c: (abs(Fraction(float(c)) - fr), int(_bits32(c)) & 1))
        return float(best)

    def to_bytes(self) -> bytes:
        flags = (1 if self.nan else 0) | (2 if self.pos_inf else 0) | (4 if self.neg_inf else 0)
        mag = abs(self.acc)
        body = mag.to_bytes((mag.bit_length() + 7) // 8 or 1, "little")
        return struct.pack("<BBI", flags, 1 if self.acc < 0 else 0, len(body)) + body

    @staticmethod
    def from_bytes(b: bytes) -> "ExactAccumulator":
        flags, neg, n = struct.unpack_from("<BBI", b, 0)
        if len(b) != 6 + n:
            raise ValueError("malformed accumulator frame")
        a = ExactAccumulator()
        a.acc = int.from_bytes(b[6:6 + n], "little") * (-1 if neg else 1)
        a.nan, a.pos_inf, a.neg_inf = bool(flags & 1), bool(flags & 2), bool(flags & 4)
        return a


def _bits32(x) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def reproducible_sum(xs) -> float:
    """Correctly rounded fp32 sum, independent of summation order."""
    return ExactAccumulator().add_all(np.asarray(xs, dtype=np.float32)).round_f32()


def reproducible_dot(a, b) -> float:
    acc = ExactAccumulator()
    for x, y in zip(np.asarray(a, dtype=np.float32).reshape(-1).tolist(), np.asarray(b, dtype=np.float32).reshape(-1).tolist()):
        acc.add_product(x, y)
    return acc.round_f32()

"""One-dimensional interpolation on tensors: every interpolant is fitted once (knots ``x [n]`` strictly increasing, values
``y [..., n]`` with any leading batch axes) and evaluated at a whole tensor of query points with one ``searchsorted``.

``LinearInterp``, ``NearestInterp``, ``CubicSpline`` (natural or not-a-knot ends; the tridiagonal system is solved for all
batch rows at once), ``Pchip`` (Fritsch-Carlson monotone slopes: no overshoot), ``Akima`` (slopes from weighted neighbouring
secants: robust to outliers), ``Barycentric`` (polynomial through all points in the numerically stable barycentric form;
Chebyshev nodes recommended). Outside the knots: piecewise forms extrapolate with their end polynomial unless
``clamp=True`` holds the end values.
Reference counterpart: scirust-interp/src/{linear,nearest,spline,pchip,akima,barycentric}.rs.
"""
from __future__ import annotations

import torch

D = torch.float64


def _knots(x, y):
    x = torch.as_tensor(x, dtype=D).reshape(-1)
    y = torch.as_tensor(y, dtype=D)
    if x.numel() < 2 or y.shape[-1] != x.numel():
        raise ValueError("need at least two knots and one value per knot")
    if bool((x[1:] <= x[:-1]).any()):
        raise ValueError("knots must be strictly increasing")
    return x, y


def _segment(x, q):
    return (torch.searchsorted(x, q.contiguous(), right=True) - 1).clamp(0, x.numel() - 2)


class _Piecewise:
    """Cubic Hermite pieces from knot values and slopes."""

    def __init__(self, x, y, slopes, clamp=False):
        self.x, self.y, self.m, self.clamp = x, y, slopes, clamp

    def __call__(self, q):
        q = torch.as_tensor(q, dtype=D)
        qq = q.clamp(self.x[0], self.x[-1]) if self.clamp else q
        i = _segment(self.x, qq.reshape(-1))
        h = self.x[i + 1] - self.x[i]
        t = (qq.reshape(-1) - self.x[i]) / h
        y0, y1, m0, m1 = self.y[..., i], self.y[..., i + 1], self.m[..., i], self.m[..., i + 1]
        t2, t3 = t * t, t * t * t
        out = (2 * t3 - 3 * t2 + 1) * y0 + (t3 - 2 * t2 + t) * h * m0 + (-2 * t3 + 3 * t2) * y1 + (t3 - t2) * h * m1
        return out.reshape(tuple(self.y.shape[:-1]) + tuple(q.shape))

    def derivative(self, q):
        q = torch.as_tensor(q, dtype=D)
        i = _segment(self.x, q.reshape(-1))
        h = self.x[i + 1] - self.x[i]
        t = (q.reshape(-1) - self.x[i]) / h
        y0, y1, m0, m1 = self.y[..., i], self.y[..., i + 1], self.m[..., i], self.m[..., i + 1]
        out = ((6 * t * t - 6 * t) * (y0 - y1)) / h + (3 * t * t - 4 * t + 1) * m0 + (3 * t * t - 2 * t) * m1
        return out.reshape(tuple(self.y.shape[:-1]) + tuple(q.shape))


class LinearInterp:
    def __init__(self, x, y, clamp: bool = False):
        self.x, self.y = _knots(x, y)
        self.clamp = clamp

    def __call__(self, q):
        q = torch.as_tensor(q, dtype=D)
        qq = q.clamp(self.x[0], self.x[-1]) if self.clamp else q
        i = _segment(self.x, qq.reshape(-1))
        t = (qq.reshape(-1) - self.x[i]) / (self.x[i + 1] - self.x[i])
        return (self.y[..., i] + t * (self.y[..., i + 1] - self.y[..., i])).reshape(tuple(self.y.shape[:-1]) + tuple(q.shape))


class NearestInterp:
    def __init__(self, x, y):
        self.x, self.y = _knots(x, y)

    def __call__(self, q):
        q = torch.as_tensor(q, dtype=D)
        i = _segment(self.x, q.reshape(-1))
        pick = torch.where((q.reshape(-1) - self.x[i]) <= (self.x[i + 1] - q.reshape(-1)), i, i + 1)     # ties go left
        return self.y[..., pick].reshape(tuple(self.y.shape[:-1]) + tuple(q.shape))


class CubicSpline(_Piecewise):
    def __init__(self, x, y, bc: str = "not-a-knot", clamp: bool = False):
        x, y = _knots(x, y)
        n = x.numel()
        h = x[1:] - x[:-1]
        d = (y[..., 1:] - y[..., :-1]) / h
        if n == 2 or (n == 3 and bc == "not-a-knot"):                          # too few knots: the parabola / line through them
            if n == 2:
                m = torch.stack([d[..., 0], d[..., 0]], -1)
            else:
                dd = (d[..., 1] - d[..., 0]) / (x[2] - x[0])
                m = torch.stack([d[..., 0] - dd * h[0], d[..., 0] + dd * h[0], d[..., 1] + dd * h[1]], -1)
            super().__init__(x, y, m, clamp)
            return
        a = torch.zeros(n, n, dtype=D)
        rhs = torch.zeros(*y.shape[:-1], n, dtype=D)
        for i in range(1, n - 1):                                             # continuity of the second derivative
            a[i, i - 1], a[i, i], a[i, i + 1] = h[i], 2 * (h[i - 1] + h[i]), h[i - 1]
            rhs[..., i] = 3 * (h[i] * d[..., i - 1] + h[i - 1] * d[..., i])
        if bc == "natural":
            a[0, 0], a[0, 1] = 2.0, 1.0
            rhs[..., 0] = 3 * d[..., 0]
            a[-1, -1], a[-1, -2] = 2.0, 1.0
            rhs[..., -1] = 3 * d[..., -1]
        elif bc == "not-a-knot":                                              # third derivative continuous at the 2nd and the 2nd-last knot
            a[0, 0], a[0, 1] = h[1], h[0] + h[1]
            rhs[..., 0] = ((3 * h[0] + 2 * h[1]) * h[1] * d[..., 0] + h[0] ** 2 * d[..., 1]) / (h[0] + h[1])
            a[-1, -1], a[-1, -2] = h[-2], h[-1] + h[-2]
            rhs[..., -1] = ((3 * h[-1] + 2 * h[-2]) * h[-2] * d[..., -1] + h[-1] ** 2 * d[..., -2]) / (h[-1] + h[-2])
        else:
            raise ValueError("bc is 'natural' or 'not-a-knot'")
        m = torch.linalg.solve(a, rhs[..., None])[..., 0]
        super().__init__(x, y, m, clamp)


class Pchip(_Piecewise):
    def __init__(self, x, y, clamp: bool = False):
        x, y = _knots(x, y)
        h = x[1:] - x[:-1]
        d = (y[..., 1:] - y[..., :-1]) / h
        n = x.numel()
        m = torch.zeros_like(y)
        if n == 2:
            m[..., 0] = m[..., 1] = d[..., 0]
        else:
            w1, w2 = 2 * h[1:] + h[:-1], h[1:] + 2 * h[:-1]
            same = (d[..., :-1] * d[..., 1:]) > 0
            harm = (w1 + w2) / (w1 / d[..., :-1].where(same, torch.ones_like(d[..., :-1])) + w2 / d[..., 1:].where(same, torch.ones_like(d[..., 1:])))
            m[..., 1:-1] = torch.where(same, harm, torch.zeros_like(harm))
            m[..., 0] = self._end(h[0], h[1], d[..., 0], d[..., 1])
            m[..., -1] = self._end(h[-1], h[-2], d[..., -1], d[..., -2])
        super().__init__(x, y, m, clamp)

    @staticmethod
    def _end(h0, h1, d0, d1):
        m = ((2 * h0 + h1) * d0 - h0 * d1) / (h0 + h1)
        m = torch.where(torch.sign(m) != torch.sign(d0), torch.zeros_like(m), m)
        return torch.where((torch.sign(d0) != torch.sign(d1)) & (m.abs() > 3 * d0.abs()), 3 * d0, m)


class Akima(_Piecewise):
    def __init__(self, x, y, clamp: bool = False):
        x, y = _knots(x, y)
        if x.numel() < 3:
            raise ValueError("Akima interpolation needs at least three knots")
        d = (y[..., 1:] - y[..., :-1]) / (x[1:] - x[:-1])
        left1 = 2 * d[..., :1] - d[..., 1:2]
        left2 = 2 * left1 - d[..., :1]
        right1 = 2 * d[..., -1:] - d[..., -2:-1]
        right2 = 2 * right1 - d[..., -1:]
        e = torch.cat([left2, left1, d, right1, right2], -1)                   # secants with two extrapolated on each side
        w1, w2 = (e[..., 3:] - e[..., 2:-1]).abs(), (e[..., 1:-2] - e[..., :-3]).abs()
        flat = (w1 + w2) < 1e-12 * (1 + e.abs().amax(-1, keepdim=True))
        m = torch.where(flat, 0.5 * (e[..., 1:-2] + e[..., 2:-1]), (w1 * e[..., 1:-2] + w2 * e[..., 2:-1]) / (w1 + w2).clamp_min(1e-300))
        super().__init__(x, y, m, clamp)


class Barycentric:
    def __init__(self, x, y):
        x = torch.as_tensor(x, dtype=D).reshape(-1)
        self.y = torch.as_tensor(y, dtype=D)
        if len(set(x.tolist())) != x.numel() or self.y.shape[-1] != x.numel():
            raise ValueError("nodes must be distinct, one value per node")
        diff = x[:, None] - x[None, :]
        diff.fill_diagonal_(1.0)
        scale = 4.0 / (x.max() - x.min())                                     # capacity scaling keeps the weights in range
        self.w = 1.0 / torch.prod(diff * scale, 1)
        self.x = x

    def __call__(self, q):
        q = torch.as_tensor(q, dtype=D)
        d = q.reshape(-1, 1) - self.x[None, :]
        hit = d == 0
        safe = torch.where(hit, torch.ones_like(d), d)
        t = self.w / safe
        val = (t @ self.y.reshape(-1, self.x.numel()).t()) / t.sum(1, keepdim=True)
        exact = self.y.reshape(-1, self.x.numel()).t()[hit.float().argmax(1)]
        out = torch.where(hit.any(1, keepdim=True), exact, val).t()
        return out.reshape(tuple(self.y.shape[:-1]) + tuple(q.shape))


def chebyshev_nodes(n: int, a: float = -1.0, b: float = 1.0):
    k = torch.arange(n, dtype=D)
    return 0.5 * (a + b) - 0.5 * (b - a) * torch.cos((2 * k + 1) * torch.pi / (2 * n))

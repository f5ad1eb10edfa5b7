"""Rotations, rigid motions and hypercomplex algebras on batched tensors (last axis = components, leading axes = batch),
differentiable and device-agnostic, so a trajectory or a point cloud is transformed in one call.

Quaternions are ``(w, x, y, z)``; Euler angles are intrinsic Tait-Bryan Z-Y-X (yaw about z, then pitch about y, then roll
about x), with ``roll = 0`` at gimbal lock; ``slerp`` takes the shorter arc and falls back to a normalised lerp for nearly
parallel inputs; ``squad`` is Shoemake's spherical cubic with ``squad_setup`` tangents. Dual quaternions ``(real, dual)``
carry rigid motions: ``from_rotation_translation``, composition, point transform, screw parameters and ``sclerp``
(constant-speed screw interpolation). ``Se2`` is the planar rigid group. ``cayley_dickson_mul`` multiplies elements of
the 2^k-dimensional Cayley-Dickson algebras by recursion (complex, quaternion, octonion, sedenion): ``(a, b)(c, d) =
(ac - d* b, da + b c*)``. ``Dual`` numbers ``a + b eps`` (eps^2 = 0) give forward-mode derivatives of scalar code.
``MahonyAhrs`` fuses gyroscope and accelerometer (and optionally magnetometer) samples into an orientation with
proportional-integral feedback. ``bezier_cubic`` and ``catmull_rom`` are the usual curve evaluators.
Reference counterpart: scirust-simd/src/geometry/{quaternion,dual_quaternion,se2,transform,ahrs,curves}.rs and
scirust-simd/src/hypercomplex/{quat,octonion,sedenion,dual}.rs.
"""
from __future__ import annotations

import math

import torch

from .numerics.quaternion_search import q_conj, q_from_axis_angle, q_mul, q_normalize  # noqa: F401  (one definition)


def _t(x, dtype=torch.float64):
    return torch.as_tensor(x, dtype=dtype) if not isinstance(x, torch.Tensor) else x


# ------------------------------------------------------------------ quaternions
def q_identity(*batch, dtype=torch.float64):
    q = torch.zeros(*batch, 4, dtype=dtype)
    q[..., 0] = 1.0
    return q


def q_inverse(q):
    return q_conj(q) / (q * q).sum(-1, keepdim=True)


def q_rotate(q, v):
    """Rotate vectors ``v [..., 3]`` by unit quaternions: v + 2 w (u x v) + 2 u x (u x v)."""
    w, u = q[..., :1], q[..., 1:]
    t = 2.0 * torch.linalg.cross(u, v)
    return v + w * t + torch.linalg.cross(u, t)


def q_to_axis_angle(q):
    q = torch.where(q[..., :1] < 0, -q, q)
    s = q[..., 1:].norm(dim=-1, keepdim=True)
    angle = 2.0 * torch.atan2(s, q[..., :1])
    default = torch.zeros_like(q[..., 1:])
    default[..., 0] = 1.0
    return torch.where(s > 1e-12, q[..., 1:] / s.clamp_min(1e-300), default), angle[..., 0]


def q_to_matrix(q):
    w, x, y, z = q_normalize(q).unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
                        2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
                        2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], -1).reshape(*q.shape[:-1], 3, 3)


def q_from_matrix(m):
    """Shepperd's method: the largest of (trace, m00, m11, m22) picks the numerically safe branch."""
    m = _t(m)
    m00, m11, m22 = m[..., 0, 0], m[..., 1, 1], m[..., 2, 2]
    tr = m00 + m11 + m22
    cands = torch.stack([
        torch.stack([1 + tr, m[..., 2, 1] - m[..., 1, 2], m[..., 0, 2] - m[..., 2, 0], m[..., 1, 0] - m[..., 0, 1]], -1),
        torch.stack([m[..., 2, 1] - m[..., 1, 2], 1 + m00 - m11 - m22, m[..., 0, 1] + m[..., 1, 0], m[..., 0, 2] + m[..., 2, 0]], -1),
        torch.stack([m[..., 0, 2] - m[..., 2, 0], m[..., 0, 1] + m[..., 1, 0], 1 - m00 + m11 - m22, m[..., 1, 2] + m[..., 2, 1]], -1),
        torch.stack([m[..., 1, 0] - m[..., 0, 1], m[..., 0, 2] + m[..., 2, 0], m[..., 1, 2] + m[..., 2, 1], 1 - m00 - m11 + m22], -1)], -2)
    pick = torch.stack([tr, m00, m11, m22], -1).argmax(-1)
    q = torch.gather(cands, -2, pick[..., None, None].expand(*pick.shape, 1, 4))[..., 0, :]
    q = q_normalize(q)
    return torch.where(q[..., :1] < 0, -q, q)


def q_from_euler(roll, pitch, yaw):
    r, p, y = (_t(a) * 0.5 for a in (roll, pitch, yaw))
    cr, sr, cp, sp, cy, sy = r.cos(), r.sin(), p.cos(), p.sin(), y.cos(), y.sin()
    return torch.stack([cr * cp * cy + sr * sp * sy, sr * cp * cy - cr * sp * sy,
                        cr * sp * cy + sr * cp * sy, cr * cp * sy - sr * sp * cy], -1)


def q_to_euler(q):
    w, x, y, z = q_normalize(q).unbind(-1)
    sp = 2.0 * (w * y - z * x)
    lock = sp.abs() > 1.0 - 1e-3
    roll = torch.atan2(2 * (w * x + y * z), 1 - 2 * (x * x + y * y))
    pitch = torch.asin(sp.clamp(-1.0, 1.0))
    yaw = torch.atan2(2 * (w * z + x * y), 1 - 2 * (y * y + z * z))
    yaw_lock = torch.where(sp > 0, -2.0 * torch.atan2(x, w), 2.0 * torch.atan2(x, w))
    half_pi = torch.full_like(sp, math.pi / 2)
    return (torch.where(lock, torch.zeros_like(roll), roll), torch.where(lock, torch.copysign(half_pi, sp), pitch),
            torch.where(lock, yaw_lock, yaw))


def q_nlerp(a, b, t):
    t = _t(t, a.dtype)[..., None] if not isinstance(t, float) else t
    b = torch.where((a * b).sum(-1, keepdim=True) < 0, -b, b)
    return q_normalize(a + (b - a) * t)


def q_slerp(a, b, t):
    t = _t(t, a.dtype)
    t = t[..., None] if t.dim() else t
    d = (a * b).sum(-1, keepdim=True)
    b = torch.where(d < 0, -b, b)
    d = d.abs().clamp(max=1.0)
    th = torch.acos(d)
    s = torch.sin(th)
    near = s < 1e-6
    wa = torch.where(near, 1.0 - t, torch.sin((1.0 - t) * th) / s.clamp_min(1e-300))
    wb = torch.where(near, t + torch.zeros_like(d), torch.sin(t * th) / s.clamp_min(1e-300))
    return q_normalize(wa * a + wb * b)


def q_log(q):
    """Unit quaternion -> pure-vector logarithm ``[..., 3]`` (half the rotation vector)."""
    axis, angle = q_to_axis_angle(q)
    return axis * (angle[..., None] * 0.5)


def q_exp(v):
    th = v.norm(dim=-1, keepdim=True)
    return torch.cat([th.cos(), torch.where(th > 1e-12, v / th.clamp_min(1e-300) * th.sin(), v)], -1)


def q_squad_setup(q_prev, q, q_next):
    inv = q_conj(q)
    return q_mul(q, q_exp(-(q_log(q_mul(inv, q_prev)) + q_log(q_mul(inv, q_next))) * 0.25))


def q_squad(q0, q1, s0, s1, t):
    t = _t(t, q0.dtype)
    return q_slerp(q_slerp(q0, q1, t), q_slerp(s0, s1, t), 2.0 * t * (1.0 - t))


# ------------------------------------------------------------------ dual quaternions: rigid motions
def dq_from_rotation_translation(q, t):
    tq = torch.cat([torch.zeros_like(t[..., :1]), t], -1)
    return q, 0.5 * q_mul(tq, q)


def dq_identity(*batch):
    return q_identity(*batch), torch.zeros(*batch, 4, dtype=torch.float64)


def dq_mul(a, b):
    return q_mul(a[0], b[0]), q_mul(a[0], b[1]) + q_mul(a[1], b[0])


def dq_conjugate(a):
    return q_conj(a[0]), q_conj(a[1])


def dq_normalize(a):
    n = a[0].norm(dim=-1, keepdim=True)
    r = a[0] / n
    d = a[1] / n
    return r, d - r * (r * d).sum(-1, keepdim=True)                        # real . dual = 0 for a rigid motion


def dq_to_rotation_translation(a):
    r, d = dq_normalize(a)
    return r, 2.0 * q_mul(d, q_conj(r))[..., 1:]


def dq_transform_point(a, p):
    r, t = dq_to_rotation_translation(a)
    return q_rotate(r, p) + t


def dq_to_screw(a):
    """-> (axis l, moment m, angle theta, pitch displacement d): rotate by theta about the line (l, m), slide by d."""
    r, t = dq_to_rotation_translation(a)
    l, theta = q_to_axis_angle(r)
    d = (t * l).sum(-1)
    half = theta[..., None] * 0.5
    cot = torch.where(half.sin().abs() > 1e-9, half.cos() / half.sin().clamp_min(1e-300), torch.zeros_like(half))
    m = 0.5 * (torch.linalg.cross(t, l) + (t - d[..., None] * l) * cot)
    return l, m, theta, d


def dq_from_screw(l, m, theta, d):
    half, hd = _t(theta)[..., None] * 0.5, _t(d)[..., None] * 0.5
    real = torch.cat([half.cos(), l * half.sin()], -1)
    dual = torch.cat([-hd * half.sin(), m * half.sin() + l * hd * half.cos()], -1)
    return real, dual


def dq_pow(a, t):
    l, m, theta, d = dq_to_screw(a)
    pure = theta.abs() < 1e-9                                               # pure translation: the axis is the direction
    r, tr = dq_to_rotation_translation(a)
    out = dq_from_screw(l, m, theta * t, d * t)
    lin = dq_from_rotation_translation(r, tr * t)
    return torch.where(pure[..., None], lin[0], out[0]), torch.where(pure[..., None], lin[1], out[1])


def dq_sclerp(a, b, t):
    """a * (a^-1 b)^t: constant angular and linear speed along the screw joining two poses."""
    return dq_mul(a, dq_pow(dq_mul(dq_conjugate(a), b), t))


# ------------------------------------------------------------------ SE(2)
class Se2:
    def __init__(self, angle, translation):
        self.angle, self.translation = _t(angle), _t(translation)

    @staticmethod
    def identity():
        return Se2(0.0, [0.0, 0.0])

    def rotation_matrix(self):
        c, s = self.angle.cos(), self.angle.sin()
        return torch.stack([c, -s, s, c], -1).reshape(*self.angle.shape, 2, 2)

    def transform_vector(self, v):
        return (self.rotation_matrix() @ _t(v)[..., None])[..., 0]

    def transform_point(self, p):
        return self.transform_vector(p) + self.translation

    def compose(self, other: "Se2") -> "Se2":
        return Se2(self.angle + other.angle, self.transform_point(other.translation))

    def inverse(self) -> "Se2":
        inv = Se2(-self.angle, torch.zeros_like(self.translation))
        return Se2(-self.angle, -inv.transform_vector(self.translation))


# ------------------------------------------------------------------ Cayley-Dickson algebras
def cd_conj(a):
    out = -a
    out[..., 0] = a[..., 0]
    return out


def cayley_dickson_mul(a, b):
    """Product in the algebra of dimension ``a.shape[-1]`` (1, 2, 4, 8, 16, ...); the quaternion case agrees with
    ``q_mul``. Octonions are not associative and sedenions have zero divisors: that is the algebra, not a bug."""
    n = a.shape[-1]
    if n != b.shape[-1] or n & (n - 1):
        raise ValueError("both operands need the same power-of-two dimension")
    if n == 1:
        return a * b
    h = n // 2
    a0, a1, b0, b1 = a[..., :h], a[..., h:], b[..., :h], b[..., h:]
    return torch.cat([cayley_dickson_mul(a0, b0) - cayley_dickson_mul(cd_conj(b1), a1),
                      cayley_dickson_mul(b1, a0) + cayley_dickson_mul(a1, cd_conj(b0))], -1)


def cd_norm_sqr(a):
    return (a * a).sum(-1)


def cd_inverse(a):
    return cd_conj(a) / cd_norm_sqr(a)[..., None]


def cd_exp(a):
    """exp(s + v) = e^s (cos|v| + v/|v| sin|v|), valid in every Cayley-Dickson algebra (power-associative)."""
    s, v = a[..., :1], a[..., 1:]
    n = v.norm(dim=-1, keepdim=True)
    return s.exp() * torch.cat([n.cos(), torch.where(n > 1e-12, v / n.clamp_min(1e-300) * n.sin(), v)], -1)


def cd_ln(a):
    s, v = a[..., :1], a[..., 1:]
    n, r = v.norm(dim=-1, keepdim=True), a.norm(dim=-1, keepdim=True)
    return torch.cat([r.log(), torch.where(n > 1e-12, v / n.clamp_min(1e-300) * torch.atan2(n, s), v)], -1)


def cd_powf(a, p: float):
    return cd_exp(cd_ln(a) * p)


# ------------------------------------------------------------------ dual numbers (forward-mode derivative)
class Dual:
    __slots__ = ("re", "eps")

    def __init__(self, re, eps=0.0):
        self.re, self.eps = _t(re), _t(eps)

    @staticmethod
    def variable(x):
        return Dual(x, torch.ones_like(_t(x)))

    def _lift(self, o):
        return o if isinstance(o, Dual) else Dual(o, 0.0)

    def __add__(self, o):
        o = self._lift(o)
        return Dual(self.re + o.re, self.eps + o.eps)

    __radd__ = __add__

    def __sub__(self, o):
        o = self._lift(o)
        return Dual(self.re - o.re, self.eps - o.eps)

    def __rsub__(self, o):
        return self._lift(o) - self

    def __neg__(self):
        return Dual(-self.re, -self.eps)

    def __mul__(self, o):
        o = self._lift(o)
        return Dual(self.re * o.re, self.re * o.eps + self.eps * o.re)

    __rmul__ = __mul__

    def __truediv__(self, o):
        o = self._lift(o)
        return Dual(self.re / o.re, (self.eps * o.re - self.re * o.eps) / (o.re * o.re))

    def __rtruediv__(self, o):
        return self._lift(o) / self

    def exp(self):
        e = self.re.exp()
        return Dual(e, self.eps * e)

    def ln(self):
        return Dual(self.re.log(), self.eps / self.re)

    def sin(self):
        return Dual(self.re.sin(), self.eps * self.re.cos())

    def cos(self):
        return Dual(self.re.cos(), -self.eps * self.re.sin())

    def sqrt(self):
        r = self.re.sqrt()
        return Dual(r, self.eps / (2.0 * r))

    def powf(self, p: float):
        return Dual(self.re ** p, self.eps * p * self.re ** (p - 1.0))


# ------------------------------------------------------------------ attitude estimation
class MahonyAhrs:
    """Complementary filter with proportional-integral feedback: the measured gravity (and magnetic north) direction is
    compared with the one predicted by the current orientation, the cross-product error corrects the gyroscope rate
    (``kp``) and accumulates into a gyroscope bias estimate (``ki``). Orientation maps body to world coordinates."""

    def __init__(self, kp: float = 1.0, ki: float = 0.0):
        self.kp, self.ki = kp, ki
        self.reset()

    def reset(self):
        self.orientation = q_identity()
        self.bias = torch.zeros(3, dtype=torch.float64)

    def _apply(self, gyro, error, dt):
        self.bias = self.bias + self.ki * error * dt
        rate = _t(gyro) + self.kp * error + self.bias
        dq = q_mul(self.orientation, torch.cat([torch.zeros(1, dtype=torch.float64), rate])) * 0.5
        self.orientation = q_normalize(self.orientation + dq * dt)

    def update_imu(self, gyro, accel, dt: float):
        a = _t(accel)
        err = torch.zeros(3, dtype=torch.float64)
        if float(a.norm()) > 1e-12:
            up_body = q_rotate(q_conj(self.orientation), torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64))
            err = torch.linalg.cross(a / a.norm(), up_body)
        self._apply(gyro, err, dt)

    def update_marg(self, gyro, accel, mag, dt: float):
        a, m = _t(accel), _t(mag)
        err = torch.zeros(3, dtype=torch.float64)
        inv = q_conj(self.orientation)
        if float(a.norm()) > 1e-12:
            err = err + torch.linalg.cross(a / a.norm(), q_rotate(inv, torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64)))
        if float(m.norm()) > 1e-12:
            mw = q_rotate(self.orientation, m / m.norm())
            ref = torch.stack([torch.hypot(mw[0], mw[1]), torch.zeros((), dtype=torch.float64), mw[2]])   # north in the x-z plane
            err = err + torch.linalg.cross(m / m.norm(), q_rotate(inv, ref))
        self._apply(gyro, err, dt)


# ------------------------------------------------------------------ curves
def bezier_cubic(p0, p1, p2, p3, t):
    t = _t(t)[..., None]
    u = 1.0 - t
    return u ** 3 * p0 + 3 * u * u * t * p1 + 3 * u * t * t * p2 + t ** 3 * p3


def bezier_cubic_tangent(p0, p1, p2, p3, t):
    t = _t(t)[..., None]
    u = 1.0 - t
    return 3 * u * u * (p1 - p0) + 6 * u * t * (p2 - p1) + 3 * t * t * (p3 - p2)


def catmull_rom(p0, p1, p2, p3, t):
    """Uniform Catmull-Rom segment from p1 (t = 0) to p2 (t = 1)."""
    t = _t(t)[..., None]
    return 0.5 * (2 * p1 + (p2 - p0) * t + (2 * p0 - 5 * p1 + 4 * p2 - p3) * t * t + (3 * p1 - p0 - 3 * p2 + p3) * t ** 3)

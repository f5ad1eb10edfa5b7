"""Sequence-mixing primitives in their two equivalent forms: the recurrence (one state update per token: what a
decoder runs) and the parallel form (matrix products over the whole sequence: what training runs). Each pair is
tested to agree; the layers of ``nn/zoo.py`` are thin parameterisations on top of them.

  retention               S_t = g S_{t-1} + k_t^T v_t,  o_t = q_t S_t            | (Q K^T * D) V, D_ij = g^(i-j) [i >= j]
  gated_linear_attention  S_t = diag(a_t) S_{t-1} + k_t^T v_t                    | cumulative log-gates
  delta_rule              S_t = S_{t-1} (I - b_t k_t^T k_t) + b_t k_t^T v_t      | triangular solve (UT transform)
  selective_scan          h_t = exp(dt_t A) h_{t-1} + dt_t B_t x_t, y_t = C_t h_t | associative scan over (a, b) pairs
  ssd_dual                scalar-decay state space (Mamba-2)                     | masked (C B^T * L) X, L from cumulative decay
  s4_scan / s5_scan       diagonal linear state space                            | parallel prefix over (A, Bu) pairs
  hgrn                    h_t = f_t h_{t-1} + (1 - f_t) c_t                      | same associative scan
  rwkv_wkv                time-decayed key-weighted average with a bonus for the current token
  slstm_scan / mlstm_scan exponential-gated scalar / matrix memories with the stabiliser state
  hyena_long_conv         causal convolution with a sequence-long filter         | FFT
  alibi_slopes / alibi_bias   linear attention biases

Counterparts: scirust-core/src/nn/nd_layers.rs:201-230 (ALiBi), :887 delta_rule, :969 selective_scan, :1092 s4_scan,
:1328 retention, :1400 gated_linear_attention, :1475 hgrn, :1546 rwkv_wkv, :1691 slstm_scan, :1736 mlstm_scan,
:1832 hyena_long_conv, :1999 ssd_dual, :2129-2190 s5_scan / s5_parallel_scan. Shapes: ``[T, d]`` per head unless said.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------------------------ ALiBi
def alibi_slopes(n_heads: int) -> torch.Tensor:
    """Geometric slopes 2^(-8 i / n) for a power-of-two head count; other counts interleave the next power's slopes."""
    def pow2(n):
        start = 2.0 ** (-8.0 / n)
        return [start ** (i + 1) for i in range(n)]
    if n_heads & (n_heads - 1) == 0:
        return torch.tensor(pow2(n_heads))
    p = 1 << (n_heads.bit_length() - 1)
    extra = pow2(2 * p)[0::2][: n_heads - p]
    return torch.tensor(pow2(p) + extra)


def alibi_bias(slopes: torch.Tensor, T: int) -> torch.Tensor:
    """``[H, T, T]`` additive bias: ``-slope * (i - j)`` for ``j <= i``, ``-inf`` above the diagonal."""
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).float()
    bias = -slopes[:, None, None] * dist.clamp(min=0)
    return bias.masked_fill(dist[None] < 0, float("-inf"))


# ------------------------------------------------------------------------------------------------ helpers
def _assoc_scan(a: torch.Tensor, b: torch.Tensor):
    """Inclusive scan of h_t = a_t * h_{t-1} + b_t (h_{-1} = 0) along dim 0 by recursive doubling:
    (a2, b2) o (a1, b1) = (a1 a2, a2 b1 + b2). log2(T) element-wise steps."""
    T = a.shape[0]
    A, B = a.clone(), b.clone()
    step = 1
    while step < T:
        A_prev = torch.cat([torch.ones_like(A[:step]), A[:-step]], 0)
        B_prev = torch.cat([torch.zeros_like(B[:step]), B[:-step]], 0)
        B = A * B_prev + B
        A = A * A_prev
        step *= 2
    return B


# ------------------------------------------------------------------------------------------------ retention
def retention_recurrent(q, k, v, gamma: float):
    S = torch.zeros(k.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = gamma * S + k[t][:, None] * v[t][None, :]
        out.append(q[t] @ S)
    return torch.stack(out)


def retention(q, k, v, gamma: float):
    T = q.shape[0]
    i = torch.arange(T)
    D = torch.where(i[:, None] >= i[None, :], gamma ** (i[:, None] - i[None, :]).clamp(min=0).to(q.dtype),
                    torch.zeros((), dtype=q.dtype))
    return ((q @ k.t()) * D) @ v


# ------------------------------------------------------------------------------------------------ GLA
def gla_recurrent(q, k, v, alpha):
    """alpha [T, dk] in (0, 1): per-key-channel forget gates."""
    S = torch.zeros(k.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = alpha[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(q[t] @ S)
    return torch.stack(out)


def gated_linear_attention(q, k, v, alpha):
    """Parallel form: with G_t = prod_{s<=t} alpha_s, o_t = sum_{j<=t} ((q_t * G_t) . (k_j / G_j)) v_j."""
    logG = torch.log(alpha).cumsum(0)
    qg, kg = q * torch.exp(logG), k * torch.exp(-logG)
    T = q.shape[0]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    return ((qg @ kg.t()) * mask) @ v


# ------------------------------------------------------------------------------------------------ delta rule
def delta_rule_recurrent(q, k, v, beta):
    S = torch.zeros(k.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = S - beta[t] * k[t][:, None] * (k[t] @ S)[None, :] + beta[t] * k[t][:, None] * v[t][None, :]
        out.append(q[t] @ S)
    return torch.stack(out)


def delta_rule(q, k, v, beta):
    """Parallel form: the written values u_t = b_t (v_t - sum_{j<t} (k_t . k_j) u_j) solve the unit lower-triangular
    system (I + tril(diag(b) K K^T, -1)) U = diag(b) V; then o = tril(Q K^T) U."""
    T = q.shape[0]
    A = torch.tril((beta[:, None] * (k @ k.t())), -1)
    U = torch.linalg.solve_triangular(torch.eye(T, dtype=q.dtype) + A, beta[:, None] * v, upper=False)
    return torch.tril(q @ k.t()) @ U


# ------------------------------------------------------------------------------------------------ state spaces
def selective_scan_recurrent(x, dt, A, B, C):
    """x, dt [T, d]; A [d, n]; B, C [T, n]."""
    h = torch.zeros(x.shape[1], A.shape[1], dtype=x.dtype)
    ys = []
    for t in range(x.shape[0]):
        h = torch.exp(dt[t][:, None] * A) * h + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(h @ C[t])
    return torch.stack(ys)


def selective_scan(x, dt, A, B, C):
    a = torch.exp(dt[:, :, None] * A[None])
    b = (dt * x)[:, :, None] * B[:, None, :]
    h = _assoc_scan(a, b)
    return torch.einsum("tdn,tn->td", h, C)


def ssd_dual_recurrent(x, a, B, C):
    """Mamba-2 head: scalar decay a_t in (0, 1] per step; x [T, p], B, C [T, n]."""
    h = torch.zeros(B.shape[1], x.shape[1], dtype=x.dtype)
    ys = []
    for t in range(x.shape[0]):
        h = a[t] * h + B[t][:, None] * x[t][None, :]
        ys.append(C[t] @ h)
    return torch.stack(ys)


def ssd_dual(x, a, B, C):
    """Quadratic dual: y = ((C B^T) * L) x with L_ij = prod_{j<s<=i} a_s for i >= j, built from cumulative logs."""
    la = torch.log(a).cumsum(0)
    T = x.shape[0]
    L = torch.exp(la[:, None] - la[None, :]) * torch.tril(torch.ones(T, T, dtype=x.dtype))
    return ((C @ B.t()) * L) @ x


def s4_scan(u, A, B, C, dt: float):
    """Diagonal S4 with zero-order hold: A, B, C [n] (complex or real), u [T]; returns y [T] (real part)."""
    Ab = torch.exp(dt * A)
    Bb = (Ab - 1) / A * B
    h = _assoc_scan(Ab[None, :].expand(u.shape[0], -1).clone(), Bb[None, :] * u[:, None].to(Bb.dtype))
    return (h * C[None, :]).sum(-1).real if h.is_complex() else (h * C[None, :]).sum(-1)


def s5_scan(u, lam, B, C):
    """S5 recurrence: x_t = diag(lam) x_{t-1} + B u_t, y_t = Re(C x_t); u [T, m], lam [n], B [n, m], C [p, n]."""
    x = torch.zeros(lam.shape[0], dtype=B.dtype)
    ys = []
    for t in range(u.shape[0]):
        x = lam * x + B @ u[t].to(B.dtype)
        ys.append(C @ x)
    y = torch.stack(ys)
    return y.real if y.is_complex() else y


def s5_parallel_scan(u, lam, B, C):
    Bu = u.to(B.dtype) @ B.t()
    h = _assoc_scan(lam[None, :].expand(u.shape[0], -1).clone(), Bu)
    y = h @ C.t()
    return y.real if y.is_complex() else y


def hgrn_recurrent(f, c):
    h = torch.zeros_like(c[0])
    out = []
    for t in range(c.shape[0]):
        h = f[t] * h + (1 - f[t]) * c[t]
        out.append(h)
    return torch.stack(out)


def hgrn(f, c):
    return _assoc_scan(f, (1 - f) * c)


# ------------------------------------------------------------------------------------------------ RWKV
def rwkv_wkv(w, u, k, v):
    """wkv_t = (sum_{i<t} e^{-(t-1-i) w + k_i} v_i + e^{u + k_t} v_t) / (same with v -> 1), per channel, computed with
    the running-maximum stabiliser so that no exponential overflows. w, u [d]; k, v [T, d]."""
    T, d = k.shape
    num = torch.zeros(d, dtype=k.dtype)
    den = torch.zeros(d, dtype=k.dtype)
    mx = torch.full((d,), -1e38, dtype=k.dtype)
    out = []
    for t in range(T):
        m1 = torch.maximum(mx, u + k[t])
        e1, e2 = torch.exp(mx - m1), torch.exp(u + k[t] - m1)
        out.append((e1 * num + e2 * v[t]) / (e1 * den + e2))
        m2 = torch.maximum(mx - w, k[t])
        e1, e2 = torch.exp(mx - w - m2), torch.exp(k[t] - m2)
        num, den, mx = e1 * num + e2 * v[t], e1 * den + e2, m2
    return torch.stack(out)


def rwkv_wkv_direct(w, u, k, v):
    """The defining sums, without stabiliser (small inputs only): the oracle of ``rwkv_wkv``."""
    T = k.shape[0]
    out = []
    for t in range(T):
        num = torch.exp(u + k[t]) * v[t]
        den = torch.exp(u + k[t])
        for i in range(t):
            e = torch.exp(-(t - 1 - i) * w + k[i])
            num, den = num + e * v[i], den + e
        out.append(num / den)
    return torch.stack(out)


# ------------------------------------------------------------------------------------------------ xLSTM
def slstm_scan(i_pre, f_pre, z, o):
    """Scalar-memory xLSTM cell with exponential input gate and the stabiliser m_t = max(f~_t + m_{t-1}, i~_t):
    c_t = f' c + i' z, n_t = f' n + i', h_t = o * c_t / n_t. All inputs [T, d] (z already tanh'ed, o already sigmoid)."""
    d = z.shape[1]
    c, n, m = torch.zeros(d), torch.zeros(d), torch.full((d,), -1e38)
    out = []
    for t in range(z.shape[0]):
        logf = torch.nn.functional.logsigmoid(f_pre[t])
        m_new = torch.maximum(logf + m, i_pre[t])
        fi, ii = torch.exp(logf + m - m_new), torch.exp(i_pre[t] - m_new)
        c, n, m = fi * c + ii * z[t], fi * n + ii, m_new
        out.append(o[t] * c / n)
    return torch.stack(out)


def mlstm_scan(q, k, v, i_pre, f_pre):
    """Matrix-memory xLSTM: C_t = f' C + i' v k^T, n_t = f' n + i' k, h_t = C_t q / max(|n_t . q|, e^{-m_t});
    q, k [T, dk] (k pre-scaled by 1/sqrt(dk)), v [T, dv], gates [T]."""
    dk, dv = k.shape[1], v.shape[1]
    C, n, m = torch.zeros(dv, dk), torch.zeros(dk), torch.tensor(-1e38)
    out = []
    for t in range(q.shape[0]):
        logf = torch.nn.functional.logsigmoid(f_pre[t])
        m_new = torch.maximum(logf + m, i_pre[t])
        fi, ii = torch.exp(logf + m - m_new), torch.exp(i_pre[t] - m_new)
        C = fi * C + ii * v[t][:, None] * k[t][None, :]
        n = fi * n + ii * k[t]
        m = m_new
        out.append((C @ q[t]) / torch.maximum((n @ q[t]).abs(), torch.exp(-m)))
    return torch.stack(out)


def mlstm_parallel(q, k, v, i_pre, f_pre):
    """Parallel form of ``mlstm_scan``: D_ij = exp(F_i - F_j + i~_j - m_i) for j <= i with F the cumulative log forget
    gates and m_i the row maximum of the exponent; h = ((Q K^T) * D) V / max(|row sum|, e^{-m})."""
    F = torch.nn.functional.logsigmoid(f_pre).cumsum(0)
    E = F[:, None] - F[None, :] + i_pre[None, :]
    T = q.shape[0]
    E = E.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
    m = E.max(1).values
    S = (q @ k.t()) * torch.exp(E - m[:, None])
    norm = torch.maximum(S.sum(1).abs(), torch.exp(-m))
    return (S @ v) / norm[:, None]


# ------------------------------------------------------------------------------------------------ Hyena
def hyena_long_conv(x, filt):
    """Causal convolution of x [T, d] with a filter of the same length per channel, by FFT (zero-padded to 2 T)."""
    T = x.shape[0]
    n = 2 * T
    y = torch.fft.irfft(torch.fft.rfft(x, n=n, dim=0) * torch.fft.rfft(filt, n=n, dim=0), n=n, dim=0)
    return y[:T]


def hyena_long_conv_direct(x, filt):
    T = x.shape[0]
    out = torch.zeros_like(x)
    for t in range(T):
        for s in range(t + 1):
            out[t] += filt[s] * x[t - s]
    return out

"""Model zoo beyond the transformer / vision families: recurrent, graph, generative, operator-learning
and linear-attention / state-space sequence layers, plus weight adapters.

Counterparts in the reference (scirust-core/src/nn): ``lstm.rs``, ``gcn.rs``, ``vae.rs``, ``kan.rs``,
``fno.rs``, ``deeponet.rs``, ``neural_ode.rs``, ``tt_linear.rs``, ``lora.rs`` (LoRA / DoRA) and the N-D
sequence layers of ``nd_layers.rs:20-2190`` (Llama block, DeltaNet, Mamba / Mamba2, S4 / S5, RetNet, GLA,
HGRN, RWKV, xLSTM, Hyena) with ``NdDecoderLM`` and its speculative heads (``nd_decoder.rs:23-615``).

Every layer is a ``torch.nn.Module`` over N-D tensors (``[batch, time, features]`` for sequence
layers), so autograd, the N-D optimizers and bf16/CUDA execution come from the framework layer. The
sequence layers are written as explicit recurrences (a scan over time), which is their definition;
they are reference implementations for parity and small models, not tuned kernels.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


# --------------------------------------------------------------------------- recurrent / graph / generative
class LSTM(nn.Module):
    """Single-layer LSTM, gates ordered (input, forget, cell, output); x: [B, T, in] -> [B, T, hidden]."""

    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.w_ih = nn.Linear(input_size, 4 * hidden_size)
        self.w_hh = nn.Linear(hidden_size, 4 * hidden_size, bias=False)

    def forward(self, x, state=None):
        B, T, _ = x.shape
        h, c = state if state is not None else (x.new_zeros(B, self.hidden_size), x.new_zeros(B, self.hidden_size))
        out = []
        xi = self.w_ih(x)
        for t in range(T):
            i, f, g, o = (xi[:, t] + self.w_hh(h)).chunk(4, -1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
            h = torch.sigmoid(o) * torch.tanh(c)
            out.append(h)
        return torch.stack(out, 1), (h, c)


class GCNLayer(nn.Module):
    """Kipf-Welling graph convolution: H' = D^-1/2 (A + I) D^-1/2 H W."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.lin = nn.Linear(in_features, out_features)

    @staticmethod
    def normalize_adjacency(adj: torch.Tensor) -> torch.Tensor:
        a = adj + torch.eye(adj.shape[0], dtype=adj.dtype, device=adj.device)
        d = a.sum(1).clamp_min(1e-12).rsqrt()
        return d[:, None] * a * d[None, :]

    def forward(self, h, adj_norm):
        return adj_norm @ self.lin(h)


class GCN(nn.Module):
    def __init__(self, in_features, hidden, n_classes):
        super().__init__()
        self.l1, self.l2 = GCNLayer(in_features, hidden), GCNLayer(hidden, n_classes)

    def forward(self, x, adj):
        a = GCNLayer.normalize_adjacency(adj)
        return self.l2(F.relu(self.l1(x, a)), a)


class VAE(nn.Module):
    """Gaussian VAE with the reparameterisation trick; ``loss`` = reconstruction + beta * KL."""

    def __init__(self, in_dim: int, hidden: int, latent: int):
        super().__init__()
        self.enc = nn.Linear(in_dim, hidden)
        self.mu, self.logvar = nn.Linear(hidden, latent), nn.Linear(hidden, latent)
        self.dec1, self.dec2 = nn.Linear(latent, hidden), nn.Linear(hidden, in_dim)

    def encode(self, x):
        h = F.relu(self.enc(x))
        return self.mu(h), self.logvar(h)

    def decode(self, z):
        return self.dec2(F.relu(self.dec1(z)))

    def forward(self, x, generator=None):
        mu, logvar = self.encode(x)
        eps = torch.randn(mu.shape, generator=generator, device=mu.device, dtype=mu.dtype)
        return self.decode(mu + eps * torch.exp(0.5 * logvar)), mu, logvar

    @staticmethod
    def loss(recon, x, mu, logvar, beta: float = 1.0):
        rec = F.mse_loss(recon, x, reduction="sum") / x.shape[0]
        kl = -0.5 * torch.sum(1 + logvar - mu.pow(2) - logvar.exp()) / x.shape[0]
        return rec + beta * kl


class KANLayer(nn.Module):
    """Kolmogorov-Arnold layer: every edge carries a learnable 1-D function, here a sum of ``grid``
    Gaussian radial basis functions plus a SiLU base term."""

    def __init__(self, in_features: int, out_features: int, grid: int = 8, span: float = 2.0):
        super().__init__()
        self.register_buffer("centers", torch.linspace(-span, span, grid))
        self.width = 2 * span / (grid - 1)
        self.coef = nn.Parameter(torch.randn(in_features, grid, out_features) * (1.0 / math.sqrt(in_features * grid)))
        self.base = nn.Linear(in_features, out_features)

    def forward(self, x):
        phi = torch.exp(-((x[..., None] - self.centers) / self.width) ** 2)        # [..., in, grid]
        return torch.einsum("...ig,igo->...o", phi, self.coef) + self.base(F.silu(x))


class SpectralConv1d(nn.Module):
    """Fourier layer: keep the lowest ``modes`` frequencies and mix channels per mode."""

    def __init__(self, in_c: int, out_c: int, modes: int):
        super().__init__()
        self.modes = modes
        scale = 1.0 / (in_c * out_c)
        self.weight = nn.Parameter(scale * torch.randn(in_c, out_c, modes, 2))

    def forward(self, x):                      # x: [B, C, N]
        xf = torch.fft.rfft(x.float(), dim=-1)
        w = torch.view_as_complex(self.weight.float())
        m = min(self.modes, xf.shape[-1])
        out = torch.zeros(x.shape[0], w.shape[1], xf.shape[-1], dtype=xf.dtype, device=x.device)
        out[..., :m] = torch.einsum("bim,iom->bom", xf[..., :m], w[..., :m])
        return torch.fft.irfft(out, n=x.shape[-1], dim=-1).to(x.dtype)


class FNO1d(nn.Module):
    def __init__(self, in_c=1, out_c=1, width=32, modes=12, n_layers=3):
        super().__init__()
        self.lift = nn.Conv1d(in_c, width, 1)
        self.spec = nn.ModuleList([SpectralConv1d(width, width, modes) for _ in range(n_layers)])
        self.skip = nn.ModuleList([nn.Conv1d(width, width, 1) for _ in range(n_layers)])
        self.proj = nn.Conv1d(width, out_c, 1)

    def forward(self, x):
        h = self.lift(x)
        for s, k in zip(self.spec, self.skip):
            h = F.gelu(s(h) + k(h))
        return self.proj(h)


class DeepONet(nn.Module):
    """G(u)(y) = sum_k branch_k(u) * trunk_k(y) + b."""

    def __init__(self, n_sensors: int, coord_dim: int, width: int = 64, p: int = 32):
        super().__init__()
        self.branch = nn.Sequential(nn.Linear(n_sensors, width), nn.Tanh(), nn.Linear(width, p))
        self.trunk = nn.Sequential(nn.Linear(coord_dim, width), nn.Tanh(), nn.Linear(width, p))
        self.bias = nn.Parameter(torch.zeros(1))

    def forward(self, u, y):                   # u: [B, sensors], y: [Q, coord] -> [B, Q]
        return self.branch(u) @ self.trunk(y).t() + self.bias


class NeuralODE(nn.Module):
    """dz/dt = f(z, t) integrated with fixed-step RK4 (gradients by backprop through the solver)."""

    def __init__(self, dim: int, hidden: int = 64, steps: int = 8):
        super().__init__()
        self.f = nn.Sequential(nn.Linear(dim + 1, hidden), nn.Tanh(), nn.Linear(hidden, dim))
        self.steps = steps

    def _rhs(self, z, t):
        return self.f(torch.cat([z, z.new_full(z.shape[:-1] + (1,), t)], -1))

    def forward(self, z, t0: float = 0.0, t1: float = 1.0):
        h = (t1 - t0) / self.steps
        t = t0
        for _ in range(self.steps):
            k1 = self._rhs(z, t)
            k2 = self._rhs(z + 0.5 * h * k1, t + 0.5 * h)
            k3 = self._rhs(z + 0.5 * h * k2, t + 0.5 * h)
            k4 = self._rhs(z + h * k3, t + h)
            z = z + (h / 6.0) * (k1 + 2 * k2 + 2 * k3 + k4)
            t += h
        return z


class TTLinear(nn.Module):
    """Linear layer whose weight is a tensor train: in = prod(in_modes), out = prod(out_modes),
    core k has shape [r_{k-1}, in_k, out_k, r_k]."""

    def __init__(self, in_modes, out_modes, rank: int = 4):
        super().__init__()
        assert len(in_modes) == len(out_modes)
        self.in_modes, self.out_modes = list(in_modes), list(out_modes)
        ranks = [1] + [rank] * (len(in_modes) - 1) + [1]
        self.cores = nn.ParameterList(
            [nn.Parameter(torch.randn(ranks[k], in_modes[k], out_modes[k], ranks[k + 1]) / math.sqrt(in_modes[k] * ranks[k]))
             for k in range(len(in_modes))])
        self.bias = nn.Parameter(torch.zeros(int(torch.tensor(out_modes).prod())))

    def full_weight(self):
        w = self.cores[0]                                        # [1, i0, o0, r1]
        for c in self.cores[1:]:
            w = torch.einsum("aior,rjps->aijops", w, c)
            a, i, j, o, p, s = w.shape
            w = w.reshape(a, i * j, o * p, s)
        return w[0, :, :, 0]                                     # [in, out]

    def forward(self, x):
        return x @ self.full_weight() + self.bias


class LoRALinear(nn.Module):
    """y = x W (frozen) + (alpha / r) x A B; ``dora=True`` re-normalises the columns of W + AB and
    scales them by a learned magnitude (DoRA)."""

    def __init__(self, base: nn.Linear, r: int = 8, alpha: float = 16.0, dora: bool = False):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.r, self.scale, self.dora = r, alpha / r, dora
        self.A = nn.Parameter(torch.randn(base.in_features, r) * (1.0 / math.sqrt(base.in_features)))
        self.B = nn.Parameter(torch.zeros(r, base.out_features))
        if dora:
            self.magnitude = nn.Parameter(base.weight.detach().t().norm(dim=0).clone())   # per output column

    def merged_weight(self):                                     # [in, out]
        w = self.base.weight.t() + self.scale * self.A @ self.B
        if self.dora:
            w = w / w.norm(dim=0, keepdim=True).clamp_min(1e-12) * self.magnitude
        return w

    def forward(self, x):
        y = x @ self.merged_weight()
        return y + self.base.bias if self.base.bias is not None else y


# --------------------------------------------------------------------------- sequence layers [B, T, D]
class RMSNormND(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def _rope(x, theta=10000.0):                     # x: [B, H, T, dh], interleaved pairs
    B, H, T, dh = x.shape
    inv = torch.pow(theta, -torch.arange(0, dh, 2, device=x.device, dtype=torch.float32) / dh)
    ang = torch.arange(T, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
    c, s = ang.cos()[None, None], ang.sin()[None, None]
    x0, x1 = x[..., 0::2].float(), x[..., 1::2].float()
    return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], -1).flatten(-2).to(x.dtype)


class LlamaBlock(nn.Module):
    """Pre-norm GQA attention with RoPE + SwiGLU MLP (the block of the SciAgent decoder, N-D form)."""

    def __init__(self, d_model, n_heads, n_kv_heads, d_ff, theta=10000.0):
        super().__init__()
        self.h, self.kv, self.dh, self.theta = n_heads, n_kv_heads, d_model // n_heads, theta
        self.n1, self.n2 = RMSNormND(d_model), RMSNormND(d_model)
        self.q = nn.Linear(d_model, n_heads * self.dh, bias=False)
        self.k = nn.Linear(d_model, n_kv_heads * self.dh, bias=False)
        self.v = nn.Linear(d_model, n_kv_heads * self.dh, bias=False)
        self.o = nn.Linear(n_heads * self.dh, d_model, bias=False)
        self.gate, self.up = nn.Linear(d_model, d_ff, bias=False), nn.Linear(d_model, d_ff, bias=False)
        self.down = nn.Linear(d_ff, d_model, bias=False)

    def forward(self, x):
        B, T, _ = x.shape
        h = self.n1(x)
        q = _rope(self.q(h).view(B, T, self.h, self.dh).transpose(1, 2), self.theta)
        k = _rope(self.k(h).view(B, T, self.kv, self.dh).transpose(1, 2), self.theta)
        v = self.v(h).view(B, T, self.kv, self.dh).transpose(1, 2)
        g = self.h // self.kv
        a = F.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, T, -1))
        h = self.n2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


class _Recurrent(nn.Module):
    """Helper: run ``self.step(x_t, state) -> (y_t, state)`` over time."""

    def init_state(self, x):
        raise NotImplementedError

    def forward(self, x, state=None):
        state = self.init_state(x) if state is None else state
        ys = []
        for t in range(x.shape[1]):
            y, state = self.step(x[:, t], state)
            ys.append(y)
        return torch.stack(ys, 1)


class RetNet(_Recurrent):
    """Retention: S_t = gamma S_{t-1} + k_t^T v_t, y_t = q_t S_t (single head per call)."""

    def __init__(self, d_model, gamma=0.97):
        super().__init__()
        self.q, self.k, self.v = (nn.Linear(d_model, d_model, bias=False) for _ in range(3))
        self.gamma = gamma

    def init_state(self, x):
        d = x.shape[-1]
        return x.new_zeros(x.shape[0], d, d)

    def step(self, xt, S):
        q, k, v = self.q(xt), self.k(xt) / math.sqrt(xt.shape[-1]), self.v(xt)
        S = self.gamma * S + k[:, :, None] * v[:, None, :]
        return torch.einsum("bd,bde->be", q, S), S

    def forward_parallel(self, x):
        """Training form: (Q K^T * decay mask) V per sequence, no loop over time (``sequence_scans.retention``)."""
        from .sequence_scans import retention
        q, k, v = self.q(x), self.k(x) / math.sqrt(x.shape[-1]), self.v(x)
        return torch.stack([retention(q[b], k[b], v[b], self.gamma) for b in range(x.shape[0])])


class GLA(_Recurrent):
    """Gated linear attention: data-dependent per-key decay alpha_t in (0, 1)."""

    def __init__(self, d_model):
        super().__init__()
        self.q, self.k, self.v, self.a = (nn.Linear(d_model, d_model, bias=False) for _ in range(4))

    def init_state(self, x):
        d = x.shape[-1]
        return x.new_zeros(x.shape[0], d, d)

    def step(self, xt, S):
        q, k, v = self.q(xt), self.k(xt) / math.sqrt(xt.shape[-1]), self.v(xt)
        alpha = torch.sigmoid(self.a(xt))
        S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
        return torch.einsum("bd,bde->be", q, S), S

    def forward_parallel(self, x):
        from .sequence_scans import gated_linear_attention
        q, k, v = self.q(x), self.k(x) / math.sqrt(x.shape[-1]), self.v(x)
        alpha = torch.sigmoid(self.a(x))
        return torch.stack([gated_linear_attention(q[b], k[b], v[b], alpha[b]) for b in range(x.shape[0])])


class DeltaNet(_Recurrent):
    """Delta rule: S_t = S_{t-1} + beta_t k_t^T (v_t - k_t S_{t-1}) with unit-norm keys."""

    def __init__(self, d_model):
        super().__init__()
        self.q, self.k, self.v = (nn.Linear(d_model, d_model, bias=False) for _ in range(3))
        self.beta = nn.Linear(d_model, 1)

    def init_state(self, x):
        d = x.shape[-1]
        return x.new_zeros(x.shape[0], d, d)

    def step(self, xt, S):
        q, v = self.q(xt), self.v(xt)
        k = F.normalize(self.k(xt), dim=-1)
        beta = torch.sigmoid(self.beta(xt))
        pred = torch.einsum("bd,bde->be", k, S)
        S = S + beta[:, :, None] * k[:, :, None] * (v - pred)[:, None, :]
        return torch.einsum("bd,bde->be", q, S), S

    def forward_parallel(self, x):
        """Training form: the written values come from one unit-triangular solve per sequence."""
        from .sequence_scans import delta_rule
        q, v = self.q(x), self.v(x)
        k = F.normalize(self.k(x), dim=-1)
        beta = torch.sigmoid(self.beta(x))[..., 0]
        return torch.stack([delta_rule(q[b], k[b], v[b], beta[b]) for b in range(x.shape[0])])


class HGRN(_Recurrent):
    """Hierarchically gated recurrence: h_t = f_t h_{t-1} + (1 - f_t) c_t, y_t = o_t * h_t, with a
    learned lower bound on the forget gate."""

    def __init__(self, d_model, lower_bound=0.0):
        super().__init__()
        self.f, self.c, self.o = (nn.Linear(d_model, d_model) for _ in range(3))
        self.lb = lower_bound

    def init_state(self, x):
        return x.new_zeros(x.shape[0], x.shape[-1])

    def step(self, xt, h):
        f = self.lb + (1 - self.lb) * torch.sigmoid(self.f(xt))
        h = f * h + (1 - f) * F.silu(self.c(xt))
        return torch.sigmoid(self.o(xt)) * h, h

    def forward_parallel(self, x):
        from .sequence_scans import hgrn
        f = self.lb + (1 - self.lb) * torch.sigmoid(self.f(x))
        h = hgrn(f.transpose(0, 1), F.silu(self.c(x)).transpose(0, 1)).transpose(0, 1)      # the scan runs along dim 0
        return torch.sigmoid(self.o(x)) * h


class Mamba2(nn.Module):
    """Mamba-2 mixer: heads of width ``head_dim`` share ONE scalar decay per step (a_t = exp(-softplus(dt_t) e^{A_log})),
    with input-dependent B_t, C_t of size ``d_state`` shared by all heads. ``forward`` is the quadratic dual form
    (``sequence_scans.ssd_dual``: masked (C B^T * L) X, matrix products only); ``step`` is the recurrence a decoder runs."""

    def __init__(self, d_model, d_state=16, head_dim=16, expand=2):
        super().__init__()
        d_in = expand * d_model
        if d_in % head_dim:
            raise ValueError("expand * d_model must be a multiple of head_dim")
        self.d_in, self.n_heads, self.hd, self.ds = d_in, d_in // head_dim, head_dim, d_state
        self.in_proj = nn.Linear(d_model, 2 * d_in + 2 * d_state + self.n_heads, bias=False)
        self.A_log = nn.Parameter(torch.zeros(self.n_heads))
        self.dt_bias = nn.Parameter(torch.full((self.n_heads,), -1.0))
        self.D = nn.Parameter(torch.ones(self.n_heads))
        self.out_proj = nn.Linear(d_in, d_model, bias=False)

    def _split(self, x):
        z, u, Bm, Cm, dt = torch.split(self.in_proj(x), [self.d_in, self.d_in, self.ds, self.ds, self.n_heads], -1)
        dt = F.softplus(dt + self.dt_bias)
        a = torch.exp(-dt * torch.exp(self.A_log))                 # per head and step, in (0, 1)
        return z, u, Bm, Cm, dt, a

    def forward(self, x):
        from .sequence_scans import ssd_dual
        Bsz, T, _ = x.shape
        z, u, Bm, Cm, dt, a = self._split(x)
        uh = u.view(Bsz, T, self.n_heads, self.hd)
        ys = []
        for b in range(Bsz):
            heads = [ssd_dual(uh[b, :, h] * dt[b, :, h, None], a[b, :, h], Bm[b], Cm[b]) + self.D[h] * uh[b, :, h]
                     for h in range(self.n_heads)]
            ys.append(torch.cat(heads, -1))
        return self.out_proj(torch.stack(ys) * F.silu(z))

    def init_state(self, x):
        return x.new_zeros(x.shape[0], self.n_heads, self.ds, self.hd)

    def step(self, xt, state):
        z, u, Bm, Cm, dt, a = self._split(xt[:, None])
        z, u, Bm, Cm, dt, a = (t[:, 0] for t in (z, u, Bm, Cm, dt, a))
        uh = u.view(-1, self.n_heads, self.hd)
        state = a[:, :, None, None] * state + Bm[:, None, :, None] * (uh * dt[:, :, None])[:, :, None, :]
        y = torch.einsum("bn,bhnp->bhp", Cm, state) + self.D[None, :, None] * uh
        return self.out_proj(y.reshape(-1, self.d_in) * F.silu(z)), state


class S5(nn.Module):
    """S5 layer: ONE multi-input multi-output diagonal state space per layer (complex eigenvalues, |lambda| < 1),
    evaluated by the parallel prefix scan in ``forward`` and by its recurrence in ``step``."""

    def __init__(self, d_model, d_state=32):
        super().__init__()
        self.log_mag = nn.Parameter(torch.log(torch.linspace(0.05, 0.6, d_state)))     # -log|lambda|
        self.phase = nn.Parameter(torch.linspace(0.0, math.pi, d_state))
        self.B = nn.Parameter(torch.randn(d_state, d_model, 2) / math.sqrt(d_model))
        self.C = nn.Parameter(torch.randn(d_model, d_state, 2) / math.sqrt(d_state))
        self.D = nn.Parameter(torch.ones(d_model))

    def _lam(self):
        return torch.exp(torch.complex(-torch.exp(self.log_mag), self.phase))

    def forward(self, x):
        from .sequence_scans import s5_parallel_scan
        lam, Bc, Cc = self._lam(), torch.view_as_complex(self.B), torch.view_as_complex(self.C)
        return torch.stack([s5_parallel_scan(x[b].float(), lam, Bc, Cc) for b in range(x.shape[0])]).to(x.dtype) + self.D * x

    def init_state(self, x):
        return torch.zeros(x.shape[0], self.log_mag.shape[0], dtype=torch.complex64, device=x.device)

    def step(self, xt, s):
        lam, Bc, Cc = self._lam(), torch.view_as_complex(self.B), torch.view_as_complex(self.C)
        s = lam * s + xt.float().to(torch.complex64) @ Bc.t()
        return (s @ Cc.t()).real.to(xt.dtype) + self.D * xt, s


class S4D(_Recurrent):
    """Diagonal state-space layer (S4D / S5 family): x' = A x + B u, y = Re(C x) + D u with a complex
    diagonal A discretised by zero-order hold, one SSM per channel."""

    def __init__(self, d_model, d_state=16, dt=0.05):
        super().__init__()
        self.log_neg_real = nn.Parameter(torch.log(0.5 * torch.ones(d_model, d_state)))
        self.imag = nn.Parameter(math.pi * torch.arange(d_state).float().repeat(d_model, 1))
        self.B = nn.Parameter(torch.ones(d_model, d_state, 2) * 0.5)
        self.C = nn.Parameter(torch.randn(d_model, d_state, 2) * 0.5)
        self.D = nn.Parameter(torch.ones(d_model))
        self.log_dt = nn.Parameter(torch.full((d_model,), math.log(dt)))

    def _discrete(self):
        A = torch.complex(-torch.exp(self.log_neg_real), self.imag)
        dt = torch.exp(self.log_dt)[:, None]
        Ab = torch.exp(A * dt)
        Bb = (Ab - 1) / A * torch.view_as_complex(self.B)
        return Ab, Bb, torch.view_as_complex(self.C)

    def init_state(self, x):
        return torch.zeros(x.shape[0], *self.log_neg_real.shape, dtype=torch.complex64, device=x.device)

    def forward(self, x, state=None):
        self._abc = self._discrete()
        return super().forward(x, state)

    def step(self, ut, s):
        Ab, Bb, C = self._abc
        s = Ab * s + Bb * ut.float()[:, :, None]
        return ((C * s).sum(-1).real + self.D * ut.float()).to(ut.dtype), s


class Mamba(_Recurrent):
    """Selective state-space block: input-dependent (dt, B, C), diagonal real A, gated output, with a
    short causal depthwise convolution in front (Mamba; ``mamba2=True`` shares one scalar A per head
    of width ``head_dim``)."""

    def __init__(self, d_model, d_state=16, expand=2, conv=4, mamba2=False, head_dim=16):
        super().__init__()
        d_in = expand * d_model
        self.d_in, self.d_state, self.conv_k = d_in, d_state, conv
        self.in_proj = nn.Linear(d_model, 2 * d_in, bias=False)
        self.conv = nn.Conv1d(d_in, d_in, conv, groups=d_in, padding=conv - 1)
        self.x_proj = nn.Linear(d_in, 2 * d_state + 1, bias=False)
        self.dt_bias = nn.Parameter(torch.full((d_in,), -2.0))
        n_a = d_in // head_dim if mamba2 else d_in
        self.expand_a = d_in // n_a
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1).float()).repeat(n_a, 1))
        self.D = nn.Parameter(torch.ones(d_in))
        self.out_proj = nn.Linear(d_in, d_model, bias=False)

    def init_state(self, x):
        return x.new_zeros(x.shape[0], self.d_in, self.d_state, dtype=torch.float32)

    def forward(self, x, state=None):
        B, T, _ = x.shape
        u, z = self.in_proj(x).chunk(2, -1)
        u = F.silu(self.conv(u.transpose(1, 2))[..., :T].transpose(1, 2))
        self._z = z
        self._t = 0
        y = super().forward(u, state)
        return self.out_proj(y * F.silu(z))

    def step(self, ut, s):
        p = self.x_proj(ut)
        Bm, Cm, dt = p[:, :self.d_state], p[:, self.d_state:2 * self.d_state], p[:, -1:]
        dt = F.softplus(dt + self.dt_bias)                                   # [B, d_in]
        A = -torch.exp(self.A_log).repeat_interleave(self.expand_a, 0)       # [d_in, N]
        s = torch.exp(dt[:, :, None] * A) * s + (dt * ut.float())[:, :, None] * Bm.float()[:, None, :]
        y = (s * Cm.float()[:, None, :]).sum(-1) + self.D * ut.float()
        return y.to(ut.dtype), s


class RWKVTimeMix(_Recurrent):
    """RWKV-4 style WKV recurrence with per-channel decay w and bonus u, numerically stabilised."""

    def __init__(self, d_model):
        super().__init__()
        self.r, self.k, self.v, self.o = (nn.Linear(d_model, d_model, bias=False) for _ in range(4))
        self.decay = nn.Parameter(torch.zeros(d_model))
        self.bonus = nn.Parameter(torch.zeros(d_model))

    def init_state(self, x):
        z = x.new_zeros(x.shape[0], x.shape[-1], dtype=torch.float32)
        return (z, z.clone(), z - 1e30)          # numerator, denominator, running max exponent

    def step(self, xt, st):
        a, b, p = st
        r, k, v = torch.sigmoid(self.r(xt)), self.k(xt).float(), self.v(xt).float()
        w = -torch.exp(self.decay)
        q = torch.maximum(p, self.bonus + k)
        e1, e2 = torch.exp(p - q), torch.exp(self.bonus + k - q)
        y = (e1 * a + e2 * v) / (e1 * b + e2)
        q2 = torch.maximum(p + w, k)
        e1, e2 = torch.exp(p + w - q2), torch.exp(k - q2)
        return self.o(r * y.to(xt.dtype)), (e1 * a + e2 * v, e1 * b + e2, q2)


class XLSTM(_Recurrent):
    """sLSTM cell of xLSTM: exponential input gate with a stabiliser state and a normaliser."""

    def __init__(self, d_model):
        super().__init__()
        self.w = nn.Linear(d_model, 4 * d_model)
        self.r = nn.Linear(d_model, 4 * d_model, bias=False)

    def init_state(self, x):
        z = x.new_zeros(x.shape[0], x.shape[-1], dtype=torch.float32)
        return (z, z.clone(), z.clone(), z.clone())     # h, c, n, m

    def step(self, xt, st):
        h, c, n, m = st
        i, f, zt, o = (self.w(xt).float() + self.r(h.to(xt.dtype)).float()).chunk(4, -1)
        m_new = torch.maximum(f + m, i)
        ig, fg = torch.exp(i - m_new), torch.exp(f + m - m_new)
        c = fg * c + ig * torch.tanh(zt)
        n = fg * n + ig
        h = torch.sigmoid(o) * c / n.clamp_min(1e-6)
        return h.to(xt.dtype), (h, c, n, m_new)


class Hyena(nn.Module):
    """Hyena operator of order 2: gated long convolutions whose filters come from a small MLP over
    positions, applied with FFTs (causal)."""

    def __init__(self, d_model, max_len=1024, filter_hidden=32):
        super().__init__()
        self.in_proj = nn.Linear(d_model, 3 * d_model)
        self.filter = nn.Sequential(nn.Linear(1, filter_hidden), nn.GELU(), nn.Linear(filter_hidden, d_model))
        self.decay = nn.Parameter(torch.linspace(1.0, 4.0, d_model))
        self.out = nn.Linear(d_model, d_model)
        self.max_len = max_len

    def forward(self, x):
        B, T, D = x.shape
        v, g1, g2 = self.in_proj(x).chunk(3, -1)
        t = torch.linspace(0, 1, T, device=x.device)[:, None]
        h = self.filter(t) * torch.exp(-self.decay[None, :] * t * 4.0)            # [T, D]
        n = 2 * T
        y = torch.fft.irfft(torch.fft.rfft((v * g1).float(), n=n, dim=1) * torch.fft.rfft(h.float(), n=n, dim=0)[None],
                            n=n, dim=1)[:, :T]
        return self.out((y.to(x.dtype)) * g2)


SEQUENCE_MIXERS = {"llama": None, "retnet": RetNet, "gla": GLA, "deltanet": DeltaNet, "hgrn": HGRN, "s4": S4D,
                   "mamba": Mamba, "mamba2": lambda d: Mamba(d, mamba2=True), "rwkv": RWKVTimeMix, "xlstm": XLSTM,
                   "hyena": Hyena}


class NdDecoderLM(nn.Module):
    """Decoder LM over any sequence mixer of this module: embedding -> N x [norm -> mixer -> +res ->
    norm -> SwiGLU -> +res] -> norm -> tied head. ``medusa_heads`` adds extra linear heads that predict
    tokens t+2, t+3, ... for speculative decoding."""

    def __init__(self, vocab, d_model=64, n_layers=2, mixer="llama", n_heads=4, n_kv_heads=2, d_ff=128,
                 medusa_heads=0):
        super().__init__()
        self.embed = nn.Embedding(vocab, d_model)
        self.blocks = nn.ModuleList()
        for _ in range(n_layers):
            if mixer == "llama":
                self.blocks.append(LlamaBlock(d_model, n_heads, n_kv_heads, d_ff))
            else:
                self.blocks.append(_MixerBlock(SEQUENCE_MIXERS[mixer](d_model), d_model, d_ff))
        self.norm = RMSNormND(d_model)
        self.medusa = nn.ModuleList([nn.Linear(d_model, d_model) for _ in range(medusa_heads)])

    def hidden(self, tokens):
        x = self.embed(tokens)
        for b in self.blocks:
            x = b(x)
        return self.norm(x)

    def forward(self, tokens):
        return self.hidden(tokens) @ self.embed.weight.t()

    def medusa_logits(self, tokens):
        h = self.hidden(tokens)
        return [(h + F.silu(m(h))) @ self.embed.weight.t() for m in self.medusa]


class _MixerBlock(nn.Module):
    def __init__(self, mixer, d_model, d_ff):
        super().__init__()
        self.n1, self.n2, self.mixer = RMSNormND(d_model), RMSNormND(d_model), mixer
        self.gate, self.up, self.down = nn.Linear(d_model, d_ff, bias=False), nn.Linear(d_model, d_ff, bias=False), \
            nn.Linear(d_ff, d_model, bias=False)

    def forward(self, x):
        x = x + self.mixer(self.n1(x))
        h = self.n2(x)
        return x + self.down(F.silu(self.gate(h)) * self.up(h))


@torch.no_grad()
def speculative_generate(target: NdDecoderLM, draft: NdDecoderLM, tokens: torch.Tensor, max_new: int, k: int = 4):
    """Greedy speculative decoding: the draft proposes ``k`` tokens, the target scores them in one pass
    and accepts the longest agreeing prefix plus its own next token. Returns (tokens, accepted_fraction);
    the output equals the target's own greedy decoding."""
    out = tokens.clone()
    proposed = accepted = 0
    while out.shape[1] - tokens.shape[1] < max_new:
        ctx = out
        for _ in range(k):
            ctx = torch.cat([ctx, draft(ctx)[:, -1].argmax(-1, keepdim=True)], 1)
        tl = target(ctx)[:, out.shape[1] - 1:-1].argmax(-1)           # target's choice at each drafted slot
        drafted = ctx[:, out.shape[1]:]
        agree = (tl == drafted).long().cumprod(1).sum(1).min().item()  # batch-wide common prefix
        proposed += k
        accepted += agree
        nxt = tl[:, agree:agree + 1] if agree < k else target(ctx)[:, -1].argmax(-1, keepdim=True)
        out = torch.cat([out, drafted[:, :agree], nxt], 1)
    return out[:, :tokens.shape[1] + max_new], accepted / max(proposed, 1)

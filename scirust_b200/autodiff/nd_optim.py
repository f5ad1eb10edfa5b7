"""Optimizers over N-D ``torch`` parameters (scirust-core/src/nn/nd_optim.rs:56-2428 and the raw-slice
family of scirust-core/src/optim.rs:40-232): RMSprop, Lion, LAMB, Adafactor, Muon (momentum
orthogonalised by Newton-Schulz iterations), Lookahead, SAM, Sophia-style clipped second-order,
Adan, AdEMAMix, schedule-free SGD, Prodigy-style distance adaptation, GaLore low-rank projection,
Shampoo and SOAP (Kronecker-factored preconditioners).
Each follows the ``torch.optim.Optimizer`` protocol (``step()`` after ``backward()``)."""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer


def newton_schulz_orthogonalize(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate the orthogonal polar factor of a 2-D matrix with the quintic Newton-Schulz
    iteration X <- aX + b(XX^T)X + c(XX^T)^2 X, (a, b, c) = (3.4445, -4.7750, 2.0315)
    (nd_optim.rs:346)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.norm() + eps)
    for _ in range(steps):
        A = x @ x.t()
        x = a * x + (b * A + c * (A @ A)) @ x
    return (x.t() if transposed else x).to(g.dtype)


class RMSprop(Optimizer):
    def __init__(self, params, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                d = p.grad + g["weight_decay"] * p if g["weight_decay"] else p.grad
                st = self.state[p]
                sq = st.setdefault("sq", torch.zeros_like(p))
                sq.mul_(g["alpha"]).addcmul_(d, d, value=1 - g["alpha"])
                p.addcdiv_(d, sq.sqrt().add_(g["eps"]), value=-g["lr"])


class Lion(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                m = self.state[p].setdefault("m", torch.zeros_like(p))
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(torch.sign(m * b1 + p.grad * (1 - b1)), alpha=-g["lr"])
                m.mul_(b2).add_(p.grad, alpha=1 - b2)


class LAMB(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                m = st.setdefault("m", torch.zeros_like(p))
                v = st.setdefault("v", torch.zeros_like(p))
                m.mul_(b1).add_(p.grad, alpha=1 - b1)
                v.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                u = (m / (1 - b1 ** st["t"])) / ((v / (1 - b2 ** st["t"])).sqrt() + g["eps"]) + g["weight_decay"] * p
                wn, un = p.norm(), u.norm()
                trust = (wn / un).item() if wn > 0 and un > 0 else 1.0
                p.add_(u, alpha=-g["lr"] * trust)


class Adafactor(Optimizer):
    """Factored second moments for matrices (row and column statistics), full for vectors."""

    def __init__(self, params, lr=1e-3, beta2=0.999, eps=1e-30, clip=1.0):
        super().__init__(params, dict(lr=lr, beta2=beta2, eps=eps, clip=clip))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st, gr = self.state[p], p.grad
                sq = gr * gr + g["eps"]
                if gr.dim() == 2:
                    r = st.setdefault("r", torch.zeros(gr.shape[0], device=gr.device))
                    c = st.setdefault("c", torch.zeros(gr.shape[1], device=gr.device))
                    r.mul_(g["beta2"]).add_(sq.mean(1), alpha=1 - g["beta2"])
                    c.mul_(g["beta2"]).add_(sq.mean(0), alpha=1 - g["beta2"])
                    v = torch.outer(r, c) / r.mean().clamp_min(1e-30)
                else:
                    v = st.setdefault("v", torch.zeros_like(gr))
                    v.mul_(g["beta2"]).add_(sq, alpha=1 - g["beta2"])
                u = gr / v.sqrt().clamp_min(1e-30)
                u = u / max(1.0, (u.pow(2).mean().sqrt() / g["clip"]).item())
                p.add_(u, alpha=-g["lr"])


class Muon(Optimizer):
    """Momentum -> Newton-Schulz orthogonalisation -> scaled update for 2-D weights; other
    parameters fall back to AdamW-style updates (scirust-sciagent/src/train/optimizer.rs:47-103)."""

    def __init__(self, params, lr=0.02, momentum=0.95, ns_steps=5, adam_lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, ns_steps=ns_steps, adam_lr=adam_lr, betas=betas, eps=eps,
                                      weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if p.dim() == 2 and min(p.shape) > 1:
                    buf = st.setdefault("buf", torch.zeros_like(p))
                    buf.mul_(g["momentum"]).add_(p.grad)
                    upd = newton_schulz_orthogonalize(p.grad + g["momentum"] * buf, g["ns_steps"])
                    scale = max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                    p.mul_(1 - g["lr"] * g["weight_decay"]).add_(upd, alpha=-g["lr"] * scale)
                else:
                    b1, b2 = g["betas"]
                    st["t"] = st.get("t", 0) + 1
                    m = st.setdefault("m", torch.zeros_like(p))
                    v = st.setdefault("v", torch.zeros_like(p))
                    m.mul_(b1).add_(p.grad, alpha=1 - b1)
                    v.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                    p.addcdiv_(m / (1 - b1 ** st["t"]), (v / (1 - b2 ** st["t"])).sqrt() + g["eps"], value=-g["adam_lr"])


class Adan(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.02, 0.08, 0.01), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2, b3 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                prev = st.get("prev", p.grad.clone())
                m = st.setdefault("m", torch.zeros_like(p))
                d = st.setdefault("d", torch.zeros_like(p))
                n = st.setdefault("n", torch.zeros_like(p))
                diff = p.grad - prev
                m.mul_(1 - b1).add_(p.grad, alpha=b1)
                d.mul_(1 - b2).add_(diff, alpha=b2)
                u = p.grad + (1 - b2) * diff
                n.mul_(1 - b3).addcmul_(u, u, value=b3)
                p.addcdiv_(m + (1 - b2) * d, n.sqrt() + g["eps"], value=-g["lr"])
                p.div_(1 + g["lr"] * g["weight_decay"])
                st["prev"] = p.grad.clone()


class AdEMAMix(Optimizer):
    """Adam with an additional slow EMA of the gradient mixed into the numerator."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999, 0.9999), alpha=5.0, eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, alpha=alpha, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2, b3 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                m1 = st.setdefault("m1", torch.zeros_like(p))
                m2 = st.setdefault("m2", torch.zeros_like(p))
                v = st.setdefault("v", torch.zeros_like(p))
                m1.mul_(b1).add_(p.grad, alpha=1 - b1)
                m2.mul_(b3).add_(p.grad, alpha=1 - b3)
                v.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                num = m1 / (1 - b1 ** st["t"]) + g["alpha"] * m2
                p.mul_(1 - g["lr"] * g["weight_decay"]).addcdiv_(num, (v / (1 - b2 ** st["t"])).sqrt() + g["eps"], value=-g["lr"])


class Sophia(Optimizer):
    """Clipped update m / max(rho * h, eps) with an EMA ``h`` of a diagonal curvature estimate
    (squared gradients, refreshed every ``k`` steps)."""

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, k=10, eps=1e-12, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, k=k, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                m = st.setdefault("m", torch.zeros_like(p))
                h = st.setdefault("h", torch.zeros_like(p))
                m.mul_(b1).add_(p.grad, alpha=1 - b1)
                if st["t"] % g["k"] == 1 or g["k"] == 1:
                    h.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_((m / torch.clamp(g["rho"] * h, min=g["eps"])).clamp_(-1, 1), alpha=-g["lr"])


class ScheduleFreeSGD(Optimizer):
    """Schedule-free SGD: gradients are taken at y = (1-beta) z + beta x; x is the running average
    of z. Call ``eval_params()`` to read x."""

    def __init__(self, params, lr=1.0, beta=0.9):
        super().__init__(params, dict(lr=lr, beta=beta))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                z = st.setdefault("z", p.detach().clone())
                x = st.setdefault("x", p.detach().clone())
                z.add_(p.grad, alpha=-g["lr"])
                x.mul_(1 - 1.0 / st["t"]).add_(z, alpha=1.0 / st["t"])
                p.copy_((1 - g["beta"]) * z + g["beta"] * x)

    def eval_params(self):
        return {p: self.state[p]["x"] for g in self.param_groups for p in g["params"] if "x" in self.state[p]}


class Lookahead:
    """Wraps an optimizer: every ``k`` fast steps the slow weights move ``alpha`` of the way."""

    def __init__(self, base: Optimizer, k: int = 5, alpha: float = 0.5):
        self.base, self.k, self.alpha, self.n = base, k, alpha, 0
        self.slow = {p: p.detach().clone() for g in base.param_groups for p in g["params"]}

    @torch.no_grad()
    def step(self):
        self.base.step()
        self.n += 1
        if self.n % self.k == 0:
            for p, s in self.slow.items():
                s.add_(p - s, alpha=self.alpha)
                p.copy_(s)

    def zero_grad(self):
        self.base.zero_grad()


class SAM:
    """Sharpness-aware minimisation: ``first_step`` climbs to w + rho g/|g|, ``second_step`` restores
    w and applies the base optimizer with the gradient taken at the perturbed point."""

    def __init__(self, base: Optimizer, rho: float = 0.05):
        self.base, self.rho, self._e = base, rho, {}

    @torch.no_grad()
    def first_step(self):
        ps = [p for g in self.base.param_groups for p in g["params"] if p.grad is not None]
        norm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in ps)) + 1e-12
        for p in ps:
            e = p.grad * (self.rho / norm)
            p.add_(e)
            self._e[p] = e

    @torch.no_grad()
    def second_step(self):
        for p, e in self._e.items():
            p.sub_(e)
        self._e = {}
        self.base.step()


class GaLore(Optimizer):
    """Adam in a rank-r subspace of each matrix gradient; the projector (left singular vectors) is
    refreshed every ``update_gap`` steps."""

    def __init__(self, params, lr=1e-3, rank=8, update_gap=50, betas=(0.9, 0.999), eps=1e-8, scale=1.0):
        super().__init__(params, dict(lr=lr, rank=rank, update_gap=update_gap, betas=betas, eps=eps, scale=scale))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                gr = p.grad.float()
                lowrank = gr.dim() == 2 and min(gr.shape) > g["rank"]
                if lowrank:
                    if "P" not in st or (st["t"] - 1) % g["update_gap"] == 0:
                        u, _, _ = torch.linalg.svd(gr, full_matrices=False)
                        st["P"] = u[:, : g["rank"]]
                        st.pop("m", None)
                        st.pop("v", None)
                    gr = st["P"].t() @ gr
                m = st.setdefault("m", torch.zeros_like(gr))
                v = st.setdefault("v", torch.zeros_like(gr))
                m.mul_(b1).add_(gr, alpha=1 - b1)
                v.mul_(b2).addcmul_(gr, gr, value=1 - b2)
                u = (m / (1 - b1 ** st["t"])) / ((v / (1 - b2 ** st["t"])).sqrt() + g["eps"])
                if lowrank:
                    u = g["scale"] * (st["P"] @ u)
                p.add_(u.to(p.dtype), alpha=-g["lr"])


class Prodigy(Optimizer):
    """Adam whose step size is multiplied by an online estimate ``d`` of the distance to the solution
    (d grows with <g, x0 - x> / |weighted gradient sum|)."""

    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, d0=1e-6):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps))
        self.d, self.num = d0, 0.0

    @torch.no_grad()
    def step(self):
        den = 0.0
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                x0 = st.setdefault("x0", p.detach().clone())
                s = st.setdefault("s", torch.zeros_like(p))
                m = st.setdefault("m", torch.zeros_like(p))
                v = st.setdefault("v", torch.zeros_like(p))
                self.num = math.sqrt(b2) * self.num + (1 - math.sqrt(b2)) * self.d * self.d * float((p.grad * (x0 - p)).sum())
                s.mul_(math.sqrt(b2)).add_(p.grad, alpha=(1 - math.sqrt(b2)) * self.d * self.d)
                den += float(s.abs().sum())
                m.mul_(b1).add_(p.grad, alpha=(1 - b1) * self.d)
                v.mul_(b2).addcmul_(p.grad, p.grad, value=(1 - b2) * self.d * self.d)
                p.addcdiv_(m, v.sqrt() + self.d * g["eps"], value=-g["lr"] * self.d)
        if den > 0:
            self.d = max(self.d, self.num / den)


def _sym_eigh(a: torch.Tensor):
    """Eigen-decomposition of a symmetric matrix in fp64 with a sign convention (largest-magnitude
    entry of every eigenvector positive), so that repeated runs give the same basis. The reference
    uses cyclic Jacobi sweeps (nd_optim.rs:720-783); any orthonormal eigenbasis serves the optimizers."""
    w, q = torch.linalg.eigh(a.double())
    idx = q.abs().argmax(dim=0)
    sign = torch.sign(q[idx, torch.arange(q.shape[1], device=q.device)])
    sign[sign == 0] = 1.0
    return w, q * sign


def inverse_pth_root(a: torch.Tensor, p: float, eps: float) -> torch.Tensor:
    """(A + eps I)^(-1/p) of a symmetric positive semi-definite matrix through its eigen-decomposition
    (nd_optim.rs:1596-1624); eigenvalues are clamped at eps before the root."""
    w, q = _sym_eigh(a)
    d = (w.clamp_min(0.0) + eps).pow(-1.0 / p)
    return ((q * d) @ q.t()).to(a.dtype)


class Shampoo(Optimizer):
    """Shampoo (nd_optim.rs:1629-1840): for a 2-D weight the Kronecker factors L = E[G G^T],
    R = E[G^T G] (running averages with decay ``beta``) and the step W -= lr * L^(-1/4) G R^(-1/4);
    the inverse roots are refreshed every ``precond_freq`` steps. Other shapes use diagonal Adagrad."""

    def __init__(self, params, lr=0.1, beta=0.95, eps=1e-6, weight_decay=0.0, precond_freq=1):
        super().__init__(params, dict(lr=lr, beta=beta, eps=eps, weight_decay=weight_decay, precond_freq=precond_freq))
        self.t = 0

    @torch.no_grad()
    def step(self):
        self.t += 1
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if p.dim() == 2 and min(p.shape) >= 2:
                    m, n = p.shape
                    if "l" not in st:
                        st["l"] = torch.zeros(m, m, dtype=torch.float32, device=p.device)
                        st["r"] = torch.zeros(n, n, dtype=torch.float32, device=p.device)
                    st["l"].mul_(g["beta"]).add_(grad @ grad.t(), alpha=1 - g["beta"])
                    st["r"].mul_(g["beta"]).add_(grad.t() @ grad, alpha=1 - g["beta"])
                    if "il" not in st or self.t % g["precond_freq"] == 0:
                        st["il"] = inverse_pth_root(st["l"], 4.0, g["eps"])
                        st["ir"] = inverse_pth_root(st["r"], 4.0, g["eps"])
                    u = st["il"] @ grad @ st["ir"]
                    p.sub_((u + g["weight_decay"] * p.float()).to(p.dtype), alpha=g["lr"])
                else:
                    g2 = st.setdefault("g2", torch.zeros_like(grad))
                    g2.addcmul_(grad, grad)
                    u = grad / (g2.sqrt() + g["eps"])
                    p.sub_((u + g["weight_decay"] * p.float()).to(p.dtype), alpha=g["lr"])


class SOAP(Optimizer):
    """SOAP (nd_optim.rs:790-1010): Adam run in the eigenbasis of Shampoo's factors. For a 2-D weight the
    gradient is rotated (G^ = Q_L^T G Q_R), Adam's moments live in that basis, the update is rotated back;
    the factors are running averages with decay ``shampoo_beta``; every ``precond_freq`` steps the bases are
    recomputed and the moments rotated into them (the second moment kept non-negative). Other shapes use
    plain Adam."""

    def __init__(self, params, lr=3e-3, betas=(0.9, 0.999), shampoo_beta=0.95, eps=1e-8, weight_decay=0.0,
                 precond_freq=10):
        super().__init__(params, dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps,
                                      weight_decay=weight_decay, precond_freq=precond_freq))
        self.t = 0

    @torch.no_grad()
    def step(self):
        self.t += 1
        for g in self.param_groups:
            b1, b2 = g["betas"]
            bc1, bc2 = 1 - b1 ** self.t, 1 - b2 ** self.t
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                if "m" not in st:
                    st["m"] = torch.zeros_like(grad)
                    st["v"] = torch.zeros_like(grad)
                matrix = p.dim() == 2 and min(p.shape) >= 2
                if matrix and "ql" not in st:      # first touch: factors and bases from this gradient
                    st["l"] = grad @ grad.t()
                    st["r"] = grad.t() @ grad
                    st["ql"] = _sym_eigh(st["l"])[1].float()
                    st["qr"] = _sym_eigh(st["r"])[1].float()
                ghat = st["ql"].t() @ grad @ st["qr"] if matrix else grad
                st["m"].mul_(b1).add_(ghat, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(ghat, ghat, value=1 - b2)
                upd = (st["m"] / bc1) / ((st["v"] / bc2).sqrt() + g["eps"])
                if matrix:
                    upd = st["ql"] @ upd @ st["qr"].t()
                p.sub_((upd + g["weight_decay"] * p.float()).to(p.dtype), alpha=g["lr"])
                if not matrix:
                    continue
                sb = g["shampoo_beta"]
                st["l"].mul_(sb).add_(grad @ grad.t(), alpha=1 - sb)
                st["r"].mul_(sb).add_(grad.t() @ grad, alpha=1 - sb)
                if self.t % g["precond_freq"] == 0:
                    ql_new = _sym_eigh(st["l"])[1].float()
                    qr_new = _sym_eigh(st["r"])[1].float()
                    rot_l, rot_r = ql_new.t() @ st["ql"], st["qr"].t() @ qr_new
                    st["m"] = rot_l @ st["m"] @ rot_r
                    st["v"] = (rot_l @ st["v"] @ rot_r).abs()
                    st["ql"], st["qr"] = ql_new, qr_new

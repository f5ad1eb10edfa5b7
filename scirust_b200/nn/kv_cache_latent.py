"""Residual-latent, adaptive and tiered KV caches: fixed-capacity, reconstruction-free.

* ``ResidualQuantizedLatentKvCache``: every key / value row is stored as quantised latent coefficients
  (rank-r projection on an orthonormal basis; fp32 / INT8 / INT4 codes with one scale per row) plus a FIXED number of
  sparse residual channels (the ``slots`` largest-magnitude entries of what the projection lost, indices as 16-bit,
  values fp32 / INT8 / INT4). Attention never rebuilds the dense rows: scores are ``(B^T q) . z_t`` plus the
  residual correction ``sum q[idx] * res``; the output is ONE up-projection of the probability-weighted latent
  sum, into which the weighted value residuals are scattered. All storage is allocated at construction; ``append``
  past the capacity is an error, ``remove_oldest`` slides the window.
* ``select_adaptive_plan`` / ``AdaptiveKvPlanner``: exhaustive, deterministic choice of key and value ranks, residual
  slot counts and storage formats under a strict byte budget per token, minimising the reconstruction error
  measured on a calibration sample; ties go to the cheaper, then to the earlier candidate.
* ``TieredResidualLatentBackend``: three such caches (hot / warm / cold) with decreasing fidelity; rows migrate
  hot -> warm -> cold as they age (re-encoded from their reconstruction), the cold tier evicts its oldest row when
  full; telemetry reports the tier populations, evictions and bytes.

Counterparts: scirust-core/src/nn/residual_latent_kv_cache.rs:20-700 (config, errors, ``append`` :450,
``attention_into`` :530, ``reconstruct_token_into`` :619, ``remove_oldest`` :669, byte accounting :363-440),
adaptive_latent_kv.rs:21-560 (policy config, plan, ``select_adaptive_plan`` :257, ``estimate_channel_bytes`` :509),
tiered_latent_kv_backend.rs:21-330 (tiers, telemetry, migration).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

FORMATS = ("fp32", "int8", "int4")
_BITS = {"fp32": 32, "int8": 8, "int4": 4}


class ResidualLatentCacheError(RuntimeError):
    pass


@dataclass(frozen=True)
class SparseResidualConfig:
    slots: int = 0
    fmt: str = "fp32"

    @staticmethod
    def disabled() -> "SparseResidualConfig":
        return SparseResidualConfig(0, "fp32")


def _quant(x: torch.Tensor, fmt: str):
    """Row-wise symmetric codes + scale; fp32 keeps the values."""
    if fmt == "fp32":
        return x.clone(), torch.ones(x.shape[0])
    qmax = 127.0 if fmt == "int8" else 7.0
    amax = x.abs().amax(-1)
    scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    return torch.clamp(torch.round(x / scale[:, None]), -qmax, qmax), scale


def estimate_channel_bytes(rank: int, fmt: str, residual: SparseResidualConfig) -> int:
    """Persistent bytes of ONE row of one channel (key or value)."""
    coef = (rank * _BITS[fmt] + 7) // 8 + (4 if fmt != "fp32" else 0)
    res = 0
    if residual.slots:
        res = residual.slots * 2 + (residual.slots * _BITS[residual.fmt] + 7) // 8 + (4 if residual.fmt != "fp32" else 0)
    return coef + res


class _Channel:
    """Latent coefficients + sparse residual of one of {keys, values}."""

    def __init__(self, dim, rank, basis, fmt, residual: SparseResidualConfig, capacity):
        if fmt not in FORMATS or residual.fmt not in FORMATS:
            raise ResidualLatentCacheError("unknown storage format")
        if not 1 <= rank <= dim or residual.slots < 0 or residual.slots > dim or dim > 65535:
            raise ResidualLatentCacheError("rank / residual slots out of range")
        self.dim, self.rank, self.fmt, self.res = dim, rank, fmt, residual
        self.B = basis[:, :rank].contiguous()
        self.coef = torch.zeros(capacity, rank)
        self.scale = torch.ones(capacity)
        self.ridx = torch.zeros(capacity, residual.slots, dtype=torch.int64)
        self.rval = torch.zeros(capacity, residual.slots)
        self.rscale = torch.ones(capacity)

    def encode(self, t: int, x: torch.Tensor) -> None:
        z = x @ self.B
        c, s = _quant(z[None, :], self.fmt)
        self.coef[t], self.scale[t] = c[0], s[0]
        if self.res.slots:
            r = x - (c[0] * s[0]) @ self.B.t()
            idx = torch.sort(torch.sort(-r.abs(), stable=True).indices[: self.res.slots]).values
            v, vs = _quant(r[idx][None, :], self.res.fmt)
            self.ridx[t], self.rval[t], self.rscale[t] = idx, v[0], vs[0]

    def latent(self, n: int) -> torch.Tensor:
        return self.coef[:n] * self.scale[:n, None]

    def residual_values(self, n: int) -> torch.Tensor:
        return self.rval[:n] * self.rscale[:n, None]

    def reconstruct(self, t: int) -> torch.Tensor:
        x = (self.coef[t] * self.scale[t]) @ self.B.t()
        if self.res.slots:
            x = x.index_add(0, self.ridx[t], self.rval[t] * self.rscale[t])
        return x

    def shift(self, n: int) -> None:
        for buf in (self.coef, self.scale, self.ridx, self.rval, self.rscale):
            buf[: n - 1] = buf[1:n].clone()

    def row_bytes(self) -> int:
        return estimate_channel_bytes(self.rank, self.fmt, self.res)


def default_basis(dim: int, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(dim, dim, generator=g))
    return q


def fit_basis(samples: torch.Tensor) -> torch.Tensor:
    """Right-singular vectors of sample rows, most important first (a full orthonormal basis)."""
    _, _, vh = torch.linalg.svd(samples.float(), full_matrices=True)
    return vh.t().contiguous()


class ResidualQuantizedLatentKvCache:
    def __init__(self, dim: int, capacity: int, key_rank: int, value_rank: int, key_fmt: str = "int8",
                 value_fmt: str = "int8", key_residual: SparseResidualConfig = SparseResidualConfig.disabled(),
                 value_residual: SparseResidualConfig = SparseResidualConfig.disabled(), key_basis=None,
                 value_basis=None):
        if capacity < 1:
            raise ResidualLatentCacheError("capacity must be positive")
        self.dim, self.capacity, self.n = dim, capacity, 0
        kb = key_basis if key_basis is not None else default_basis(dim, 1)
        vb = value_basis if value_basis is not None else default_basis(dim, 2)
        self.k = _Channel(dim, key_rank, kb, key_fmt, key_residual, capacity)
        self.v = _Channel(dim, value_rank, vb, value_fmt, value_residual, capacity)

    def __len__(self) -> int:
        return self.n

    def append(self, key, value) -> None:
        if self.n >= self.capacity:
            raise ResidualLatentCacheError("cache is full")
        key, value = torch.as_tensor(key).float().reshape(-1), torch.as_tensor(value).float().reshape(-1)
        if key.numel() != self.dim or value.numel() != self.dim:
            raise ResidualLatentCacheError("row has the wrong dimension")
        if not bool(torch.isfinite(key).all() and torch.isfinite(value).all()):
            raise ResidualLatentCacheError("non-finite value in an appended row")
        self.k.encode(self.n, key)
        self.v.encode(self.n, value)
        self.n += 1

    def attention(self, q, scale: float | None = None) -> torch.Tensor:
        """softmax(q K^T * scale) V over the cached rows, without rebuilding K or V."""
        if self.n == 0:
            raise ResidualLatentCacheError("attention over an empty cache")
        q = torch.as_tensor(q).float().reshape(-1)
        n = self.n
        scale = 1.0 / math.sqrt(self.dim) if scale is None else scale
        s = self.k.latent(n) @ (self.k.B.t() @ q)                     # scores in the latent space
        if self.k.res.slots:
            s = s + (q[self.k.ridx[:n]] * self.k.residual_values(n)).sum(-1)
        p = torch.softmax(s * scale, 0)
        out = (p @ self.v.latent(n)) @ self.v.B.t()                   # one up-projection
        if self.v.res.slots:
            out = out.index_add(0, self.v.ridx[:n].reshape(-1), (p[:, None] * self.v.residual_values(n)).reshape(-1))
        return out

    # AttentionBackend surface
    def decode_step(self, q, scale=None):
        return self.attention(q, scale)

    def reconstruct_token(self, t: int):
        if not 0 <= t < self.n:
            raise ResidualLatentCacheError("token index out of range")
        return self.k.reconstruct(t), self.v.reconstruct(t)

    def key_residual_indices_for(self, t: int):
        return self.k.ridx[t].tolist() if 0 <= t < self.n and self.k.res.slots else None

    def remove_oldest(self) -> None:
        if self.n == 0:
            raise ResidualLatentCacheError("cache is empty")
        self.k.shift(self.n)
        self.v.shift(self.n)
        self.n -= 1

    def bytes_per_token(self) -> int:
        return self.k.row_bytes() + self.v.row_bytes()

    def used_bytes(self) -> int:
        return self.n * self.bytes_per_token()

    def allocated_bytes(self) -> int:
        return self.capacity * self.bytes_per_token()

    def nbytes(self) -> int:
        return self.used_bytes()


# ------------------------------------------------------------------------------------- adaptive planner
@dataclass(frozen=True)
class AdaptiveChannelPlan:
    rank: int
    fmt: str
    residual: SparseResidualConfig
    bytes_per_token: int
    error: float


@dataclass(frozen=True)
class AdaptiveKvPlan:
    key: AdaptiveChannelPlan
    value: AdaptiveChannelPlan

    @property
    def bytes_per_token(self) -> int:
        return self.key.bytes_per_token + self.value.bytes_per_token

    @property
    def error(self) -> float:
        return self.key.error + self.value.error


def _channel_candidates(samples, basis, ranks, slot_choices, formats):
    dim = samples.shape[1]
    out = []
    for rank in ranks:
        for fmt in formats:
            for slots in slot_choices:
                for rfmt in (formats if slots else ("fp32",)):
                    res = SparseResidualConfig(slots, rfmt)
                    ch = _Channel(dim, rank, basis, fmt, res, samples.shape[0])
                    err = 0.0
                    for t in range(samples.shape[0]):
                        ch.encode(t, samples[t])
                        err += float((samples[t] - ch.reconstruct(t)).pow(2).sum())
                    out.append(AdaptiveChannelPlan(rank, fmt, res, estimate_channel_bytes(rank, fmt, res),
                                                   err / samples.shape[0]))
    return out


def select_adaptive_plan(key_samples, value_samples, budget_bytes_per_token: int, ranks=(4, 8, 16),
                         slot_choices=(0, 2, 4), formats=FORMATS, key_basis=None, value_basis=None,
                         key_weight: float = 1.0):
    """The plan with the least ``key_weight * key error + value error`` among those within the budget; ties: fewer
    bytes, then enumeration order. Raises if nothing fits."""
    ks, vs = torch.as_tensor(key_samples).float(), torch.as_tensor(value_samples).float()
    dim = ks.shape[1]
    ranks = [r for r in ranks if r <= dim]
    kb = key_basis if key_basis is not None else fit_basis(ks)
    vb = value_basis if value_basis is not None else fit_basis(vs)
    kc = _channel_candidates(ks, kb, ranks, slot_choices, formats)
    vc = _channel_candidates(vs, vb, ranks, slot_choices, formats)
    best, best_key = None, None
    for a in kc:
        for b in vc:
            nb = a.bytes_per_token + b.bytes_per_token
            if nb > budget_bytes_per_token:
                continue
            key = (key_weight * a.error + b.error, nb)
            if best_key is None or key < best_key:
                best, best_key = AdaptiveKvPlan(a, b), key
    if best is None:
        raise ResidualLatentCacheError("no storage plan fits the byte budget")
    return best, kb, vb


class AdaptiveKvPlanner:
    """Collects calibration rows, then plans once: ``observe(k, v)`` ... ``plan(budget)`` -> cache factory."""

    def __init__(self, dim: int, **search):
        self.dim, self.search = dim, search
        self.keys, self.values = [], []

    def observe(self, key, value) -> None:
        self.keys.append(torch.as_tensor(key).float().reshape(-1))
        self.values.append(torch.as_tensor(value).float().reshape(-1))

    def plan(self, budget_bytes_per_token: int):
        if len(self.keys) < 2:
            raise ResidualLatentCacheError("planner needs at least two observed rows")
        return select_adaptive_plan(torch.stack(self.keys), torch.stack(self.values), budget_bytes_per_token,
                                    **self.search)

    def build(self, budget_bytes_per_token: int, capacity: int) -> ResidualQuantizedLatentKvCache:
        plan, kb, vb = self.plan(budget_bytes_per_token)
        return ResidualQuantizedLatentKvCache(self.dim, capacity, plan.key.rank, plan.value.rank, plan.key.fmt,
                                              plan.value.fmt, plan.key.residual, plan.value.residual, kb, vb)


# ------------------------------------------------------------------------------------------- tiers
@dataclass(frozen=True)
class TieredLatentTelemetry:
    hot_tokens: int
    warm_tokens: int
    cold_tokens: int
    evictions: int
    planned_persistent_bytes: int
    allocated_bytes: int


class TieredResidualLatentBackend:
    """Newest rows in the hot tier (highest fidelity), ageing into warm and cold; ``tiers`` = three
    ``dict(capacity=..., key_rank=..., value_rank=..., key_fmt=..., ...)`` configurations, hot first."""

    def __init__(self, dim: int, hot: dict, warm: dict, cold: dict, key_basis=None, value_basis=None):
        kb = key_basis if key_basis is not None else default_basis(dim, 1)
        vb = value_basis if value_basis is not None else default_basis(dim, 2)
        self.dim = dim
        self.hot, self.warm, self.cold = (ResidualQuantizedLatentKvCache(dim, key_basis=kb, value_basis=vb, **cfg)
                                          for cfg in (hot, warm, cold))
        self.evictions = 0

    def __len__(self) -> int:
        return len(self.hot) + len(self.warm) + len(self.cold)

    def _demote(self, src, dst) -> None:
        k, v = src.reconstruct_token(0)
        src.remove_oldest()
        if len(dst) >= dst.capacity:
            if dst is self.cold:
                dst.remove_oldest()
                self.evictions += 1
            else:
                self._demote(dst, self.cold)
        dst.append(k, v)

    def append(self, key, value) -> None:
        if len(self.hot) >= self.hot.capacity:
            self._demote(self.hot, self.warm)
        self.hot.append(key, value)

    def attention(self, q, scale: float | None = None) -> torch.Tensor:
        """Attention over all tiers at once: per-tier scores are concatenated in age order, normalised together,
        and each tier contributes its probability-weighted values."""
        q = torch.as_tensor(q).float().reshape(-1)
        scale = 1.0 / math.sqrt(self.dim) if scale is None else scale
        tiers = [t for t in (self.cold, self.warm, self.hot) if len(t)]
        if not tiers:
            raise ResidualLatentCacheError("attention over an empty cache")
        scores = []
        for t in tiers:
            n = len(t)
            s = t.k.latent(n) @ (t.k.B.t() @ q)
            if t.k.res.slots:
                s = s + (q[t.k.ridx[:n]] * t.k.residual_values(n)).sum(-1)
            scores.append(s * scale)
        p = torch.softmax(torch.cat(scores), 0)
        out, off = torch.zeros(self.dim), 0
        for t in tiers:
            n = len(t)
            pt = p[off:off + n]
            off += n
            o = (pt @ t.v.latent(n)) @ t.v.B.t()
            if t.v.res.slots:
                o = o.index_add(0, t.v.ridx[:n].reshape(-1), (pt[:, None] * t.v.residual_values(n)).reshape(-1))
            out = out + o
        return out

    def decode_step(self, q, scale=None):
        return self.attention(q, scale)

    def telemetry(self) -> TieredLatentTelemetry:
        alloc = self.hot.allocated_bytes() + self.warm.allocated_bytes() + self.cold.allocated_bytes()
        return TieredLatentTelemetry(len(self.hot), len(self.warm), len(self.cold), self.evictions,
                                     self.hot.used_bytes() + self.warm.used_bytes() + self.cold.used_bytes(), alloc)

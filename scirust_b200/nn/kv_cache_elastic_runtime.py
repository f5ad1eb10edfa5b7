"""Elastic latent KV: online basis learning with committed versions, the HOT / WARM / COLD lifecycle controller,
representation metadata with epochs, and the integrated decode runtime that ties them to the adaptive planner and
the tiered residual-latent backend of ``kv_cache_latent``.

* ``DeterministicBasisLearner``: Oja-style subspace tracking. Per sample: project (``c = B^T x``), residual
  (``r = x - B c``), rank-one update ``B += lr * r c^T``, classical Gram-Schmidt every ``reorthogonalize_interval``
  samples (a degenerate column is replaced by a unit vector). The captured-energy fraction of the sample, in basis
  points, is the quality; a new VERSION is committed when enough samples passed, the quality gained enough over the
  last commit and the version table has room. Each version records an FNV-1a fingerprint over the exact fp32 bit
  patterns of the basis. ``CommittedBasisLearner`` also archives the basis snapshot of every version, so a decode
  session can be built from an immutable committed basis while learning continues.
* ``LatentKvLifecycle``: a fixed-capacity ring of token records (position, basis version, temperature, last access).
  ``admit`` evicts the oldest record when full; ``rebalance`` assigns temperatures by age (newest ``hot_tokens`` hot,
  next ``warm_tokens`` warm, rest cold) and returns the transitions with their target compression tier.
* ``KvRepresentationMetadata`` / ``RepresentedElasticKvCache``: what a cache stores (id, epoch, key transform scope,
  widths); a representation change must keep the contract (head dim, scope) and advance the epoch by exactly one.
* ``ElasticLatentDecodeRuntime``: one tiered backend per attention head, planned under a byte budget split evenly
  over the heads (remainder to the first heads); ``decode_step(token)`` projects q/k/v for all heads in one matrix
  product each, appends, attends per head and applies the output projection; telemetry counts steps, planned and
  allocated bytes, lifecycle transitions and evictions. ``ElasticLatentEncoderSession`` runs a whole pre-norm
  encoder one token at a time through such runtimes (LayerNorm, residuals and FFN unchanged).

Reference counterparts: scirust-core/src/nn/adaptive_latent_basis.rs:15-360, elastic_latent_basis_handoff.rs:26-380,
latent_kv_lifecycle.rs:8-330, elastic_kv_representation.rs:13-300, represented_elastic_kv_cache.rs:11-110,
elastic_latent_runtime.rs:30-480, elastic_latent_transformer.rs:23-260, elastic_latent_encoder_handoff.rs:21-120.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace

import numpy as np
import torch

from .kv_cache import ElasticKvCache
from .kv_cache_latent import (AdaptiveKvPlan, ResidualLatentCacheError, SparseResidualConfig,
                              TieredResidualLatentBackend, select_adaptive_plan)

_FNV_OFFSET, _FNV_PRIME, _M64 = 0xCBF29CE484222325, 0x100000001B3, (1 << 64) - 1


def basis_fingerprint(basis) -> int:
    """FNV-1a over the 32-bit patterns of the values, one value per round (row-major)."""
    bits = np.ascontiguousarray(torch.as_tensor(basis, dtype=torch.float32).cpu().numpy()).view(np.uint32).reshape(-1)
    h = _FNV_OFFSET
    for b in bits.tolist():
        h = ((h ^ b) * _FNV_PRIME) & _M64
    return h


# ---------------------------------------------------------------------------------- basis learning
class BasisLearningError(ValueError):
    pass


@dataclass(frozen=True)
class BasisLearningConfig:
    dimension: int
    rank: int
    learning_rate: float = 0.05
    reorthogonalize_interval: int = 4
    minimum_samples_between_versions: int = 16
    minimum_quality_gain_bps: int = 100
    maximum_versions: int = 8

    def validate(self):
        for name in ("dimension", "rank", "reorthogonalize_interval", "minimum_samples_between_versions",
                     "maximum_versions"):
            if getattr(self, name) == 0:
                raise BasisLearningError(f"{name} must be non-zero")
        if self.rank > self.dimension:
            raise BasisLearningError("basis rank exceeds dense dimension")
        lr = self.learning_rate
        if not (lr == lr) or lr <= 0.0 or lr > 1.0:
            raise BasisLearningError("learning rate must be finite and in (0, 1]")


@dataclass(frozen=True)
class BasisVersion:
    version: int
    samples_seen: int
    quality_bps: int
    fingerprint: int


@dataclass(frozen=True)
class BasisObservation:
    quality_bps: int
    committed: BasisVersion | None


def identity_prefix(dimension: int, rank: int) -> torch.Tensor:
    return torch.eye(dimension)[:, :rank].clone()


class DeterministicBasisLearner:
    def __init__(self, config: BasisLearningConfig, initial_basis):
        config.validate()
        b = torch.as_tensor(initial_basis, dtype=torch.float32)
        if b.numel() != config.dimension * config.rank:
            raise BasisLearningError(f"basis length mismatch: expected {config.dimension * config.rank}, got {b.numel()}")
        if not bool(torch.isfinite(b).all()):
            raise BasisLearningError("basis learning input contains a non-finite value")
        self.config = config
        self._basis = b.reshape(config.dimension, config.rank).clone()
        self.samples_seen = 0
        self._last_version_sample = 0
        self._last_quality = 0
        self.current_version = 0
        self._orthonormalize()
        self.versions = [BasisVersion(0, 0, 0, basis_fingerprint(self._basis))]

    def basis(self) -> torch.Tensor:
        return self._basis

    def _orthonormalize(self):
        B = self._basis
        d, r = B.shape
        for c in range(r):
            for p in range(c):
                B[:, c] -= (B[:, c] * B[:, p]).sum() * B[:, p]
            n2 = float((B[:, c] * B[:, c]).sum())
            if n2 <= float(np.finfo(np.float32).eps):
                B[:, c] = 0.0
                B[c % d, c] = 1.0
                n2 = 1.0
            B[:, c] *= 1.0 / (n2 ** 0.5)

    def _quality_bps(self, x) -> int:
        total = float((x * x).sum())
        if total == 0.0:
            return 10_000
        c = self._basis.t() @ x
        return int(round(min(max(float((c * c).sum()) / total, 0.0), 1.0) * 10_000.0))

    def observe(self, sample) -> BasisObservation:
        x = torch.as_tensor(sample, dtype=torch.float32).reshape(-1)
        cfg = self.config
        if x.numel() != cfg.dimension:
            raise BasisLearningError(f"sample length mismatch: expected {cfg.dimension}, got {x.numel()}")
        if not bool(torch.isfinite(x).all()):
            raise BasisLearningError("basis learning input contains a non-finite value")
        c = self._basis.t() @ x
        r = x - self._basis @ c
        self._basis += cfg.learning_rate * torch.outer(r, c)
        self.samples_seen += 1
        if self.samples_seen % cfg.reorthogonalize_interval == 0:
            self._orthonormalize()
        q = self._quality_bps(x)
        committed = None
        if (self.samples_seen - self._last_version_sample >= cfg.minimum_samples_between_versions
                and max(q - self._last_quality, 0) >= cfg.minimum_quality_gain_bps
                and len(self.versions) < cfg.maximum_versions):
            self.current_version += 1
            self._last_version_sample = self.samples_seen
            self._last_quality = q
            committed = BasisVersion(self.current_version, self.samples_seen, q, basis_fingerprint(self._basis))
            self.versions.append(committed)
        return BasisObservation(q, committed)


class CommittedBasisLearner:
    """A learner plus the exact basis snapshot of every committed version (storage reserved up front)."""

    def __init__(self, config: BasisLearningConfig, initial_basis):
        self.learner = DeterministicBasisLearner(config, initial_basis)
        self._archive = torch.zeros(config.maximum_versions, config.dimension, config.rank)
        self._archive[0] = self.learner.basis()

    def observe(self, sample) -> BasisObservation:
        obs = self.learner.observe(sample)
        if obs.committed is not None:
            self._archive[len(self.learner.versions) - 1] = self.learner.basis()
        return obs

    def basis(self):
        return self.learner.basis()

    def versions(self):
        return self.learner.versions

    def committed_basis(self, version: int):
        for i, v in enumerate(self.learner.versions):
            if v.version == version:
                snap = self._archive[i]
                if basis_fingerprint(snap) != v.fingerprint:
                    raise BasisLearningError(f"archived basis of version {version} does not match its fingerprint")
                return snap
        return None

    def latest_committed_basis(self):
        return self._archive[len(self.learner.versions) - 1]


def complete_basis(partial: torch.Tensor) -> torch.Tensor:
    """Extend ``[d, r]`` orthonormal columns to a full ``[d, d]`` orthonormal basis (deterministic: unit vectors are
    tried in index order and orthogonalised against what is there)."""
    d, r = partial.shape
    cols = [partial[:, i].clone() for i in range(r)]
    for e in range(d):
        if len(cols) == d:
            break
        v = torch.zeros(d)
        v[e] = 1.0
        for c in cols:
            v -= (v * c).sum() * c
        n = float(v.norm())
        if n > 1e-4:
            cols.append(v / n)
    return torch.stack(cols, 1)


# ---------------------------------------------------------------------------------- lifecycle
class CacheTemperature(enum.Enum):
    HOT = "hot"
    WARM = "warm"
    COLD = "cold"


class LifecycleError(ValueError):
    pass


@dataclass(frozen=True)
class CompressionTier:
    coefficient_format: str = "int8"
    residual_format: str = "int8"
    maximum_residual_slots: int = 0
    rank_divisor: int = 1


@dataclass(frozen=True)
class LifecycleConfig:
    capacity_tokens: int
    hot_tokens: int
    warm_tokens: int
    hot: CompressionTier = CompressionTier("fp32", "fp32", 4, 1)
    warm: CompressionTier = CompressionTier("int8", "int8", 2, 1)
    cold: CompressionTier = CompressionTier("int4", "int4", 0, 2)

    def validate(self):
        if self.capacity_tokens == 0:
            raise LifecycleError("lifecycle capacity must be non-zero")
        if self.hot_tokens + self.warm_tokens > self.capacity_tokens:
            raise LifecycleError("HOT and WARM windows exceed capacity")
        if 0 in (self.hot.rank_divisor, self.warm.rank_divisor, self.cold.rank_divisor):
            raise LifecycleError("compression rank divisor must be non-zero")

    @property
    def cold_tokens(self) -> int:
        return self.capacity_tokens - self.hot_tokens - self.warm_tokens


@dataclass
class TokenLifecycle:
    position: int
    basis_version: int
    temperature: CacheTemperature
    last_access_tick: int


@dataclass(frozen=True)
class Admission:
    position: int
    evicted: TokenLifecycle | None


@dataclass(frozen=True)
class LifecycleAction:
    position: int
    basis_version: int
    source: CacheTemperature
    to: CacheTemperature
    target: CompressionTier


class LatentKvLifecycle:
    def __init__(self, config: LifecycleConfig):
        config.validate()
        self.config = config
        self._slots: list = [None] * config.capacity_tokens
        self._start = self._len = self._next = self._tick = 0

    def __len__(self):
        return self._len

    def admit(self, basis_version: int) -> Admission:
        cap = self.config.capacity_tokens
        self._tick += 1
        evicted = None
        if self._len == cap:
            evicted = self._slots[self._start]
            self._start = (self._start + 1) % cap
        else:
            self._len += 1
        pos = self._next
        self._next += 1
        self._slots[(self._start + self._len - 1) % cap] = TokenLifecycle(pos, basis_version, CacheTemperature.HOT, self._tick)
        return Admission(pos, evicted)

    def _index(self, position: int):
        if self._len == 0:
            return None
        off = position - self._slots[self._start].position
        if not 0 <= off < self._len:
            return None
        return (self._start + off) % self.config.capacity_tokens

    def touch(self, position: int) -> None:
        self._tick += 1
        i = self._index(position)
        if i is None:
            raise LifecycleError(f"token position {position} is not resident")
        self._slots[i].last_access_tick = self._tick

    def get(self, position: int):
        i = self._index(position)
        return None if i is None else self._slots[i]

    def tier(self, temperature: CacheTemperature) -> CompressionTier:
        return {CacheTemperature.HOT: self.config.hot, CacheTemperature.WARM: self.config.warm,
                CacheTemperature.COLD: self.config.cold}[temperature]

    def rebalance(self, limit: int | None = None) -> list:
        """Assign temperatures by age; returns the transitions (at most ``limit`` are REPORTED, all are applied)."""
        cfg, actions = self.config, []
        for off in range(self._len):
            rec = self._slots[(self._start + off) % cfg.capacity_tokens]
            age = self._len - 1 - off
            want = CacheTemperature.HOT if age < cfg.hot_tokens else \
                CacheTemperature.WARM if age < cfg.hot_tokens + cfg.warm_tokens else CacheTemperature.COLD
            if rec.temperature != want:
                if limit is None or len(actions) < limit:
                    actions.append(LifecycleAction(rec.position, rec.basis_version, rec.temperature, want, self.tier(want)))
                rec.temperature = want
        return actions

    def counts(self) -> dict:
        out = {t: 0 for t in CacheTemperature}
        for off in range(self._len):
            out[self._slots[(self._start + off) % self.config.capacity_tokens].temperature] += 1
        return out


# ---------------------------------------------------------------------------------- representation metadata
class KvRepresentationError(ValueError):
    pass


class KvKeyTransformScope(enum.Enum):
    NONE = "none"
    PER_HEAD = "per_head"
    PER_LAYER = "per_layer"
    GLOBAL = "global"


@dataclass(frozen=True)
class KvRepresentationMetadata:
    representation_id: str
    epoch: int
    head_dim: int
    key_transform_scope: KvKeyTransformScope = KvKeyTransformScope.NONE
    key_width: int = 0
    value_width: int = 0

    def __post_init__(self):
        if not self.representation_id or not self.representation_id.strip():
            raise KvRepresentationError("representation id must not be empty")
        if self.epoch < 0 or self.head_dim <= 0:
            raise KvRepresentationError("epoch must be >= 0 and head_dim positive")

    def same_contract(self, other: "KvRepresentationMetadata") -> bool:
        return self.head_dim == other.head_dim and self.key_transform_scope == other.key_transform_scope

    def validate_successor(self, target: "KvRepresentationMetadata") -> None:
        if not self.same_contract(target):
            raise KvRepresentationError("successor representation changes the head dimension or the key transform scope")
        if target.epoch != self.epoch + 1:
            raise KvRepresentationError(f"successor epoch must be {self.epoch + 1}, got {target.epoch}")

    def next_epoch(self, representation_id: str | None = None) -> "KvRepresentationMetadata":
        return replace(self, epoch=self.epoch + 1, representation_id=representation_id or self.representation_id)


class RepresentedElasticKvCache:
    """``ElasticKvCache`` + what it currently stores; ``commit_representation`` only accepts a valid successor."""

    def __init__(self, dim: int, window: int, representation: KvRepresentationMetadata, budget_bytes=None):
        if representation.head_dim != dim:
            raise KvRepresentationError("representation head_dim differs from the cache dimension")
        self.inner = ElasticKvCache(dim, window, budget_bytes)
        self.representation = representation
        self.history = [representation]

    def commit_representation(self, target: KvRepresentationMetadata) -> None:
        self.representation.validate_successor(target)
        self.representation = target
        self.history.append(target)

    def append(self, k, v):
        self.inner.append(k, v)

    def attention(self, q, scale=None):
        return self.inner.decode_step(q, scale)

    def __len__(self):
        return len(self.inner)

    def compressed_bytes(self) -> int:
        return self.inner.nbytes()


# ---------------------------------------------------------------------------------- integrated runtime
class ElasticLatentRuntimeError(RuntimeError):
    pass


@dataclass(frozen=True)
class HeadCalibration:
    key_basis: torch.Tensor          # full [dh, dh] orthonormal basis for keys
    value_basis: torch.Tensor
    key_samples: torch.Tensor        # calibration rows [n, dh] that the planner measures error on
    value_samples: torch.Tensor
    basis_version: int = 0


@dataclass(frozen=True)
class ElasticLatentRuntimeConfig:
    capacity_tokens: int
    minimum_rank: int
    maximum_rank: int
    maximum_residual_slots: int
    persistent_budget_bytes: int          # whole runtime, all heads, at full capacity
    allocated_ceiling_bytes: int
    lifecycle: LifecycleConfig = field(default=None)


@dataclass(frozen=True)
class ElasticLatentTelemetry:
    steps: int
    planned_persistent_bytes: int
    allocated_bytes: int
    worst_quality_bps: int
    last_lifecycle_transitions: int
    last_lifecycle_evictions: int
    total_lifecycle_evictions: int


def _tier_cfg(plan: AdaptiveKvPlan, tier: CompressionTier, capacity: int, min_rank: int) -> dict:
    kr = max(min_rank, plan.key.rank // tier.rank_divisor)
    vr = max(min_rank, plan.value.rank // tier.rank_divisor)
    ks = min(plan.key.residual.slots, tier.maximum_residual_slots)
    vs = min(plan.value.residual.slots, tier.maximum_residual_slots)
    order = ("fp32", "int8", "int4")
    coarser = lambda a, b: order[max(order.index(a), order.index(b))]      # a tier never stores finer than planned
    return dict(capacity=max(capacity, 1), key_rank=kr, value_rank=vr,
                key_fmt=coarser(plan.key.fmt, tier.coefficient_format), value_fmt=coarser(plan.value.fmt, tier.coefficient_format),
                key_residual=SparseResidualConfig(ks, tier.residual_format) if ks else SparseResidualConfig.disabled(),
                value_residual=SparseResidualConfig(vs, tier.residual_format) if vs else SparseResidualConfig.disabled())


def _quality_bps(samples: torch.Tensor, basis: torch.Tensor, rank: int) -> int:
    total = float((samples * samples).sum())
    if total == 0.0:
        return 10_000
    c = samples @ basis[:, :rank]
    return int(round(min(float((c * c).sum()) / total, 1.0) * 10_000))


class ElasticLatentDecodeRuntime:
    def __init__(self, attention, config: ElasticLatentRuntimeConfig, calibrations):
        H, dh = attention.n_heads, attention.dh
        if H == 0:
            raise ElasticLatentRuntimeError("attention has no heads")
        if len(calibrations) != H:
            raise ElasticLatentRuntimeError(f"expected {H} head calibrations, got {len(calibrations)}")
        lc = config.lifecycle
        if lc is None or lc.capacity_tokens != config.capacity_tokens:
            raise ElasticLatentRuntimeError("lifecycle capacity differs from the runtime capacity")
        lc.validate()
        ranks = [r for r in range(config.minimum_rank, min(config.maximum_rank, dh) + 1)
                 if r == config.minimum_rank or r == min(config.maximum_rank, dh) or (r & (r - 1)) == 0]
        slots = sorted({0, config.maximum_residual_slots // 2, config.maximum_residual_slots})
        base, rem = divmod(config.persistent_budget_bytes, H)
        self.backends, self.plans, self.lifecycles, self.basis_versions = [], [], [], []
        planned = allocated = 0
        worst = 10_000
        for h, cal in enumerate(calibrations):
            head_budget = base + (1 if h < rem else 0)
            per_token = head_budget // config.capacity_tokens
            try:
                plan, _, _ = select_adaptive_plan(cal.key_samples, cal.value_samples, per_token, ranks=ranks,
                                                  slot_choices=slots, key_basis=cal.key_basis, value_basis=cal.value_basis)
            except ResidualLatentCacheError as e:
                raise ElasticLatentRuntimeError(f"head {h}: {e}") from e
            caps = (lc.hot_tokens, lc.warm_tokens, lc.cold_tokens)
            tiers = [_tier_cfg(plan, t, c, config.minimum_rank) for t, c in zip((lc.hot, lc.warm, lc.cold), caps)]
            be = TieredResidualLatentBackend(dh, *tiers, key_basis=cal.key_basis, value_basis=cal.value_basis)
            planned += plan.bytes_per_token * config.capacity_tokens
            allocated += be.telemetry().allocated_bytes
            for tcfg, c in zip(tiers, caps):
                if c:
                    worst = min(worst, _quality_bps(cal.key_samples, cal.key_basis, tcfg["key_rank"]),
                                _quality_bps(cal.value_samples, cal.value_basis, tcfg["value_rank"]))
            self.backends.append(be)
            self.plans.append(plan)
            self.lifecycles.append(LatentKvLifecycle(lc))
            self.basis_versions.append(cal.basis_version)
        if allocated > config.allocated_ceiling_bytes:
            raise ElasticLatentRuntimeError(f"allocation {allocated} B exceeds the ceiling {config.allocated_ceiling_bytes} B")
        self.config = config
        self._planned, self._allocated, self._worst = planned, allocated, worst
        self.steps = self._last_tr = self._last_ev = self._total_ev = 0

    def telemetry(self) -> ElasticLatentTelemetry:
        return ElasticLatentTelemetry(self.steps, self._planned, self._allocated, self._worst, self._last_tr,
                                      self._last_ev, self._total_ev)

    @torch.no_grad()
    def decode_step(self, attention, token) -> torch.Tensor:
        x = torch.as_tensor(token, dtype=torch.float32).reshape(1, -1)
        if x.shape[1] != attention.d_model:
            raise ElasticLatentRuntimeError(f"token length {x.shape[1]} != d_model {attention.d_model}")
        H, dh = attention.n_heads, attention.dh
        q, k, v = (lin(x).reshape(H, dh) for lin in (attention.w_q, attention.w_k, attention.w_v))
        ctx = torch.empty(H, dh)
        transitions = evictions = 0
        for h in range(H):
            be = self.backends[h]
            be.append(k[h], v[h])
            ctx[h] = be.attention(q[h])
            adm = self.lifecycles[h].admit(self.basis_versions[h])
            evictions += adm.evicted is not None
            transitions += len(self.lifecycles[h].rebalance())
        self.steps += 1
        self._last_tr, self._last_ev = transitions, evictions
        self._total_ev += evictions
        return attention.w_o(ctx.reshape(1, -1))[0]


class ElasticLatentEncoderSession:
    """Token-at-a-time inference through a pre-norm ``TransformerEncoder`` / ``TransformerDecoder`` whose attention
    layers read and write elastic latent KV runtimes instead of dense caches."""

    def __init__(self, encoder, config: ElasticLatentRuntimeConfig, layer_calibrations):
        blocks = list(encoder.blocks)
        if len(layer_calibrations) != len(blocks):
            raise ElasticLatentRuntimeError(f"expected calibrations for {len(blocks)} layers, got {len(layer_calibrations)}")
        self.encoder = encoder
        self.runtimes = [ElasticLatentDecodeRuntime(b.attn, config, cal) for b, cal in zip(blocks, layer_calibrations)]

    def layers(self) -> int:
        return len(self.runtimes)

    def layer_telemetry(self, layer: int):
        return self.runtimes[layer].telemetry() if 0 <= layer < len(self.runtimes) else None

    @torch.no_grad()
    def infer_step(self, x_t) -> torch.Tensor:
        x = torch.as_tensor(x_t, dtype=torch.float32).reshape(1, -1)
        for blk, rt in zip(self.encoder.blocks, self.runtimes):
            x = x + rt.decode_step(blk.attn, blk.ln1(x)[0])[None]
            x = x + blk.ffn(blk.ln2(x))
        return self.encoder.ln(x)[0]


def calibrate_heads(attention, tokens: torch.Tensor, learners=None):
    """Per-head ``HeadCalibration`` from a batch of token vectors ``[n, d_model]``: key / value rows are this layer's
    projections; the bases are each head's principal directions (or the latest COMMITTED bases of ``learners``, a list
    of ``(key CommittedBasisLearner, value CommittedBasisLearner)`` per head, completed to full rank)."""
    with torch.no_grad():
        H, dh = attention.n_heads, attention.dh
        K = attention.w_k(tokens.float()).reshape(-1, H, dh)
        V = attention.w_v(tokens.float()).reshape(-1, H, dh)
    out = []
    for h in range(H):
        ks, vs = K[:, h].contiguous(), V[:, h].contiguous()
        if learners is None:
            kb = torch.linalg.svd(ks, full_matrices=True)[2].t().contiguous()
            vb = torch.linalg.svd(vs, full_matrices=True)[2].t().contiguous()
            version = 0
        else:
            kl, vl = learners[h]
            kb, vb = complete_basis(kl.latest_committed_basis()), complete_basis(vl.latest_committed_basis())
            version = kl.versions()[-1].version
        out.append(HeadCalibration(kb, vb, ks, vs, version))
    return out

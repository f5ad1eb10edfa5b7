"""Evidence-based kernel selection: describe a problem class and a deterministic search space, rank statically valid
candidates with a cost model, MEASURE the survivors under an explicit protocol, and promote a measured, correctness-
qualified candidate into an execution plan that can be persisted and replayed.

* ``ElasticCandidate``: kernel family + revision + sorted integer parameters + determinism flag + temporary bytes.
* ``ElasticAutoTuner.rank_candidates``: enumerate, deduplicate, drop what the constraint solver rejects (and, under the
  ``deterministic-only`` objective, what is not deterministic), order by estimated cost then by the candidate itself.
* ``MeasurementProtocol``: warm-up and measured iteration counts, timing source (host wall clock or device timestamps),
  residence (resident vs transfer-inclusive) and synchronisation boundary; ``summarize`` turns integer-nanosecond samples
  into median / p95 / p99 (nearest rank) / MAD. ``measure`` is the harness: on a GPU it brackets every iteration with
  CUDA events on the current stream, on a CPU it reads the monotonic clock.
* ``RacingPolicy``: successive halving: each round keeps ``ceil(n / divisor)`` candidates (at least ``min_survivors``)
  ordered by the objective's key (latency: median, p95, p99, MAD, bytes, rank; memory: bytes first; balanced: how many
  other candidates dominate it) and multiplies the measured iterations by ``measurement_growth``.
* ``select_measured_evidence`` picks the winner; ``plan_from_evidence`` validates the evidence (correctness evidence
  present, samples > 0, median <= p95 <= p99, MAD <= p99).
* Operating modes: ``cold`` (heuristic only, nothing measured or stored), ``learn`` (explore, measure, store), ``locked``
  (persisted plan only; missing plan is an error), ``audit`` (replay and measure, never mutate).
* ``PersistedPlanStore``: one JSON file per plan key under a directory; a decoded plan must match its key, schema and
  evidence rules or it is refused.
Reference counterpart: elastic-autotuner/src/{lib,measurement_protocol,racing,measured_selection,operating_mode,
persistence,evidence_validation}.rs.
"""
from __future__ import annotations

import enum
import hashlib
import json
import math
import os
import time
from dataclasses import dataclass, field

from .hardware import HardwareCapabilities, canonical_hardware_profile_bytes

SCHEMA_VERSION = 1


class ElasticError(Exception):
    pass


class ElasticMode(enum.Enum):
    COLD = "cold"
    LEARN = "learn"
    LOCKED = "locked"
    AUDIT = "audit"


class ElasticObjective(enum.Enum):
    MIN_LATENCY = "min-latency"
    MAX_THROUGHPUT = "max-throughput"
    MIN_TEMPORARY_MEMORY = "min-temporary-memory"
    BALANCED_LATENCY_MEMORY = "balanced-latency-memory"
    DETERMINISTIC_ONLY = "deterministic-only"


@dataclass(frozen=True)
class ElasticConfig:
    mode: ElasticMode = ElasticMode.COLD
    objective: ElasticObjective = ElasticObjective.MIN_LATENCY
    max_ranked_candidates: int = 0


@dataclass(frozen=True)
class HardwareProfile:
    canonical_bytes: bytes
    schema_version: int = SCHEMA_VERSION

    @staticmethod
    def from_capabilities(hw: HardwareCapabilities) -> "HardwareProfile":
        return HardwareProfile(canonical_hardware_profile_bytes(hw))


@dataclass(frozen=True)
class ProblemClass:
    family: str
    class_key: bytes

    @staticmethod
    def gemm(m: int, n: int, k: int, dtype: str = "bf16", form: str = "nn") -> "ProblemClass":
        return ProblemClass("gemm", f"{form}:{dtype}:{m}x{n}x{k}".encode())


@dataclass(frozen=True, order=True)
class ElasticCandidate:
    kernel_family: str
    kernel_revision: bytes
    parameters: tuple                 # sorted ((name, value), ...)
    deterministic: bool
    temporary_bytes: int

    @staticmethod
    def new(kernel_family, kernel_revision, parameters, deterministic, temporary_bytes) -> "ElasticCandidate":
        items = sorted((str(k), int(v)) for k, v in (parameters.items() if isinstance(parameters, dict) else parameters))
        for a, b in zip(items, items[1:]):
            if a[0] == b[0]:
                raise ElasticError(f"duplicate tuning parameter `{a[0]}`")
        rev = kernel_revision.encode() if isinstance(kernel_revision, str) else bytes(kernel_revision)
        return ElasticCandidate(kernel_family, rev, tuple(items), bool(deterministic), int(temporary_bytes))

    def param(self, name, default=None):
        return dict(self.parameters).get(name, default)


@dataclass(frozen=True)
class ElasticMeasurement:
    sample_count: int
    median_ns: int
    p95_ns: int
    p99_ns: int
    mad_ns: int


@dataclass(frozen=True)
class ElasticEvidence:
    candidate: ElasticCandidate
    correctness_evidence: bytes
    measurement: ElasticMeasurement

    def validate(self) -> None:
        m = self.measurement
        if not self.correctness_evidence:
            raise ElasticError("correctness evidence is required")
        if m.sample_count == 0:
            raise ElasticError("at least one timing sample is required")
        if not m.median_ns <= m.p95_ns <= m.p99_ns:
            raise ElasticError("timing quantiles must satisfy median <= p95 <= p99")
        if m.mad_ns > m.p99_ns:
            raise ElasticError("timing MAD must not exceed p99 latency")


@dataclass(frozen=True)
class PlanKey:
    hardware: HardwareProfile
    problem: ProblemClass
    objective: ElasticObjective
    schema_version: int = SCHEMA_VERSION

    def digest(self) -> str:
        h = hashlib.sha256()
        for part in (str(self.schema_version).encode(), self.hardware.canonical_bytes, self.problem.family.encode(),
                     self.problem.class_key, self.objective.value.encode()):
            h.update(len(part).to_bytes(8, "little"))
            h.update(part)
        return h.hexdigest()


@dataclass(frozen=True)
class ExecutionPlan:
    hardware: HardwareProfile
    problem: ProblemClass
    objective: ElasticObjective
    evidence: ElasticEvidence
    schema_version: int = SCHEMA_VERSION

    def key(self) -> PlanKey:
        return PlanKey(self.hardware, self.problem, self.objective, self.schema_version)


@dataclass(frozen=True)
class RankedCandidate:
    estimated_cost_units: int
    candidate: ElasticCandidate


# ------------------------------------------------------------------ measurement
class TimingSource(enum.Enum):
    HOST_WALL_CLOCK = 0
    DEVICE_TIMESTAMP = 1


class ResidenceMode(enum.Enum):
    RESIDENT = 0
    TRANSFER_INCLUSIVE = 1


class SynchronizationBoundary(enum.Enum):
    PER_ITERATION = 0
    BATCH_END = 1


def _median_sorted(v):
    m = len(v) // 2
    if len(v) % 2:
        return v[m]
    a, b = v[m - 1], v[m]
    return a // 2 + b // 2 + (a % 2 + b % 2) // 2


def _nearest_rank(v, pct):
    return v[max(-(-pct * len(v) // 100), 1) - 1]


@dataclass(frozen=True)
class MeasurementProtocol:
    warmup_iterations: int
    measured_iterations: int
    timing_source: TimingSource = TimingSource.DEVICE_TIMESTAMP
    residence_mode: ResidenceMode = ResidenceMode.RESIDENT
    synchronization: SynchronizationBoundary = SynchronizationBoundary.PER_ITERATION
    schema_version: int = SCHEMA_VERSION

    def validate(self) -> None:
        if self.schema_version != SCHEMA_VERSION:
            raise ElasticError(f"measurement protocol schema mismatch: expected {SCHEMA_VERSION}, got {self.schema_version}")
        if self.measured_iterations == 0:
            raise ElasticError("measurement protocol requires at least one measured iteration")

    def summarize(self, samples_ns) -> ElasticMeasurement:
        self.validate()
        s = [int(x) for x in samples_ns]
        if len(s) != self.measured_iterations:
            raise ElasticError(f"measurement sample count mismatch: expected {self.measured_iterations}, got {len(s)}")
        w = sorted(s)
        med = _median_sorted(w)
        dev = sorted(abs(x - med) for x in s)
        return ElasticMeasurement(len(s), med, _nearest_rank(w, 95), _nearest_rank(w, 99), _median_sorted(dev))

    def canonical_bytes(self) -> bytes:
        self.validate()
        return (self.schema_version.to_bytes(4, "little") + self.warmup_iterations.to_bytes(4, "little")
                + self.measured_iterations.to_bytes(4, "little")
                + bytes([self.timing_source.value, self.residence_mode.value, self.synchronization.value]))

    def measure(self, fn, flush=None) -> ElasticMeasurement:
        """Run ``fn`` under this protocol. ``flush`` (optional) runs untimed before every measured iteration, e.g. a write
        larger than the L2 so that every sample starts cold."""
        self.validate()
        import torch
        use_dev = self.timing_source is TimingSource.DEVICE_TIMESTAMP and torch.cuda.is_available()
        for _ in range(self.warmup_iterations):
            fn()
        if use_dev:
            torch.cuda.synchronize()
        samples = []
        if use_dev:
            pairs = []
            for _ in range(self.measured_iterations):
                if flush:
                    flush()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                if self.synchronization is SynchronizationBoundary.PER_ITERATION:
                    b.synchronize()
                pairs.append((a, b))
            torch.cuda.synchronize()
            samples = [max(int(a.elapsed_time(b) * 1e6), 1) for a, b in pairs]
        else:
            for _ in range(self.measured_iterations):
                if flush:
                    flush()
                t0 = time.perf_counter_ns()
                fn()
                samples.append(max(time.perf_counter_ns() - t0, 1))
        return self.summarize(samples)


# ------------------------------------------------------------------ tuner
def _latency_key(rank, ev):
    m = ev.measurement
    return (m.median_ns, m.p95_ns, m.p99_ns, m.mad_ns, ev.candidate.temporary_bytes, rank)


def _memory_key(rank, ev):
    m = ev.measurement
    return (ev.candidate.temporary_bytes, m.median_ns, m.p95_ns, m.p99_ns, m.mad_ns, rank)


def _dominates(a: ElasticEvidence, b: ElasticEvidence) -> bool:
    la, lb, ma, mb = a.measurement.median_ns, b.measurement.median_ns, a.candidate.temporary_bytes, b.candidate.temporary_bytes
    return la <= lb and ma <= mb and (la < lb or ma < mb)


_PERMISSIONS = {   # heuristic, persisted, measure, explore, mutate, audit replay
    ElasticMode.COLD: (True, False, False, False, False, False),
    ElasticMode.LEARN: (True, True, True, True, True, False),
    ElasticMode.LOCKED: (False, True, False, False, False, False),
    ElasticMode.AUDIT: (False, True, True, False, False, True),
}


@dataclass(frozen=True)
class ModePermissions:
    may_use_heuristic_plan: bool
    may_use_persisted_plan: bool
    may_measure: bool
    may_explore: bool
    may_mutate_selection: bool
    audit_replay: bool


class ElasticAutoTuner:
    def __init__(self, config: ElasticConfig = ElasticConfig()):
        self.config = config

    # -- ranking
    def rank_candidates(self, hardware, problem, search_space, constraints, cost_model):
        """``search_space(hardware, problem) -> iterable of candidates``; ``constraints(hardware, problem, c) -> bool``;
        ``cost_model(hardware, problem, c, objective) -> int``."""
        cands = sorted(set(search_space(hardware, problem)))
        det_only = self.config.objective is ElasticObjective.DETERMINISTIC_ONLY
        ranked = [RankedCandidate(int(cost_model(hardware, problem, c, self.config.objective)), c)
                  for c in cands if constraints(hardware, problem, c) and (not det_only or c.deterministic)]
        ranked.sort(key=lambda r: (r.estimated_cost_units, r.candidate))
        k = self.config.max_ranked_candidates
        return ranked[:k] if k else ranked

    # -- evidence
    def plan_from_evidence(self, hardware, problem, evidence: ElasticEvidence) -> ExecutionPlan:
        evidence.validate()
        if self.config.objective is ElasticObjective.DETERMINISTIC_ONLY and not evidence.candidate.deterministic:
            raise ElasticError("deterministic-only objective received a non-deterministic candidate")
        return ExecutionPlan(hardware, problem, self.config.objective, evidence)

    def _matched(self, ranked, evidence, require_all):
        out = []
        for i, r in enumerate(ranked):
            recs = [e for e in evidence if e.candidate == r.candidate]
            if not recs:
                if require_all:
                    raise ElasticError(f"missing racing evidence for ranked candidate {i}")
                continue
            if len(recs) > 1:
                raise ElasticError(f"duplicate evidence for ranked candidate {i}")
            recs[0].validate()
            if self.config.objective is ElasticObjective.DETERMINISTIC_ONLY and not recs[0].candidate.deterministic:
                raise ElasticError(f"deterministic-only selection received non-deterministic candidate {i}")
            out.append((i, r, recs[0]))
        return out

    def _order(self, matched):
        obj = self.config.objective
        if obj is ElasticObjective.MIN_TEMPORARY_MEMORY:
            return sorted(matched, key=lambda t: _memory_key(t[0], t[2]))
        if obj is ElasticObjective.BALANCED_LATENCY_MEMORY:
            return sorted(matched, key=lambda t: (sum(_dominates(o[2], t[2]) for o in matched), t[0],
                                                  t[2].measurement.median_ns, t[2].candidate.temporary_bytes))
        return sorted(matched, key=lambda t: _latency_key(t[0], t[2]))

    def select_measured_evidence(self, ranked, evidence) -> ElasticEvidence:
        if not ranked:
            raise ElasticError("no ranked candidates")
        matched = self._matched(ranked, evidence, False)
        if not matched:
            raise ElasticError("no ranked candidate has been measured")
        if self.config.objective is ElasticObjective.BALANCED_LATENCY_MEMORY:
            front = [t for t in matched if not any(_dominates(o[2], t[2]) for o in matched)]
            return min(front, key=lambda t: _latency_key(t[0], t[2]))[2]
        return self._order(matched)[0][2]

    # -- modes
    def mode_permissions(self) -> ModePermissions:
        return ModePermissions(*_PERMISSIONS[self.config.mode])

    def startup_strategy(self, has_valid_persisted_plan: bool) -> str:
        m = self.config.mode
        if m is ElasticMode.COLD:
            return "qualified-heuristic"
        if m is ElasticMode.LEARN:
            return "persisted-then-explore" if has_valid_persisted_plan else "qualified-heuristic-then-explore"
        if m is ElasticMode.LOCKED:
            if not has_valid_persisted_plan:
                raise ElasticError("locked mode requires a validated persisted plan")
            return "persisted-only"
        return "audit-only"

    def load_plan_for_mode(self, cache, key: PlanKey):
        if self.config.mode is ElasticMode.COLD:
            return None
        plan = cache.load(key)
        if plan is None:
            if self.config.mode is ElasticMode.LOCKED:
                raise ElasticError("locked mode requires a validated persisted plan")
            return None
        _validate_cached(key, plan)
        return plan

    def store_plan_for_mode(self, cache, key: PlanKey, plan: ExecutionPlan) -> None:
        if not self.mode_permissions().may_mutate_selection:
            raise ElasticError(f"selection mutation is forbidden in {self.config.mode.value} mode")
        _validate_cached(key, plan)
        cache.store(key, plan)

    def require_exploration(self) -> None:
        if not self.mode_permissions().may_explore:
            raise ElasticError(f"exploration is forbidden in {self.config.mode.value} mode")

    def require_measurement(self) -> None:
        if not self.mode_permissions().may_measure:
            raise ElasticError(f"measurement is forbidden in {self.config.mode.value} mode")


def _validate_cached(key: PlanKey, plan: ExecutionPlan) -> None:
    if plan.schema_version != SCHEMA_VERSION:
        raise ElasticError(f"cached plan schema mismatch: expected {SCHEMA_VERSION}, got {plan.schema_version}")
    if plan.key() != key:
        raise ElasticError("cached plan does not match its plan-cache key")
    try:
        plan.evidence.validate()
    except ElasticError as e:
        raise ElasticError(f"cached plan contains invalid evidence: {e}") from e


@dataclass(frozen=True)
class RacingPolicy:
    survivor_divisor: int = 2
    min_survivors: int = 1
    measurement_growth: int = 2

    def validate(self) -> None:
        if self.survivor_divisor < 2:
            raise ElasticError("racing survivor divisor must be at least two")
        if self.min_survivors == 0:
            raise ElasticError("racing must retain at least one survivor")
        if self.measurement_growth == 0:
            raise ElasticError("measurement growth factor must be non-zero")

    def protocol_for_round(self, base: MeasurementProtocol, rnd: int) -> MeasurementProtocol:
        self.validate()
        base.validate()
        n = base.measured_iterations * self.measurement_growth ** rnd
        if n >= 1 << 32:
            raise ElasticError("racing measurement budget overflowed u32")
        return MeasurementProtocol(base.warmup_iterations, n, base.timing_source, base.residence_mode, base.synchronization)

    def race_round(self, tuner: ElasticAutoTuner, ranked, evidence):
        self.validate()
        if not ranked:
            raise ElasticError("racing requires at least one active candidate")
        ordered = tuner._order(tuner._matched(ranked, evidence, True))
        keep = min(max(-(-len(ranked) // self.survivor_divisor), self.min_survivors), len(ranked))
        return [t[1] for t in ordered[:keep]]


def race(tuner: ElasticAutoTuner, ranked, run, base: MeasurementProtocol, policy: RacingPolicy = RacingPolicy(),
         correctness=None, max_rounds: int = 8):
    """Successive halving to one survivor. ``run(candidate) -> callable`` builds the thing to time;
    ``correctness(candidate) -> bytes`` (non-empty) qualifies a candidate before it is timed (a failing check raises or
    returns b"" and removes it). Returns (winning evidence, evidence of the last round)."""
    tuner.require_measurement()
    alive, evidence = list(ranked), []
    for rnd in range(max_rounds):
        proto = policy.protocol_for_round(base, rnd)
        evidence, still = [], []
        for r in alive:
            proof = correctness(r.candidate) if correctness else b"unchecked"
            if not proof:
                continue
            evidence.append(ElasticEvidence(r.candidate, proof, proto.measure(run(r.candidate))))
            still.append(r)
        if not still:
            raise ElasticError("no candidate passed its correctness check")
        alive = policy.race_round(tuner, still, evidence)
        if len(alive) == 1:
            break
    return tuner.select_measured_evidence(alive, evidence), evidence


# ------------------------------------------------------------------ caches
class InMemoryPlanCache:
    def __init__(self):
        self._plans = {}

    def load(self, key: PlanKey):
        return self._plans.get(key)

    def store(self, key: PlanKey, plan: ExecutionPlan) -> None:
        self._plans[key] = plan


def encode_plan(plan: ExecutionPlan) -> bytes:
    plan.evidence.validate()
    e, m = plan.evidence, plan.evidence.measurement
    doc = {"schema_version": plan.schema_version, "hardware": plan.hardware.canonical_bytes.hex(),
           "hardware_schema": plan.hardware.schema_version, "family": plan.problem.family,
           "class_key": plan.problem.class_key.hex(), "objective": plan.objective.value,
           "candidate": {"kernel_family": e.candidate.kernel_family, "kernel_revision": e.candidate.kernel_revision.hex(),
                         "parameters": [list(p) for p in e.candidate.parameters], "deterministic": e.candidate.deterministic,
                         "temporary_bytes": e.candidate.temporary_bytes},
           "correctness_evidence": e.correctness_evidence.hex(),
           "measurement": [m.sample_count, m.median_ns, m.p95_ns, m.p99_ns, m.mad_ns]}
    body = json.dumps(doc, sort_keys=True, separators=(",", ":")).encode()
    return b"SBPLAN1\n" + hashlib.sha256(body).hexdigest().encode() + b"\n" + body


def decode_plan(data: bytes) -> ExecutionPlan:
    try:
        magic, digest, body = data.split(b"\n", 2)
        if magic != b"SBPLAN1":
            raise ValueError("bad magic")
        if hashlib.sha256(body).hexdigest().encode() != digest:
            raise ValueError("checksum mismatch")
        d = json.loads(body)
        c = d["candidate"]
        cand = ElasticCandidate.new(c["kernel_family"], bytes.fromhex(c["kernel_revision"]), [tuple(p) for p in c["parameters"]],
                                    c["deterministic"], c["temporary_bytes"])
        plan = ExecutionPlan(HardwareProfile(bytes.fromhex(d["hardware"]), d["hardware_schema"]),
                             ProblemClass(d["family"], bytes.fromhex(d["class_key"])), ElasticObjective(d["objective"]),
                             ElasticEvidence(cand, bytes.fromhex(d["correctness_evidence"]), ElasticMeasurement(*d["measurement"])),
                             d["schema_version"])
    except ElasticError:
        raise
    except Exception as e:  # noqa: BLE001  (any malformed field is the same refusal)
        raise ElasticError(f"persisted plan is malformed: {e}") from e
    if plan.schema_version != SCHEMA_VERSION:
        raise ElasticError(f"persisted plan schema mismatch: expected {SCHEMA_VERSION}, got {plan.schema_version}")
    plan.evidence.validate()
    return plan


class PersistedPlanStore:
    """Plans as files ``<sha256 of the key>.plan`` in one directory; writes are atomic (temporary file + rename)."""

    def __init__(self, directory):
        self.dir = str(directory)
        os.makedirs(self.dir, exist_ok=True)

    def _path(self, key: PlanKey) -> str:
        return os.path.join(self.dir, key.digest() + ".plan")

    def load(self, key: PlanKey):
        p = self._path(key)
        if not os.path.exists(p):
            return None
        with open(p, "rb") as f:
            return decode_plan(f.read())

    def store(self, key: PlanKey, plan: ExecutionPlan) -> None:
        tmp = self._path(key) + ".partial"
        with open(tmp, "wb") as f:
            f.write(encode_plan(plan))
        os.replace(tmp, self._path(key))

"""One machine-readable row shape for every benchmark: ``{kernel, dataset, method, seed, metric, value}`` are REQUIRED (a
row whose randomness cannot be reproduced is not a reproducible artefact, so the seed is not optional); a confidence
interval, a certificate, a preregistration record (hashes of the plan and of the code, one-shot flag: a row is
CONFIRMATORY only when it is a preregistered one-shot run) and a typed evidence statement attach optionally and are
omitted from the JSON when absent. JSON lines in, JSON lines out, with typed refusals for malformed rows.
``from_bench_line`` converts the JSON line printed by this repository's ``bench.py`` into such rows.
Reference counterpart: scirust-bench-schema/src/{lib,evidence}.rs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

EVIDENCE_KINDS = ("empirical_validation", "validated_numerical_implementation", "numerical_approximation", "exact_mathematical_result",
                  "phenomenological_model", "speculative_model", "rejection_criterion")
DISPOSITIONS = ("supports", "rejects", "inconclusive", "not_applicable")


class BenchSchemaError(ValueError):
    pass


@dataclass(frozen=True)
class ConfidenceInterval:
    lo: float
    hi: float
    level: float


@dataclass(frozen=True)
class Certificate:
    description: str
    bound_ulps: float | None = None
    determinism: str | None = None


@dataclass(frozen=True)
class Preregistration:
    preregistration_sha256: str
    code_sha256: str
    one_shot: bool
    criterion: str | None = None


@dataclass(frozen=True)
class ScientificEvidence:
    kind: str
    disposition: str
    statement: str

    def __post_init__(self):
        if self.kind not in EVIDENCE_KINDS:
            raise BenchSchemaError(f"unknown evidence kind {self.kind!r}")
        if self.disposition not in DISPOSITIONS:
            raise BenchSchemaError(f"unknown evidence disposition {self.disposition!r}")
        if not self.statement.strip():
            raise BenchSchemaError("scientific evidence statement must not be empty")

    def is_negative_result(self) -> bool:
        return self.disposition == "rejects"


def _drop_none(d: dict) -> dict:
    return {k: v for k, v in d.items() if v is not None}


@dataclass(frozen=True)
class BenchRecord:
    kernel: str
    dataset: str
    method: str
    seed: int
    metric: str
    value: float
    ci: ConfidenceInterval | None = None
    cert: Certificate | None = None
    prereg: Preregistration | None = None
    evidence: ScientificEvidence | None = None

    def __post_init__(self):
        for name in ("kernel", "dataset", "method", "metric"):
            if not isinstance(getattr(self, name), str):
                raise BenchSchemaError(f"{name} must be a string")
        if isinstance(self.seed, bool) or not isinstance(self.seed, int) or not 0 <= self.seed < 1 << 64:
            raise BenchSchemaError("seed must be an unsigned 64-bit integer")
        if isinstance(self.value, bool) or not isinstance(self.value, (int, float)):
            raise BenchSchemaError("value must be a number")

    def with_ci(self, ci): return _replace(self, ci=ci)
    def with_cert(self, cert): return _replace(self, cert=cert)
    def with_prereg(self, prereg): return _replace(self, prereg=prereg)
    def with_evidence(self, evidence): return _replace(self, evidence=evidence)

    def is_confirmatory(self) -> bool:
        return self.prereg is not None and self.prereg.one_shot

    def to_json_row(self) -> str:
        d = {"kernel": self.kernel, "dataset": self.dataset, "method": self.method, "seed": self.seed, "metric": self.metric,
             "value": float(self.value)}
        if self.ci is not None:
            d["ci"] = vars(self.ci)
        if self.cert is not None:
            d["cert"] = _drop_none(vars(self.cert))
        if self.prereg is not None:
            d["prereg"] = _drop_none(vars(self.prereg))
        if self.evidence is not None:
            d["evidence"] = vars(self.evidence)
        return json.dumps(d, separators=(",", ":"))


def _replace(rec, **kw):
    from dataclasses import replace
    return replace(rec, **kw)


def _from_dict(d: dict) -> BenchRecord:
    try:
        extra = {}
        if d.get("ci") is not None:
            extra["ci"] = ConfidenceInterval(**d["ci"])
        if d.get("cert") is not None:
            extra["cert"] = Certificate(**d["cert"])
        if d.get("prereg") is not None:
            extra["prereg"] = Preregistration(**d["prereg"])
        if d.get("evidence") is not None:
            extra["evidence"] = ScientificEvidence(**d["evidence"])
        unknown = set(d) - {"kernel", "dataset", "method", "seed", "metric", "value", "ci", "cert", "prereg", "evidence"}
        if unknown:
            raise BenchSchemaError(f"unknown field {sorted(unknown)[0]!r}")
        return BenchRecord(d["kernel"], d["dataset"], d["method"], d["seed"], d["metric"], d["value"], **extra)
    except KeyError as e:
        raise BenchSchemaError(f"missing field {e.args[0]!r}") from e
    except TypeError as e:
        raise BenchSchemaError(str(e)) from e


def to_jsonl(records) -> str:
    return "".join(r.to_json_row() + "\n" for r in records)


def write_jsonl(path, records) -> None:
    with open(path, "w", encoding="utf-8") as f:
        f.write(to_jsonl(records))


def parse_jsonl(text: str) -> list:
    out = []
    for n, line in enumerate(text.splitlines(), 1):
        if not line.strip():
            continue
        try:
            d = json.loads(line)
        except json.JSONDecodeError as e:
            raise BenchSchemaError(f"line {n}: {e}") from e
        if not isinstance(d, dict):
            raise BenchSchemaError(f"line {n}: a row is a JSON object")
        out.append(_from_dict(d))
    return out


def from_bench_line(line: str, seed: int = 0) -> list:
    """Rows for the headline value and the end-to-end value of one ``bench.py`` JSON line."""
    d = json.loads(line)
    cfg = d.get("config", {})
    dataset = f"{d.get('data', 'synthetic')}:B{cfg.get('global_batch')}xS{cfg.get('seq_len')}"
    method = f"{d.get('impl', 'ours')}:{cfg.get('parallelism', 'dp1')}:{d.get('dtype', 'bf16')}"
    kernel = cfg.get("model", "model")
    rows = [BenchRecord(kernel, dataset, method, seed, f"{d['metric']} [{d.get('unit', '')}]", float(d["value"]))]
    if isinstance(d.get("e2e"), dict) and d["e2e"].get("value") is not None:
        rows.append(BenchRecord(kernel, dataset, method + ":e2e", seed, f"{d['metric']} [{d['e2e'].get('unit', '')}]", float(d["e2e"]["value"])))
    if d.get("ms_per_step") is not None:
        rows.append(BenchRecord(kernel, dataset, method, seed, "ms_per_step", float(d["ms_per_step"])))
    return rows

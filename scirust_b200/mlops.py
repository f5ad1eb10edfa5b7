"""Deployment monitoring and packaging (scirust-mlops/src/drift.rs:1-260, shadow.rs:1-180,
ota.rs:1-200): data drift by the population stability index against a reference histogram, model
drift by windowed mean absolute error against a baseline, shadow deployment (a candidate scored
beside the production model on the same inputs, with a promote / keep / inconclusive verdict) and
signed update packages.

The update package is signed with HMAC-SHA256 from the standard library, where the reference uses a
toy keyed hash that it marks as not for production; the package layout (version, hash, bytes,
signature with key id, target device, roll-back flag) is the same.
"""
from __future__ import annotations

import hashlib
import hmac
import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

NO_DRIFT, DATA_DRIFT, MODEL_DRIFT, BOTH = "no_drift", "data_drift", "model_drift", "both"


@dataclass
class DriftReport:
    drift_type: str
    data_drift_score: float
    model_drift_score: float
    threshold: float
    details: List[Tuple[str, float]]
    sample_count: int


class DataDriftDetector:
    """PSI between a reference histogram and each full window of new samples. Below 0.1 is read as
    no drift, 0.1 to 0.25 as moderate, above 0.25 as drift that calls for retraining (drift.rs:24-30)."""

    def __init__(self, reference: Sequence[float], n_bins: int = 10, window_size: int = 200, threshold: float = 0.25):
        self.n_bins, self.window_size, self.threshold = n_bins, window_size, threshold
        self.window: List[float] = []
        self.sample_count = 0
        self.reference_hist = [0] * n_bins
        self.data_min = self.data_max = 0.0
        ref = list(reference)
        if ref and n_bins > 0 and max(ref) - min(ref) > 2.220446049250313e-16:
            self.data_min, self.data_max = min(ref), max(ref)
            self.reference_hist = self._hist(ref)

    def _hist(self, values):
        width = (self.data_max - self.data_min) / self.n_bins
        hist = [0] * self.n_bins
        for v in values:
            b = int(max(v - self.data_min, 0.0) / width)      # values below the range fall in bin 0
            hist[min(b, self.n_bins - 1)] += 1
        return hist

    def add_sample(self, value: float) -> None:
        self.window.append(float(value))
        self.sample_count += 1

    def window_fill(self) -> int:
        return len(self.window)

    def psi(self, current_hist: Sequence[int]) -> float:
        rt, ct = float(sum(self.reference_hist)), float(sum(current_hist))
        if rt < 1 or ct < 1:
            return 0.0
        out = 0.0
        for r, c in zip(self.reference_hist, current_hist):
            rp, cp = (r + 0.5) / rt, (c + 0.5) / ct           # half-count smoothing keeps the log finite
            out += (cp - rp) * math.log(cp / rp)
        return out

    def check(self) -> Optional[DriftReport]:
        if len(self.window) < self.window_size or self.data_max - self.data_min < 2.220446049250313e-16:
            return None
        score = self.psi(self._hist(self.window))
        self.window.clear()
        return DriftReport(DATA_DRIFT if score > self.threshold else NO_DRIFT, score, 0.0, self.threshold,
                           [("psi", score), ("window_size", float(self.window_size))], self.sample_count)


class ModelDriftDetector:
    """Windowed mean absolute error over (prediction, actual) pairs; drift when it exceeds
    ``threshold_factor`` times the baseline error (drift.rs:190-260)."""

    def __init__(self, window_size: int, baseline_error: float, threshold_factor: float):
        self.window_size, self.baseline_error, self.threshold_factor = window_size, baseline_error, threshold_factor
        self.window: List[Tuple[float, float]] = []
        self.sample_count = 0

    def add_observation(self, prediction: float, actual: float) -> None:
        self.window.append((float(prediction), float(actual)))
        self.sample_count += 1

    def check(self) -> Optional[DriftReport]:
        if len(self.window) < self.window_size:
            return None
        mae = sum(abs(p - a) for p, a in self.window) / len(self.window)
        rel = mae / self.baseline_error if self.baseline_error > 2.220446049250313e-16 else 1.0
        self.window.clear()
        return DriftReport(MODEL_DRIFT if rel > self.threshold_factor else NO_DRIFT, 0.0, rel, self.threshold_factor,
                           [("current_mae", mae), ("baseline_mae", self.baseline_error), ("relative_change", rel)],
                           self.sample_count)


def combine_reports(data: Optional[DriftReport], model: Optional[DriftReport]) -> str:
    """One verdict from the two detectors."""
    d = data is not None and data.drift_type == DATA_DRIFT
    m = model is not None and model.drift_type == MODEL_DRIFT
    return BOTH if d and m else DATA_DRIFT if d else MODEL_DRIFT if m else NO_DRIFT


PROMOTE, KEEP, INCONCLUSIVE = "promote", "keep", "inconclusive"
_LOWER_IS_BETTER = ("mae", "mse")


@dataclass
class ShadowResult:
    production_metric: float
    shadow_metric: float
    delta: float
    improvement: bool
    sample_count: int
    metric_type: str
    recommendation: str


class ShadowDeployment:
    """Scores a candidate beside the production model. ``metric`` is one of "mae", "mse", "accuracy"
    (|prediction - actual| < 0.5) or "f1" (binary, positive above 0.5); promotion needs a relative
    improvement above ``min_improvement`` (shadow.rs:41-180)."""

    def __init__(self, window_size: int, metric: str = "mae", min_improvement: float = 0.05):
        if metric not in ("mae", "mse", "accuracy", "f1"):
            raise ValueError(metric)
        self.window_size, self.metric, self.min_improvement = window_size, metric, min_improvement
        self.production: List[Tuple[float, float]] = []
        self.shadow: List[Tuple[float, float]] = []
        self.sample_count = 0

    def add_observation(self, production_pred: float, shadow_pred: float, actual: float) -> None:
        self.production.append((float(production_pred), float(actual)))
        self.shadow.append((float(shadow_pred), float(actual)))
        self.sample_count += 1

    def _score(self, obs) -> float:
        if not obs:
            return 0.0
        if self.metric == "mae":
            return sum(abs(p - a) for p, a in obs) / len(obs)
        if self.metric == "mse":
            return sum((p - a) ** 2 for p, a in obs) / len(obs)
        if self.metric == "accuracy":
            return sum(1 for p, a in obs if abs(p - a) < 0.5) / len(obs)
        tp = sum(1 for p, a in obs if p > 0.5 and a > 0.5)
        fp = sum(1 for p, a in obs if p > 0.5 and a <= 0.5)
        fn = sum(1 for p, a in obs if p <= 0.5 and a > 0.5)
        prec = tp / (tp + fp) if tp + fp else 0.0
        rec = tp / (tp + fn) if tp + fn else 0.0
        return 2 * prec * rec / (prec + rec) if prec + rec > 0 else 0.0

    def evaluate(self) -> Optional[ShadowResult]:
        if len(self.production) < self.window_size:
            return None
        pm, sm = self._score(self.production), self._score(self.shadow)
        delta = pm - sm if self.metric in _LOWER_IS_BETTER else sm - pm
        rel = delta / abs(pm) if abs(pm) > 2.220446049250313e-16 else 0.0
        rec = PROMOTE if rel > self.min_improvement else KEEP if rel < -self.min_improvement else INCONCLUSIVE
        self.production.clear()
        self.shadow.clear()
        return ShadowResult(pm, sm, delta, delta > 0, self.sample_count, self.metric, rec)


@dataclass
class SigningKey:
    """A named 32-byte key. ``derive`` builds one from a pass-phrase (PBKDF2-HMAC-SHA256)."""
    key_id: str
    key_bytes: bytes

    @staticmethod
    def derive(key_id: str, passphrase: str, iterations: int = 10_000) -> "SigningKey":
        return SigningKey(key_id, hashlib.pbkdf2_hmac("sha256", passphrase.encode(), key_id.encode(), iterations, 32))

    def sign(self, model_hash: bytes) -> bytes:
        return hmac.new(self.key_bytes, model_hash, hashlib.sha256).digest()

    def verify(self, model_hash: bytes, signature: bytes) -> bool:
        return hmac.compare_digest(self.sign(model_hash), signature)


@dataclass
class ModelSignature:
    model_hash: bytes
    signature: bytes
    key_id: str
    model_version: str
    timestamp: float = 0.0


@dataclass
class OtaResult:
    success: bool
    model_hash: str
    signature_valid: bool
    bytes_downloaded: int
    message: str


@dataclass
class OtaUpdate:
    """A model image with its SHA-256, a signature over the hash, the target device and a roll-back flag
    (ota.rs:82-170). ``apply`` refuses a package whose bytes, signature or key id do not check out."""
    model_bytes: bytes
    model_version: str
    target_device_id: str
    model_hash: bytes = b""
    signature: Optional[ModelSignature] = None
    rollback_on_failure: bool = True
    history: List[str] = field(default_factory=list)

    @staticmethod
    def create(model_bytes: bytes, model_version: str, target_device_id: str, key: SigningKey) -> "OtaUpdate":
        h = hashlib.sha256(model_bytes).digest()
        return OtaUpdate(model_bytes, model_version, target_device_id, h,
                         ModelSignature(h, key.sign(h), key.key_id, model_version))

    def verify(self, key: SigningKey) -> bool:
        if self.signature is None or hashlib.sha256(self.model_bytes).digest() != self.model_hash:
            return False
        return key.verify(self.model_hash, self.signature.signature) and key.key_id == self.signature.key_id

    def apply(self, key: SigningKey) -> OtaResult:
        ok = self.verify(key)
        msg = f"Model {self.model_version} applied successfully" if ok else "Signature verification failed"
        self.history.append(msg)
        return OtaResult(ok, self.model_hash.hex(), ok, len(self.model_bytes), msg)

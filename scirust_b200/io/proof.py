"""``SCIRUST-PROOF-1`` bundles for QSR1 int8 artefacts (scirust-runtime/src/proof.rs:34-200,
proofcli.rs:16-60): a canonical ``key=value`` text that pins the artefact's SHA-256, its resource
certificate (activation/accumulator scratch bytes, MAC count) and, for each seed, the FNV-1a and
SHA-256 fingerprints of the output of full-integer inference on a splitmix64-generated input.
``verify`` trusts nothing: every field is recomputed from the artefact bytes."""
from __future__ import annotations

import hashlib

import numpy as np

from .artifacts import FNV_INIT, QModel, fnv_fold_f32

_M = (1 << 64) - 1


def gen_input(seed: int, n: int) -> np.ndarray:
    s = seed & _M
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s + 0x9E3779B97F4A7C15) & _M
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
        z ^= z >> 31
        out[i] = np.float32(np.float32(z % 2000) / np.float32(1000.0) - np.float32(1.0))
    return out


def resource_certificate(model: QModel, batch: int) -> dict:
    max_w = max(max(l.in_f, l.out_f) for l in model.layers)
    max_out = max(l.out_f for l in model.layers)
    last = model.layers[-1].out_f
    act, acc, out = batch * max_w, batch * max_out * 4, batch * last * 4
    return {"layers": len(model.layers), "out_dim": last, "scratch_ram_bytes": act * 2 + acc + out,
            "mac_count": sum(batch * l.in_f * l.out_f for l in model.layers)}


def _sha_f32(x: np.ndarray) -> str:
    return hashlib.sha256(np.asarray(x, dtype="<f4").tobytes()).hexdigest()


def build_bundle(artifact: bytes, batch: int, seeds) -> str:
    model = QModel.from_bytes(artifact)
    cert = resource_certificate(model, batch)
    lines = ["format=SCIRUST-PROOF-1", f"artifact_sha256={hashlib.sha256(artifact).hexdigest()}",
             f"artifact_bytes={len(artifact)}", f"batch={batch}", f"layers={cert['layers']}",
             f"out_dim={cert['out_dim']}", f"ram_scratch_bytes={cert['scratch_ram_bytes']}",
             f"mac_count={cert['mac_count']}", f"vectors={len(seeds)}"]
    for i, seed in enumerate(seeds):
        n = batch * model.layers[0].in_f
        out = model.infer(gen_input(seed, n), batch).reshape(-1)
        lines += [f"vec.{i}.seed={seed}", f"vec.{i}.input_len={n}", f"vec.{i}.out_fp={fnv_fold_f32(FNV_INIT, out):016x}",
                  f"vec.{i}.out_sha256={_sha_f32(out)}"]
    body = "".join(l + "\n" for l in lines)
    return body + f"bundle_sha256={hashlib.sha256(body.encode()).hexdigest()}\n"


def parse_canonical(text: str) -> dict:
    kv = {}
    for line in text.splitlines():
        if not line:
            continue
        if "=" not in line:
            raise ValueError(f"line without '=': {line}")
        k, v = line.split("=", 1)
        kv[k] = v
    for k in ("format", "artifact_sha256", "artifact_bytes", "batch", "layers", "out_dim", "ram_scratch_bytes",
              "mac_count", "vectors"):
        if k not in kv:
            raise ValueError(f"missing field {k}")
    return kv


def verify_bundle(text: str, artifact: bytes) -> list:
    """Returns the list of mismatches (empty = verified)."""
    kv = parse_canonical(text)
    errs = []
    if kv["format"] != "SCIRUST-PROOF-1":
        return [f"unknown format {kv['format']}"]
    try:
        batch = int(kv["batch"])
        seeds = [int(kv[f"vec.{i}.seed"]) for i in range(int(kv["vectors"]))]
    except (KeyError, ValueError) as e:
        return [f"malformed bundle: {e}"]
    expect = parse_canonical(build_bundle(artifact, batch, seeds))
    for k, v in expect.items():
        if kv.get(k) != v:
            errs.append(f"{k}: claimed {kv.get(k)!r}, recomputed {v!r}")
    return errs

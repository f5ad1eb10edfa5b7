"""Ahead-of-time compiler for small static MLPs: a layer list plus a little-endian fp32 weight stream become ONE
self-contained C++ translation unit (weights baked in as exact hexadecimal float literals, fixed loop bounds, no
allocation, no dependency), optionally compiled to a shared object and loaded back for inference on hosts that have no
Python ML stack. Weight stream layout per ``Linear``: ``in*out`` weights in ``[in, out]`` row-major order, then ``out``
biases; ``y = x @ W + b`` with the inner sum accumulated in index order starting from the bias, so the result is
reproducible bit for bit by ``reference_forward``. Exported symbols: ``static_model_in_dim``, ``static_model_out_dim``,
``static_model_forward(const float* in, float* out, int batch)``.
Reference counterpart: scirust-core/src/aot.rs:4-182 (which emits Rust source; C++ is what this toolchain compiles).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
import subprocess
import tempfile
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Linear:
    in_features: int
    out_features: int


@dataclass(frozen=True)
class ReLU:
    pass


def _dims(layers):
    lin = [l for l in layers if isinstance(l, Linear)]
    if not lin:
        raise ValueError("a static pipeline needs at least one Linear layer")
    cur = lin[0].in_features
    for l in layers:
        if isinstance(l, Linear):
            if l.in_features != cur:
                raise ValueError(f"Linear expects {l.in_features} inputs but the previous layer produces {cur}")
            cur = l.out_features
    return lin[0].in_features, cur


def expected_weight_bytes(layers) -> int:
    return 4 * sum(l.in_features * l.out_features + l.out_features for l in layers if isinstance(l, Linear))


def split_weights(layers, weights_bytes: bytes):
    """-> list of (W [in, out], b [out]) per Linear; raises on a short or over-long stream."""
    if len(weights_bytes) != expected_weight_bytes(layers):
        raise ValueError(f"weight stream has {len(weights_bytes)} bytes, the layers need {expected_weight_bytes(layers)}")
    out, off = [], 0
    for l in layers:
        if isinstance(l, Linear):
            nw = l.in_features * l.out_features
            w = np.frombuffer(weights_bytes, "<f4", nw, off).reshape(l.in_features, l.out_features)
            off += 4 * nw
            b = np.frombuffer(weights_bytes, "<f4", l.out_features, off)
            off += 4 * l.out_features
            out.append((w, b))
    return out


def pack_weights(pairs) -> bytes:
    """Inverse of ``split_weights``: [(W [in, out], b [out]), ...] -> byte stream."""
    return b"".join(np.ascontiguousarray(w, "<f4").tobytes() + np.ascontiguousarray(b, "<f4").tobytes() for w, b in pairs)


def _lit(v) -> str:
    v = float(np.float32(v))
    if v != v or v in (float("inf"), float("-inf")):
        raise ValueError("weights must be finite")
    return f"{v.hex()}f"


def generate_static_pipeline(layers, weights_bytes: bytes) -> str:
    in_dim, out_dim = _dims(layers)
    params = split_weights(layers, weights_bytes)
    widest = max([in_dim] + [l.out_features for l in layers if isinstance(l, Linear)])
    src = ["// Generated static inference pipeline: weights are compile-time constants.",
           f"// sha256(weights) = {hashlib.sha256(weights_bytes).hexdigest()}",
           f"static const int IN_DIM = {in_dim};", f"static const int OUT_DIM = {out_dim};", ""]
    k = 0
    for i, l in enumerate(layers):
        if isinstance(l, Linear):
            w, b = params[k]
            k += 1
            rows = ",\n".join("    {" + ", ".join(_lit(x) for x in row) + "}" for row in w)
            src.append(f"static const float weight_{i}[{l.in_features}][{l.out_features}] = {{\n{rows}\n}};")
            src.append(f"static const float bias_{i}[{l.out_features}] = {{" + ", ".join(_lit(x) for x in b) + "};")
    src += ["", 'extern "C" int static_model_in_dim() { return IN_DIM; }',
            'extern "C" int static_model_out_dim() { return OUT_DIM; }', "",
            'extern "C" void static_model_forward(const float* in, float* out, int batch) {',
            f"  float a[{widest}], c[{widest}];", "  for (int n = 0; n < batch; ++n) {",
            "    float* cur = a; float* nxt = c;",
            "    for (int i = 0; i < IN_DIM; ++i) cur[i] = in[n * IN_DIM + i];"]
    cur = in_dim
    for i, l in enumerate(layers):
        if isinstance(l, Linear):
            src += [f"    for (int o = 0; o < {l.out_features}; ++o) {{", f"      float acc = bias_{i}[o];",
                    f"      for (int i = 0; i < {l.in_features}; ++i) acc += cur[i] * weight_{i}[i][o];",
                    "      nxt[o] = acc;", "    }", "    { float* t = cur; cur = nxt; nxt = t; }"]
            cur = l.out_features
        elif isinstance(l, ReLU):
            src.append(f"    for (int d = 0; d < {cur}; ++d) if (cur[d] < 0.0f) cur[d] = 0.0f;")
        else:
            raise ValueError(f"unsupported layer {l!r}")
    src += ["    for (int o = 0; o < OUT_DIM; ++o) out[n * OUT_DIM + o] = cur[o];", "  }", "}", ""]
    return "\n".join(src)


def reference_forward(layers, weights_bytes: bytes, x) -> np.ndarray:
    """The same arithmetic in the same order in fp32 (no fused multiply-add), for checking a compiled artefact."""
    params = iter(split_weights(layers, weights_bytes))
    cur = np.asarray(x, np.float32)
    for l in layers:
        if isinstance(l, Linear):
            w, b = next(params)
            acc = np.broadcast_to(b, (cur.shape[0], l.out_features)).astype(np.float32).copy()
            for i in range(l.in_features):
                acc = (acc + (cur[:, i:i + 1] * w[i][None, :]).astype(np.float32)).astype(np.float32)
            cur = acc
        else:
            cur = np.maximum(cur, np.float32(0))
    return cur


class CompiledPipeline:
    def __init__(self, so_path: str):
        self.path = so_path
        self._lib = ctypes.CDLL(so_path)
        self._lib.static_model_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        self.in_dim = self._lib.static_model_in_dim()
        self.out_dim = self._lib.static_model_out_dim()

    def __call__(self, x) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        if x.ndim != 2 or x.shape[1] != self.in_dim:
            raise ValueError(f"expected [batch, {self.in_dim}] inputs, got {x.shape}")
        out = np.empty((x.shape[0], self.out_dim), np.float32)
        self._lib.static_model_forward(x.ctypes.data, out.ctypes.data, x.shape[0])
        return out


def compile_pipeline(layers, weights_bytes: bytes, out_dir: str | None = None, cxx: str = "g++") -> CompiledPipeline:
    """Write the source, build it with ``-ffp-contract=off`` (so no fused multiply-add changes the rounding) and load it."""
    out_dir = out_dir or tempfile.mkdtemp(prefix="static_pipeline_")
    os.makedirs(out_dir, exist_ok=True)
    src = generate_static_pipeline(layers, weights_bytes)
    tag = hashlib.sha256(src.encode()).hexdigest()[:16]
    cpp, so = os.path.join(out_dir, f"static_model_{tag}.cpp"), os.path.join(out_dir, f"static_model_{tag}.so")
    with open(cpp, "w") as f:
        f.write(src)
    subprocess.run([cxx, "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-o", so, cpp], check=True, capture_output=True)
    return CompiledPipeline(so)


def from_torch_sequential(seq):
    """``torch.nn.Sequential`` of ``Linear`` (with bias) / ``ReLU`` -> (layers, weight stream)."""
    import torch
    layers, pairs = [], []
    for m in seq:
        if isinstance(m, torch.nn.Linear):
            layers.append(Linear(m.in_features, m.out_features))
            b = m.bias.detach() if m.bias is not None else torch.zeros(m.out_features)
            pairs.append((m.weight.detach().t().contiguous().float().numpy(), b.float().numpy()))
        elif isinstance(m, torch.nn.ReLU):
            layers.append(ReLU())
        else:
            raise ValueError(f"unsupported module {type(m).__name__}")
    return layers, pack_weights(pairs)

"""Inference artefacts of the reference runtime, read and written byte-compatibly.

* **SRT1** weight container (scirust-runtime/src/lib.rs:13-77): ``b"SRT1"``, ``u32 n``, then per key
  in sorted order ``u32 klen, key, u32 rows, u32 cols, u64 len, f32[len]`` (little-endian).
* **manifest** text (scirust-runtime/src/lib.rs:196-340): one layer per line -
  ``linear I O`` / ``relu`` / ``sigmoid`` / ``layernorm D eps`` / ``batchnorm2d C`` /
  ``conv2d ic oc k s same|valid h w`` / ``maxpool2d k s c h w``; ``#`` comments and blank lines skipped.
* **QSR1** int8 model (scirust-runtime/src/quant.rs:110-232): ``b"QSR1"``, ``u32 n_layers``; per
  layer ``u32 tag(0), u32 in_f, u32 out_f, f32 s_in, u8 relu_after, u32 ns, f32[ns] scales,
  u32 nw, i8[nw] weights, u32 nb, i32[nb] bias``; full-integer inference with fixed-point
  requantisation (quant.rs:35-66, 236-285).
* FNV-1a fingerprints over fp32 bit patterns (scirust-runtime/src/lib.rs fnv_*).

Parsers raise ``ValueError`` on truncated or inconsistent input.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------- SRT1


def srt1_to_bytes(sd: dict) -> bytes:
    out = [b"SRT1", struct.pack("<I", len(sd))]
    for k in sorted(sd, key=lambda s: s.encode("utf-8")):
        t = torch.as_tensor(sd[k]).detach().float().cpu()
        if t.dim() == 1:
            t = t.reshape(1, -1)
        if t.dim() != 2:
            raise ValueError(f"SRT1 holds 2-D tensors; {k!r} has shape {tuple(t.shape)}")
        kb = k.encode("utf-8")
        a = t.contiguous().numpy().astype("<f4", copy=False)
        out += [struct.pack("<I", len(kb)), kb, struct.pack("<IIQ", t.shape[0], t.shape[1], a.size), a.tobytes()]
    return b"".join(out)


def srt1_from_bytes(buf: bytes) -> dict:
    if len(buf) < 8 or buf[:4] != b"SRT1":
        raise ValueError("bad SRT1 magic")
    p = 4

    def need(k):
        if p + k > len(buf):
            raise ValueError("SRT1 truncated")
    need(4)
    (n,) = struct.unpack_from("<I", buf, p)
    p += 4
    sd = {}
    for _ in range(n):
        need(4)
        (klen,) = struct.unpack_from("<I", buf, p)
        p += 4
        need(klen)
        try:
            key = buf[p:p + klen].decode("utf-8")
        except UnicodeDecodeError:
            raise ValueError("SRT1 key is not utf-8") from None
        p += klen
        need(16)
        rows, cols, dlen = struct.unpack_from("<IIQ", buf, p)
        p += 16
        need(dlen * 4)
        if rows * cols != dlen:
            raise ValueError(f"SRT1 entry {key!r}: {rows}x{cols} != {dlen}")
        a = np.frombuffer(buf, dtype="<f4", count=dlen, offset=p).copy()
        p += dlen * 4
        sd[key] = torch.from_numpy(a).reshape(rows, cols)
    return sd


def save_weights(sd: dict, path) -> None:
    Path(path).write_bytes(srt1_to_bytes(sd))


def load_weights(path) -> dict:
    return srt1_from_bytes(Path(path).read_bytes())


# --------------------------------------------------------------------------- FNV fingerprints
FNV_INIT = 0xCBF29CE484222325
FNV_PRIME = 0x100000001B3
_M64 = (1 << 64) - 1


def fnv_fold_f32(fp: int, data) -> int:
    bits = np.asarray(torch.as_tensor(data).detach().float().cpu().contiguous().numpy()).view("<u4").reshape(-1)
    for b in bits.tolist():
        fp = ((fp ^ b) * FNV_PRIME) & _M64
    return fp


def fnv_bytes(data: bytes) -> int:
    fp = FNV_INIT
    for b in data:
        fp = ((fp ^ b) * FNV_PRIME) & _M64
    return fp


# --------------------------------------------------------------------------- manifest
@dataclass
class LayerSpec:
    kind: str
    args: tuple = ()


def _fmt_f32(x: float) -> str:
    """Shortest decimal that round-trips through fp32 (how Rust's Display prints an f32)."""
    x32 = np.float32(x)
    if x32 == np.floor(x32) and abs(x32) < 1e16:
        return str(int(x32))
    return np.format_float_positional(x32, unique=True, trim="-")


def write_manifest(specs) -> str:
    lines = []
    for s in specs:
        k, a = s.kind, s.args
        if k == "linear":
            lines.append(f"linear {a[0]} {a[1]}")
        elif k in ("relu", "sigmoid"):
            lines.append(k)
        elif k == "layernorm":
            lines.append(f"layernorm {a[0]} {_fmt_f32(a[1])}")
        elif k == "batchnorm2d":
            lines.append(f"batchnorm2d {a[0]}")
        elif k == "conv2d":
            ic, oc, ks, st, same, h, w = a
            lines.append(f"conv2d {ic} {oc} {ks} {st} {'same' if same else 'valid'} {h} {w}")
        elif k == "maxpool2d":
            lines.append("maxpool2d " + " ".join(str(v) for v in a))
        else:
            raise ValueError(f"unknown layer kind {k!r}")
    return "".join(l + "\n" for l in lines)


def parse_manifest(text: str):
    out = []
    for i, raw in enumerate(text.splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        t = line.split()

        def num(s):
            try:
                v = int(s)
                if v < 0:
                    raise ValueError
                return v
            except ValueError:
                raise ValueError(f"line {i}: invalid integer {s!r}") from None

        def need(n):
            if len(t) < n:
                raise ValueError(f"line {i}: layer {t[0]!r} expects {n - 1} fields, got {len(t) - 1}")
        k = t[0]
        if k == "linear":
            need(3)
            out.append(LayerSpec("linear", (num(t[1]), num(t[2]))))
        elif k in ("relu", "sigmoid"):
            out.append(LayerSpec(k))
        elif k == "layernorm":
            need(3)
            try:
                eps = float(t[2])
            except ValueError:
                raise ValueError(f"line {i}: invalid float {t[2]!r}") from None
            out.append(LayerSpec("layernorm", (num(t[1]), eps)))
        elif k == "batchnorm2d":
            need(2)
            out.append(LayerSpec("batchnorm2d", (num(t[1]),)))
        elif k == "conv2d":
            need(8)
            if t[5] not in ("same", "valid"):
                raise ValueError(f"line {i}: padding {t[5]!r}")
            out.append(LayerSpec("conv2d", (num(t[1]), num(t[2]), num(t[3]), num(t[4]), t[5] == "same", num(t[6]),
                                            num(t[7]))))
        elif k == "maxpool2d":
            need(6)
            out.append(LayerSpec("maxpool2d", tuple(num(v) for v in t[1:6])))
        else:
            raise ValueError(f"line {i}: unknown layer {k!r}")
    return out


# --------------------------------------------------------------------------- QSR1
@dataclass
class QLinear:
    in_f: int
    out_f: int
    s_in: float
    relu_after: bool
    scales: np.ndarray      # f32 [out_f]
    w_q: np.ndarray         # i8 [in_f * out_f], row-major [in, out]
    bias_i32: np.ndarray    # i32 [out_f]


@dataclass
class QModel:
    layers: list = field(default_factory=list)

    def to_bytes(self) -> bytes:
        b = [b"QSR1", struct.pack("<I", len(self.layers))]
        for l in self.layers:
            b.append(struct.pack("<IIIfB", 0, l.in_f, l.out_f, float(np.float32(l.s_in)), 1 if l.relu_after else 0))
            b.append(struct.pack("<I", len(l.scales)) + np.asarray(l.scales, dtype="<f4").tobytes())
            b.append(struct.pack("<I", len(l.w_q)) + np.asarray(l.w_q, dtype="i1").tobytes())
            b.append(struct.pack("<I", len(l.bias_i32)) + np.asarray(l.bias_i32, dtype="<i4").tobytes())
        return b"".join(b)

    @staticmethod
    def from_bytes(buf: bytes) -> "QModel":
        if len(buf) < 8 or buf[:4] != b"QSR1":
            raise ValueError("bad QSR1 magic")
        p = 4

        def take(fmt):
            nonlocal p
            size = struct.calcsize(fmt)
            if p + size > len(buf):
                raise ValueError(f"QSR1 truncated: {size} byte(s) needed at offset {p} (length {len(buf)})")
            v = struct.unpack_from(fmt, buf, p)
            p += size
            return v

        def arr(dtype, n):
            nonlocal p
            size = np.dtype(dtype).itemsize * n
            if p + size > len(buf):
                raise ValueError(f"QSR1 truncated: {size} byte(s) needed at offset {p} (length {len(buf)})")
            a = np.frombuffer(buf, dtype=dtype, count=n, offset=p).copy()
            p += size
            return a
        (n,) = take("<I")
        layers = []
        for _ in range(n):
            (tag,) = take("<I")
            if tag != 0:
                raise ValueError(f"unknown QSR1 layer tag {tag}")
            in_f, out_f, s_in, relu = take("<IIfB")
            (ns,) = take("<I")
            scales = arr("<f4", ns)
            (nw,) = take("<I")
            w_q = arr("i1", nw)
            (nb,) = take("<I")
            bias = arr("<i4", nb)
            if ns != out_f or nb != out_f or nw != in_f * out_f:
                raise ValueError(f"inconsistent QSR1 layer: out_f={out_f}, scales={ns}, bias={nb}, w_q={nw}")
            layers.append(QLinear(in_f, out_f, s_in, relu == 1, scales, w_q, bias))
        return QModel(layers)

    def save(self, path) -> bytes:
        b = self.to_bytes()
        Path(path).write_bytes(b)
        return b

    @staticmethod
    def load(path) -> "QModel":
        return QModel.from_bytes(Path(path).read_bytes())

    # full-integer inference (scirust-runtime/src/quant.rs:236-285)
    def infer(self, x, batch: int) -> np.ndarray:
        if not self.layers:
            raise ValueError("empty QModel")
        x = np.asarray(x, dtype=np.float32).reshape(batch, -1)
        cur = quantize_tensor(x, self.layers[0].s_in)
        for li, l in enumerate(self.layers):
            w = l.w_q.reshape(l.in_f, l.out_f).astype(np.int64)
            acc = np.clip(cur.astype(np.int64) @ w, -2**31, 2**31 - 1).astype(np.int32)
            a = (acc + l.bias_i32[None, :].astype(np.int32)).astype(np.int32)  # i32 wrapping add
            if li + 1 == len(self.layers):
                return (a.astype(np.float32) * np.float32(l.s_in)) * l.scales[None, :].astype(np.float32)
            s_out = self.layers[li + 1].s_in
            q = np.empty_like(a, dtype=np.int8)
            for o in range(l.out_f):
                m, sh = quantize_multiplier((float(np.float32(l.s_in)) * float(l.scales[o])) / float(np.float32(s_out)))
                r = requant_i32(a[:, o].astype(np.int64), m, sh)
                if l.relu_after:
                    r = np.maximum(r, 0)
                q[:, o] = np.clip(r, -128, 127).astype(np.int8)
            cur = q
        raise AssertionError("unreachable")


def quantize_tensor(x: np.ndarray, scale: float) -> np.ndarray:
    """round-half-away-from-zero(x / scale) clamped to int8 (Rust ``f32::round``)."""
    v = np.asarray(x, dtype=np.float32) / np.float32(scale)
    r = np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5)))
    # f32::round rounds half away from zero exactly; floor(v+0.5) can differ when v+0.5 rounds up
    frac_issue = (np.abs(v) < 8388608.0) & (np.abs(r - v) > 0.5)
    r = np.where(frac_issue, np.trunc(v), r)
    return np.clip(r, -128.0, 127.0).astype(np.int8)


def quantize_multiplier(m: float):
    if m <= 0.0:
        return 0, 0
    frac, shift = m, 0
    while frac < 0.5:
        frac *= 2.0
        shift += 1
    mult = int(np.floor(frac * float(1 << 31) + 0.5))
    if mult >= (1 << 31):
        mult = 1 << 30
        shift = max(shift - 1, 0)
    return mult, shift


def requant_i32(acc, mult: int, shift: int):
    total = 31 + shift
    if total >= 63:
        return np.zeros_like(acc)
    return (acc * mult + (1 << (total - 1))) >> total

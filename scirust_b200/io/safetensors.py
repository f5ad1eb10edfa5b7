"""safetensors reader/writer compatible with the reference's own implementation
(scirust-core/src/io/safetensors.rs:61-200): ``u64 LE header length``, a compact JSON header with
no spaces (``"name":{"dtype":"F32","shape":[r,c],"data_offsets":[a,b]}`` in the given order), then
little-endian fp32 payloads. The writer emits exactly those bytes, so a file written here is
byte-identical to one written by the reference from the same tensors; the reader additionally
accepts N-D shapes, ``__metadata__`` and the F16/BF16/F64/I8/I32/I64/U8 dtypes that other
producers write. Malformed input raises ``ValueError`` (never an unchecked exception), as the
reference's parser returns ``Err`` (fuzz target fuzz/fuzz_targets/safetensors.rs)."""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np
import torch

MAX_HEADER_SIZE = 16 * 1024 * 1024

_DT = {"F32": (np.dtype("<f4"), torch.float32), "F64": (np.dtype("<f8"), torch.float64),
       "F16": (np.dtype("<f2"), torch.float16), "BF16": (np.dtype("<u2"), torch.bfloat16),
       "I8": (np.dtype("i1"), torch.int8), "U8": (np.dtype("u1"), torch.uint8),
       "I32": (np.dtype("<i4"), torch.int32), "I64": (np.dtype("<i8"), torch.int64)}


def _escape(s: str) -> str:
    return s.replace("\\", "\\\\").replace('"', '\\"')


def serialize(tensors, metadata: dict | None = None) -> bytes:
    """``tensors``: ordered iterable of (name, tensor). fp32 tensors; 1-D tensors are written as
    ``[1, n]`` like the reference's 2-D tensor type, N-D shapes are kept."""
    items = list(tensors.items()) if isinstance(tensors, dict) else list(tensors)
    entries, blobs, off = [], [], 0
    if metadata:
        md = ",".join(f'"{_escape(str(k))}":"{_escape(str(v))}"' for k, v in metadata.items())
        entries.append(f'"__metadata__":{{{md}}}')
    for name, t in items:
        a = torch.as_tensor(t).detach().to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
        shape = list(a.shape)
        if len(shape) == 0:
            shape = [1, 1]
        elif len(shape) == 1:
            shape = [1, shape[0]]
        n = a.size * 4
        entries.append(f'"{_escape(name)}":{{"dtype":"F32","shape":[{",".join(str(s) for s in shape)}],'
                       f'"data_offsets":[{off},{off + n}]}}')
        blobs.append(a.tobytes())
        off += n
    header = ("{" + ",".join(entries) + "}").encode("utf-8")
    return struct.pack("<Q", len(header)) + header + b"".join(blobs)


def save_safetensors(tensors, path, metadata: dict | None = None) -> None:
    Path(path).write_bytes(serialize(tensors, metadata))


def deserialize(data: bytes, with_metadata: bool = False):
    if len(data) < 8:
        raise ValueError("safetensors: file too short")
    (hlen,) = struct.unpack("<Q", data[:8])
    if hlen > MAX_HEADER_SIZE:
        raise ValueError(f"safetensors: header too large ({hlen} bytes)")
    if 8 + hlen > len(data):
        raise ValueError("safetensors: invalid header size")
    try:
        header = json.loads(data[8:8 + hlen].decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as e:
        raise ValueError(f"safetensors: bad header: {e}") from None
    if not isinstance(header, dict):
        raise ValueError("safetensors: header is not an object")
    body = memoryview(data)[8 + hlen:]
    out, meta = {}, {}
    for name, info in header.items():
        if name == "__metadata__":
            if isinstance(info, dict):
                meta = {str(k): str(v) for k, v in info.items()}
            continue
        try:
            dt, shape, (a, b) = info["dtype"], [int(s) for s in info["shape"]], info["data_offsets"]
            a, b = int(a), int(b)
        except (KeyError, TypeError, ValueError):
            raise ValueError(f"safetensors: malformed entry {name!r}") from None
        if dt not in _DT:
            raise ValueError(f"safetensors: unsupported dtype {dt!r} for {name!r}")
        npdt, tdt = _DT[dt]
        count = 1
        for s in shape:
            if s < 0:
                raise ValueError(f"safetensors: negative dimension in {name!r}")
            count *= s
        if a < 0 or b < a or b > len(body) or (b - a) != count * npdt.itemsize:
            raise ValueError(f"safetensors: bad data_offsets for {name!r}")
        arr = np.frombuffer(body[a:b], dtype=npdt).copy()
        t = torch.from_numpy(arr)
        if dt == "BF16":
            t = t.view(torch.int16).view(torch.bfloat16)
        out[name] = t.reshape(shape)
    return (out, meta) if with_metadata else out


def load_safetensors(path, with_metadata: bool = False):
    return deserialize(Path(path).read_bytes(), with_metadata)


def header_order(data: bytes) -> list[str]:
    """Tensor names in file order (the reference writes SciAgent checkpoints with sorted keys)."""
    (hlen,) = struct.unpack("<Q", data[:8])
    return [k for k in json.loads(data[8:8 + hlen].decode("utf-8")) if k != "__metadata__"]

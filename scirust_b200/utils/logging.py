"""Training telemetry (scirust-core/src/logging.rs:36-327): a CSV logger with the columns
``step,tag,value,timestamp`` and a TensorBoard event-file writer (TFRecord framing with masked
CRC32C, hand-encoded ``Event``/``Summary`` protobuf messages - no TensorFlow dependency)."""
from __future__ import annotations

import os
import struct
import time
from pathlib import Path


class TrainingLogger:
    def __init__(self, path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        new = not self.path.exists()
        self.f = open(self.path, "a", buffering=1)
        if new:
            self.f.write("step,tag,value,timestamp\n")

    def log(self, step: int, tag: str, value: float, timestamp: float | None = None):
        ts = time.time() if timestamp is None else timestamp
        self.f.write(f"{int(step)},{tag},{float(value)!r},{ts:.3f}\n")

    def close(self):
        self.f.close()


_CRC_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _CRC_TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


class TensorBoardWriter:
    def __init__(self, logdir):
        Path(logdir).mkdir(parents=True, exist_ok=True)
        self.path = Path(logdir) / f"events.out.tfevents.{int(time.time())}.{os.uname().nodename}"
        self.f = open(self.path, "wb")
        self._write(_field(1, 1, struct.pack("<d", time.time())) + _field(3, 2, _varint(len(b"brain.Event:2")) + b"brain.Event:2"))

    def _write(self, event: bytes):
        hdr = struct.pack("<Q", len(event))
        self.f.write(hdr + struct.pack("<I", _masked(hdr)) + event + struct.pack("<I", _masked(event)))
        self.f.flush()

    def add_scalar(self, tag: str, value: float, step: int, wall_time: float | None = None):
        t = tag.encode()
        val = _field(1, 2, _varint(len(t)) + t) + _field(2, 5, struct.pack("<f", float(value)))
        summary = _field(1, 2, _varint(len(val)) + val)
        ev = (_field(1, 1, struct.pack("<d", time.time() if wall_time is None else wall_time)) +
              _field(2, 0, _varint(int(step))) + _field(5, 2, _varint(len(summary)) + summary))
        self._write(ev)

    def close(self):
        self.f.close()


def read_tfrecords(path):
    """Yield the payload of every record, verifying both checksums."""
    data = Path(path).read_bytes()
    p = 0
    while p < len(data):
        (n,) = struct.unpack_from("<Q", data, p)
        if struct.unpack_from("<I", data, p + 8)[0] != _masked(data[p:p + 8]):
            raise ValueError("corrupt record length")
        body = data[p + 12:p + 12 + n]
        if struct.unpack_from("<I", data, p + 12 + n)[0] != _masked(body):
            raise ValueError("corrupt record body")
        yield body
        p += 16 + n

"""Verifiable inference and the hash-chained attestation log.

``VModel`` is an integer linear layer ``Y = W X`` over the prime field GF(2^31 - 1), committed by the SHA-256 of its
weights. A claimed batched output is checked without recomputing it by Freivalds' test ``W (X r) == Y r`` with the
challenge ``r`` derived (Fiat-Shamir) from the commitment, the input and the claimed output; a wrong output passes a
challenge with probability at most 1/p. ``AttestationLog`` chains inference events
``entry_n = H(entry_{n-1} | seq | commitment | H(input) | H(output))`` so that altering, dropping or reordering an
event changes the head; ``attest_and_record`` appends only outputs that pass the check.

Counterparts in the reference: scirust-runtime/src/vinfer.rs (field, commitment, Freivalds verifier) and
scirust-runtime/src/attest.rs (log, chain rule, ``attest_and_record``); `scirust attest` of the CLI
(scirust-cli/src/synergy.rs:163-230) drives both.
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field

P = 2_147_483_647            # 2^31 - 1: products of two residues fit a signed 64-bit integer
GENESIS = bytes(32)


def _le64(x: int) -> bytes:
    return struct.pack("<q", x)


def hash_i64(xs) -> bytes:
    h = hashlib.sha256()
    for x in xs:
        h.update(_le64(int(x)))
    return h.digest()


class VModel:
    """Row-major ``(out, in)`` weights reduced into ``[0, p)``."""

    def __init__(self, w, out: int, inn: int):
        w = [int(v) % P for v in w]
        if len(w) != out * inn:
            raise ValueError("VModel: weight count must be out * in")
        self.w, self.out, self.inn = w, out, inn

    def commit(self) -> bytes:
        h = hashlib.sha256()
        h.update(struct.pack("<Q", self.out))
        h.update(struct.pack("<Q", self.inn))
        for v in self.w:
            h.update(_le64(v))
        return h.digest()

    def infer(self, x, batch: int):
        """``x`` row-major ``(in, batch)`` -> row-major ``(out, batch)``."""
        if len(x) != self.inn * batch:
            raise ValueError("VModel.infer: input size")
        y = [0] * (self.out * batch)
        for o in range(self.out):
            row = self.w[o * self.inn:(o + 1) * self.inn]
            for j in range(batch):
                acc = 0
                for i, wv in enumerate(row):
                    acc = (acc + wv * (int(x[i * batch + j]) % P)) % P
                y[o * batch + j] = acc
        return y


def _challenge(commitment: bytes, x, y, batch: int, k: int):
    """Fiat-Shamir: the k-th challenge vector of ``batch`` field elements."""
    seed = hashlib.sha256(commitment + hash_i64(x) + hash_i64(y) + struct.pack("<Q", k)).digest()
    out = []
    ctr = 0
    while len(out) < batch:
        block = hashlib.sha256(seed + struct.pack("<Q", ctr)).digest()
        for i in range(0, 32, 8):
            if len(out) < batch:
                out.append(int.from_bytes(block[i:i + 8], "little") % P)
        ctr += 1
    return out


def verify_inference(model: VModel, x, batch: int, y, challenges: int = 2) -> bool:
    """True when ``y`` is ``model.infer(x, batch)`` (up to the soundness error ``p^-challenges``); costs
    ``O(out*in + (in + out)*batch)`` per challenge instead of ``O(out*in*batch)``."""
    if len(x) != model.inn * batch or len(y) != model.out * batch:
        return False
    c = model.commit()
    for k in range(challenges):
        r = _challenge(c, x, y, batch, k)
        xr = [sum((int(x[i * batch + j]) % P) * r[j] for j in range(batch)) % P for i in range(model.inn)]
        yr = [sum((int(y[o * batch + j]) % P) * r[j] for j in range(batch)) % P for o in range(model.out)]
        for o in range(model.out):
            row = model.w[o * model.inn:(o + 1) * model.inn]
            if sum(wv * xv for wv, xv in zip(row, xr)) % P != yr[o]:
                return False
    return True


@dataclass
class InferenceEvent:
    seq: int
    model_commitment: bytes
    input_hash: bytes
    output_hash: bytes
    entry_hash: bytes


@dataclass
class AttestationLog:
    events: list = field(default_factory=list)
    head: bytes = GENESIS

    @staticmethod
    def _entry(prev: bytes, seq: int, commitment: bytes, ih: bytes, oh: bytes) -> bytes:
        return hashlib.sha256(prev + struct.pack("<Q", seq) + commitment + ih + oh).digest()

    def record(self, model_commitment: bytes, x, y) -> bytes:
        seq = len(self.events)
        ih, oh = hash_i64(x), hash_i64(y)
        entry = self._entry(self.head, seq, model_commitment, ih, oh)
        self.events.append(InferenceEvent(seq, model_commitment, ih, oh, entry))
        self.head = entry
        return entry

    def verify_chain(self) -> bool:
        """Recompute every link from the genesis head."""
        prev = GENESIS
        for i, e in enumerate(self.events):
            if e.seq != i or self._entry(prev, i, e.model_commitment, e.input_hash, e.output_hash) != e.entry_hash:
                return False
            prev = e.entry_hash
        return prev == self.head

    def __len__(self):
        return len(self.events)


def attest_and_record(log: AttestationLog, model: VModel, x, batch: int, y, challenges: int = 2):
    """Append ``(x, y)`` only if it is a genuine inference of ``model``; returns the new head or ``None``."""
    if not verify_inference(model, x, batch, y, challenges):
        return None
    return log.record(model.commit(), x, y)

"""Additively homomorphic encryption (Paillier), for aggregating integers under encryption:
``decrypt(add_encrypted(E(a), E(b))) = a + b (mod n)`` and ``decrypt(mul_plain(E(m), k)) = k * m (mod n)``.

Random primes of the requested size come from the operating system's CSPRNG (``secrets``) and are tested with
Miller-Rabin; every encryption draws a fresh blinding factor ``r`` in Z*_n, so the same plaintext encrypts differently each
time. A caller-supplied source must be a ``secrets.SystemRandom``-like object with ``randbits``/``randbelow`` (a seeded
``random.Random`` is accepted only through ``UnsafeSeededSource``, which exists for reproducible tests). NOT production
cryptography: Python's modular exponentiation is not constant-time, ciphertexts carry no integrity check and the code
is unaudited; sizes below 2048 bits exist so that tests run quickly. ``encode_fixed`` / ``decode_fixed`` map signed
fixed-point numbers into Z_n so that gradient-like vectors can be summed under encryption (``encrypt_vector`` /
``add_vectors`` / ``decrypt_vector``).
Reference counterpart: scirust-core/src/homomorphic.rs:29-396.
"""
from __future__ import annotations

import math
import random
import secrets
from dataclasses import dataclass

_SMALL_PRIMES = [p for p in range(3, 1000, 2) if all(p % q for q in range(3, int(p ** 0.5) + 1, 2))]


class OsSource:
    def randbits(self, k: int) -> int:
        return secrets.randbits(k)

    def randbelow(self, n: int) -> int:
        return secrets.randbelow(n)


class UnsafeSeededSource:
    """Deterministic source for tests only; never for real keys or blinding factors."""

    def __init__(self, seed: int):
        self._r = random.Random(seed)

    def randbits(self, k: int) -> int:
        return self._r.getrandbits(k)

    def randbelow(self, n: int) -> int:
        return self._r.randrange(n)


@dataclass(frozen=True)
class PaillierPublicKey:
    n: int
    g: int
    nn: int


@dataclass(frozen=True)
class PaillierPrivateKey:
    lam: int
    mu: int
    n: int


def is_probable_prime(n: int, rounds: int = 40, source=None) -> bool:
    if n < 2:
        return False
    if n in (2, 3):
        return True
    if n % 2 == 0:
        return False
    for p in _SMALL_PRIMES:
        if n == p:
            return True
        if n % p == 0:
            return False
    source = source or OsSource()
    d, s = n - 1, 0
    while d % 2 == 0:
        d //= 2
        s += 1
    for _ in range(rounds):
        a = 2 + source.randbelow(n - 3)
        x = pow(a, d, n)
        if x in (1, n - 1):
            continue
        for _ in range(s - 1):
            x = x * x % n
            if x == n - 1:
                break
        else:
            return False
    return True


def random_prime(bits: int, source=None) -> int:
    if bits < 8:
        raise ValueError("primes need at least 8 bits")
    source = source or OsSource()
    while True:
        c = source.randbits(bits) | (1 << (bits - 1)) | 1             # top bit set (exact size), odd
        if is_probable_prime(c, source=source):
            return c


def generate_keypair(bit_size: int, source=None):
    """Modulus of about ``bit_size`` bits (two distinct primes of half that size); g = n + 1."""
    if bit_size < 16:
        raise ValueError("bit_size must be at least 16")
    source = source or OsSource()
    half = bit_size // 2
    while True:
        p, q = random_prime(half, source), random_prime(bit_size - half, source)
        if p == q:
            continue
        n = p * q
        if math.gcd(n, (p - 1) * (q - 1)) != 1:
            continue
        lam = math.lcm(p - 1, q - 1)
        nn = n * n
        g = n + 1
        l = (pow(g, lam, nn) - 1) // n
        try:
            mu = pow(l, -1, n)
        except ValueError:
            continue
        return PaillierPublicKey(n, g, nn), PaillierPrivateKey(lam, mu, n)


def encrypt(plain: int, pk: PaillierPublicKey, source=None) -> int:
    source = source or OsSource()
    m = plain % pk.n
    while True:
        r = source.randbelow(pk.n)
        if r and math.gcd(r, pk.n) == 1:
            break
    return pow(pk.g, m, pk.nn) * pow(r, pk.n, pk.nn) % pk.nn


def decrypt(cipher: int, sk: PaillierPrivateKey) -> int:
    nn = sk.n * sk.n
    return (pow(cipher, sk.lam, nn) - 1) // sk.n * sk.mu % sk.n


def add_encrypted(a: int, b: int, pk: PaillierPublicKey) -> int:
    return a * b % pk.nn


def mul_plain(cipher: int, k: int, pk: PaillierPublicKey) -> int:
    return pow(cipher, k % pk.n, pk.nn)


# ------------------------------------------------------------------ signed fixed-point vectors
def encode_fixed(x: float, pk: PaillierPublicKey, frac_bits: int = 24) -> int:
    """Signed fixed point in Z_n: negatives wrap to the top half of the ring."""
    if not math.isfinite(x):
        raise ValueError("only finite values can be encoded")
    v = int(round(x * (1 << frac_bits)))
    if abs(v) >= pk.n // 2:
        raise ValueError("value does not fit the modulus")
    return v % pk.n


def decode_fixed(m: int, pk_or_sk, frac_bits: int = 24) -> float:
    n = pk_or_sk.n
    v = m - n if m > n // 2 else m
    return v / (1 << frac_bits)


def encrypt_vector(xs, pk, frac_bits: int = 24, source=None) -> list:
    return [encrypt(encode_fixed(float(x), pk, frac_bits), pk, source) for x in xs]


def add_vectors(a, b, pk) -> list:
    if len(a) != len(b):
        raise ValueError("vectors differ in length")
    return [add_encrypted(x, y, pk) for x, y in zip(a, b)]


def decrypt_vector(cs, sk, frac_bits: int = 24) -> list:
    return [decode_fixed(decrypt(c, sk), sk, frac_bits) for c in cs]

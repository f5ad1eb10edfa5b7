"""KV-cache family (scirust-core/src/nn/{paged_attention,kv_backend,elastic_kv_cache,
latent_kv_cache,residual_latent_kv_cache,tiered_latent_kv_backend}.rs).

All caches implement the ``AttentionBackend`` surface - ``append(k, v)`` for one new position and
``decode_step(q)`` returning the attention output over everything cached - so they are
interchangeable and testable against ``PlainKvCache``:

* ``PlainKvCache``     contiguous fp32 rows.
* ``PagedKvCache``     fixed-size pages + block table; gathers pages in logical order, so its output
                       is bit-identical to the contiguous cache (paged_attention.rs:21-147).
* ``QuantKvCache``     per-row symmetric INT8 or INT4 codes + fp32 scale.
* ``ElasticKvCache``   two levels: the most recent ``window`` rows in fp32, older rows INT4; under a
                       byte budget the oldest quantised rows with the least accumulated attention
                       mass are evicted (elastic_kv_cache.rs).
* ``LatentKvCache``    rows stored in a rank-r latent space (fixed orthonormal projection), optional
                       INT8 residual correction (latent / residual-latent caches).
* ``TieredKvCache``    recent rows plain, middle rows latent+residual, oldest rows latent only.
The numeric ``decode_step`` is single-head; multi-head use stacks one cache per head.
"""
from __future__ import annotations

import math

import torch


def _attend(q, K, V, scale=None):
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    s = (K @ q.reshape(-1)) * scale
    p = torch.softmax(s, 0)
    return p @ V, p


class AttentionBackend:
    def append(self, k, v): raise NotImplementedError
    def keys_values(self): raise NotImplementedError
    def __len__(self): raise NotImplementedError
    def nbytes(self) -> int: raise NotImplementedError

    def decode_step(self, q, scale=None):
        K, V = self.keys_values()
        out, p = _attend(q.float(), K, V, scale)
        self._observe(p)
        return out

    def _observe(self, p):
        pass


class PlainKvCache(AttentionBackend):
    def __init__(self, dim: int):
        self.dim, self.k, self.v = dim, [], []

    def append(self, k, v):
        self.k.append(k.detach().float().reshape(-1).clone())
        self.v.append(v.detach().float().reshape(-1).clone())

    def keys_values(self):
        return torch.stack(self.k), torch.stack(self.v)

    def __len__(self): return len(self.k)
    def nbytes(self): return 2 * len(self.k) * self.dim * 4


class PagedKvCache(AttentionBackend):
    def __init__(self, dim: int, page: int = 16, n_pages: int = 64):
        self.dim, self.page = dim, page
        self.pool_k = torch.zeros(n_pages, page, dim)
        self.pool_v = torch.zeros(n_pages, page, dim)
        self.free = list(range(n_pages - 1, -1, -1))
        self.table, self.n = [], 0

    def append(self, k, v):
        if self.n % self.page == 0:
            if not self.free:
                raise MemoryError("paged KV cache: no free page")
            self.table.append(self.free.pop())
        blk, slot = self.table[-1], self.n % self.page
        self.pool_k[blk, slot] = k.detach().float().reshape(-1)
        self.pool_v[blk, slot] = v.detach().float().reshape(-1)
        self.n += 1

    def keys_values(self):
        idx = torch.tensor(self.table, dtype=torch.long)
        return self.pool_k[idx].reshape(-1, self.dim)[: self.n], self.pool_v[idx].reshape(-1, self.dim)[: self.n]

    def release(self):
        self.free.extend(reversed(self.table))
        self.table, self.n = [], 0

    def __len__(self): return self.n
    def nbytes(self): return 2 * len(self.table) * self.page * self.dim * 4


def quantize_rows(x, bits: int):
    qmax = float(2 ** (bits - 1) - 1)
    mx = x.abs().amax(-1, keepdim=True)
    scale = torch.where(mx > 0, mx / qmax, torch.ones_like(mx))
    q = torch.clamp(torch.round(x / scale), -qmax - 1, qmax).to(torch.int8)
    return q, scale


class QuantKvCache(AttentionBackend):
    def __init__(self, dim: int, bits: int = 8):
        self.dim, self.bits = dim, bits
        self.kq, self.ks, self.vq, self.vs = [], [], [], []

    def append(self, k, v):
        for x, qs, ss in ((k, self.kq, self.ks), (v, self.vq, self.vs)):
            q, s = quantize_rows(x.detach().float().reshape(1, -1), self.bits)
            qs.append(q[0]); ss.append(s[0])

    def keys_values(self):
        K = torch.stack(self.kq).float() * torch.stack(self.ks)
        V = torch.stack(self.vq).float() * torch.stack(self.vs)
        return K, V

    def __len__(self): return len(self.kq)
    def nbytes(self): return 2 * len(self.kq) * (self.dim * self.bits // 8 + 4)


class ElasticKvCache(AttentionBackend):
    def __init__(self, dim: int, window: int = 32, budget_bytes: int | None = None):
        self.dim, self.window, self.budget = dim, window, budget_bytes
        self.recent = PlainKvCache(dim)
        self.old = QuantKvCache(dim, bits=4)
        self.mass = []          # accumulated attention mass of each old row
        self.evicted = 0

    def append(self, k, v):
        self.recent.append(k, v)
        if len(self.recent) > self.window:
            k0, v0 = self.recent.k.pop(0), self.recent.v.pop(0)
            self.old.append(k0, v0)
            self.mass.append(0.0)
        while self.budget is not None and self.nbytes() > self.budget and len(self.old) > 0:
            i = min(range(len(self.mass)), key=lambda j: (self.mass[j], j))
            for lst in (self.old.kq, self.old.ks, self.old.vq, self.old.vs, self.mass):
                lst.pop(i)
            self.evicted += 1

    def keys_values(self):
        parts_k, parts_v = [], []
        if len(self.old):
            K, V = self.old.keys_values()
            parts_k.append(K); parts_v.append(V)
        if len(self.recent):
            K, V = self.recent.keys_values()
            parts_k.append(K); parts_v.append(V)
        return torch.cat(parts_k), torch.cat(parts_v)

    def _observe(self, p):
        for i in range(len(self.mass)):
            self.mass[i] += float(p[i])

    def __len__(self): return len(self.old) + len(self.recent)
    def nbytes(self): return self.old.nbytes() + self.recent.nbytes()


def _orthonormal(dim: int, rank: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    q, _ = torch.linalg.qr(torch.randn(dim, rank, generator=g))
    return q


class LatentKvCache(AttentionBackend):
    """Rows projected to rank ``r`` with a fixed orthonormal basis; ``residual_bits`` adds a
    quantised correction of what the projection lost."""

    def __init__(self, dim: int, rank: int, residual_bits: int = 0, seed: int = 0, basis=None):
        self.dim, self.rank, self.residual_bits = dim, rank, residual_bits
        self.P = basis if basis is not None else _orthonormal(dim, rank, seed)
        self.zk, self.zv, self.rk, self.rv = [], [], [], []

    def fit(self, samples: torch.Tensor):
        """Replace the random basis by the top right-singular vectors of sample rows."""
        _, _, vh = torch.linalg.svd(samples.float(), full_matrices=False)
        self.P = vh[: self.rank].t().contiguous()

    def append(self, k, v):
        for x, zs, rs in ((k, self.zk, self.rk), (v, self.zv, self.rv)):
            x = x.detach().float().reshape(-1)
            z = x @ self.P
            zs.append(z)
            if self.residual_bits:
                rs.append(quantize_rows((x - z @ self.P.t()).reshape(1, -1), self.residual_bits))

    def _decode(self, zs, rs):
        X = torch.stack(zs) @ self.P.t()
        if self.residual_bits:
            X = X + torch.cat([q.float() * s for q, s in rs])
        return X

    def keys_values(self):
        return self._decode(self.zk, self.rk), self._decode(self.zv, self.rv)

    def __len__(self): return len(self.zk)

    def nbytes(self):
        per = self.rank * 4 + ((self.dim * self.residual_bits // 8 + 4) if self.residual_bits else 0)
        return 2 * len(self.zk) * per


class TieredKvCache(AttentionBackend):
    def __init__(self, dim: int, rank: int, hot: int = 16, warm: int = 64, seed: int = 0):
        self.dim, self.hot_n, self.warm_n = dim, hot, warm
        P = _orthonormal(dim, rank, seed)
        self.hot = PlainKvCache(dim)
        self.warm = LatentKvCache(dim, rank, residual_bits=8, basis=P)
        self.cold = LatentKvCache(dim, rank, residual_bits=0, basis=P)

    def append(self, k, v):
        self.hot.append(k, v)
        if len(self.hot) > self.hot_n:
            k0, v0 = self.hot.k.pop(0), self.hot.v.pop(0)
            self.warm.append(k0, v0)
            if len(self.warm) > self.warm_n:
                K, V = self.warm.keys_values()
                self.cold.append(K[0], V[0])
                for lst in (self.warm.zk, self.warm.zv, self.warm.rk, self.warm.rv):
                    lst.pop(0)

    def keys_values(self):
        ks, vs = [], []
        for c in (self.cold, self.warm, self.hot):
            if len(c):
                K, V = c.keys_values()
                ks.append(K); vs.append(V)
        return torch.cat(ks), torch.cat(vs)

    def __len__(self): return len(self.cold) + len(self.warm) + len(self.hot)
    def nbytes(self): return self.cold.nbytes() + self.warm.nbytes() + self.hot.nbytes()

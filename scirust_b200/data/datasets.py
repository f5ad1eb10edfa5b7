"""Datasets and loaders (scirust-core/src/data/{mod,dataloader,loader,mnist,cifar10,augment}.rs;
scirust-sciagent/src/train/dataset.rs:8-368).

* ``InMemoryDataset`` + ``DataLoader``: batches over ``(features, labels)``; shuffling is a
  Fisher-Yates permutation from the PCG stream seeded with ``seed + epoch``, so epoch order is a
  pure function of ``(seed, epoch)`` and a resumed run replays it.
* MNIST IDX and CIFAR-10 binary readers; synthetic stand-ins of the same shapes (no network here).
* ``gaussian_clusters``: the seeded toy classification set used by the deterministic CPU example.
* ``TokenShardDataset``: little-endian u32 token shards (``.bin``), out-of-vocabulary ids mapped to
  ``<unk>`` = 3, fixed-length windows, hash-selected validation windows.
* ``augment``: random horizontal flip / padded crop / normalise / gaussian noise from a seeded stream.
Pinned host staging and a background prefetch thread feed the GPU trainers.
"""
from __future__ import annotations

import gzip
import queue
import struct
import threading
from pathlib import Path

import numpy as np
import torch

from ..nn.rng import PcgEngine


class InMemoryDataset:
    def __init__(self, features, labels):
        self.x = torch.as_tensor(features)
        self.y = torch.as_tensor(labels)
        if self.x.shape[0] != self.y.shape[0]:
            raise ValueError("features and labels differ in length")

    def __len__(self):
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i], self.y[i]


class DataLoader:
    def __init__(self, dataset, batch_size: int, shuffle: bool = True, seed: int = 0, drop_last: bool = False,
                 pin_memory: bool = False, prefetch: int = 0):
        self.ds, self.batch_size, self.shuffle, self.seed = dataset, batch_size, shuffle, seed
        self.drop_last, self.pin_memory, self.prefetch = drop_last, pin_memory, prefetch
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def order(self, epoch: int | None = None) -> torch.Tensor:
        n = len(self.ds)
        if not self.shuffle:
            return torch.arange(n)
        return PcgEngine(self.seed + (self.epoch if epoch is None else epoch)).shuffle(n)

    def __len__(self):
        n = len(self.ds)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def _batches(self):
        idx = self.order()
        for b in range(len(self)):
            sel = idx[b * self.batch_size:(b + 1) * self.batch_size]
            x, y = self.ds.x[sel], self.ds.y[sel]
            if self.pin_memory and torch.cuda.is_available():
                x, y = x.pin_memory(), y.pin_memory()
            yield x, y

    def __iter__(self):
        if self.prefetch <= 0:
            yield from self._batches()
        else:
            q: queue.Queue = queue.Queue(maxsize=self.prefetch)

            def work():
                for item in self._batches():
                    q.put(item)
                q.put(None)
            threading.Thread(target=work, daemon=True).start()
            while True:
                item = q.get()
                if item is None:
                    break
                yield item
        self.epoch += 1


# ----------------------------------------------------------------------------- file formats
def _open(path):
    path = str(path)
    return gzip.open(path, "rb") if path.endswith(".gz") else open(path, "rb")


def load_mnist_idx(images_path, labels_path):
    with _open(images_path) as f:
        magic, n, h, w = struct.unpack(">IIII", f.read(16))
        if magic != 2051:
            raise ValueError(f"bad IDX image magic {magic}")
        x = np.frombuffer(f.read(n * h * w), dtype=np.uint8).reshape(n, h * w).astype(np.float32) / 255.0
    with _open(labels_path) as f:
        magic, n2 = struct.unpack(">II", f.read(8))
        if magic != 2049 or n2 != n:
            raise ValueError("bad IDX label file")
        y = np.frombuffer(f.read(n), dtype=np.uint8).astype(np.int64)
    return InMemoryDataset(torch.from_numpy(x), torch.from_numpy(y))


def load_cifar10_bin(paths):
    xs, ys = [], []
    for p in paths:
        raw = np.frombuffer(Path(p).read_bytes(), dtype=np.uint8)
        if raw.size % 3073:
            raise ValueError(f"{p}: not a CIFAR-10 binary batch")
        rec = raw.reshape(-1, 3073)
        ys.append(rec[:, 0].astype(np.int64))
        xs.append(rec[:, 1:].astype(np.float32) / 255.0)
    return InMemoryDataset(torch.from_numpy(np.concatenate(xs)), torch.from_numpy(np.concatenate(ys)))


def synthetic_mnist(n: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return InMemoryDataset(torch.rand(n, 784, generator=g), torch.randint(0, 10, (n,), generator=g))


def synthetic_cifar10(n: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return InMemoryDataset(torch.randn(n, 3 * 32 * 32, generator=g), torch.randint(0, 10, (n,), generator=g))


def gaussian_clusters(n: int = 150, classes: int = 3, dim: int = 4, sigma: float = 0.5, seed: int = 42):
    """``classes`` isotropic Gaussian clusters: centers ~ U[-2, 2]^dim, points = center + sigma*N(0,1),
    all drawn in order from one PCG stream (centers first, then the samples class by class)."""
    rng = PcgEngine(seed)
    centers = rng.fill_uniform_signed((classes, dim), 2.0)
    per = n // classes
    xs, ys = [], []
    for c in range(classes):
        cnt = per if c < classes - 1 else n - per * (classes - 1)
        xs.append(centers[c][None, :] + rng.fill_normal((cnt, dim), 0.0, sigma))
        ys.append(torch.full((cnt,), c, dtype=torch.int64))
    return InMemoryDataset(torch.cat(xs), torch.cat(ys))


# ----------------------------------------------------------------------------- token shards
def write_token_shard(path, tokens) -> None:
    np.asarray(tokens, dtype="<u4").tofile(str(path))


def _hash64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return x ^ (x >> 31)


class TokenShardDataset:
    """Windows of ``seq_len + 1`` tokens over concatenated ``.bin`` shards. A window belongs to the
    validation split when ``hash(window index) % 10000 < val_frac * 10000`` (split_version 1), so the
    split is stable under resharding and resume. ``batch(step)`` is a pure function of
    ``(seed, step)``: epoch = step*batch // n_train, order = PCG shuffle seeded by seed + epoch."""

    def __init__(self, paths, seq_len: int, vocab_size: int, val_frac: float = 0.0, seed: int = 0, shuffle: bool = True):
        arrs = [np.fromfile(str(p), dtype="<u4") for p in paths]
        tok = np.concatenate(arrs) if arrs else np.zeros(0, dtype=np.uint32)
        tok = np.where(tok >= vocab_size, 3, tok).astype(np.int64)
        self.tokens = torch.from_numpy(tok)
        self.seq_len, self.seed, self.shuffle = seq_len, seed, shuffle
        n_win = max(0, (len(tok) - 1) // seq_len)
        thresh = int(val_frac * 10000)
        is_val = np.array([_hash64(i) % 10000 < thresh for i in range(n_win)], dtype=bool) if n_win else np.zeros(0, bool)
        self.train_windows = np.nonzero(~is_val)[0]
        self.val_windows = np.nonzero(is_val)[0]
        self._order_epoch, self._order = None, None

    def corpus_tokens(self) -> int:
        return int(self.tokens.numel())

    def corpus_hash(self) -> int:
        h = 0xCBF29CE484222325
        for b in self.tokens[: 1 << 16].numpy().astype("<u4").tobytes():
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        return h

    def window(self, w: int) -> torch.Tensor:
        s = int(w) * self.seq_len
        return self.tokens[s:s + self.seq_len + 1]

    def _epoch_order(self, epoch: int):
        if self._order_epoch != epoch:
            n = len(self.train_windows)
            perm = PcgEngine(self.seed + epoch).shuffle(n).numpy() if self.shuffle else np.arange(n)
            self._order, self._order_epoch = self.train_windows[perm], epoch
        return self._order

    def batch(self, step: int, batch_size: int) -> torch.Tensor:
        n = len(self.train_windows)
        if n == 0:
            raise ValueError("no training windows")
        rows = []
        for j in range(batch_size):
            g = step * batch_size + j
            rows.append(self.window(self._epoch_order(g // n)[g % n]))
        return torch.stack(rows)

    def val_batches(self, batch_size: int):
        for i in range(0, len(self.val_windows), batch_size):
            yield torch.stack([self.window(w) for w in self.val_windows[i:i + batch_size]])


def augment(x: torch.Tensor, c: int, h: int, w: int, seed: int, flip: bool = True, crop_pad: int = 0,
            mean=None, std=None, noise: float = 0.0) -> torch.Tensor:
    """Seeded augmentation of flattened NCHW images."""
    g = torch.Generator().manual_seed(seed)
    B = x.shape[0]
    img = x.reshape(B, c, h, w).clone()
    if flip:
        m = torch.rand(B, generator=g) < 0.5
        img[m] = img[m].flip(-1)
    if crop_pad > 0:
        padded = torch.nn.functional.pad(img, (crop_pad,) * 4)
        oy = torch.randint(0, 2 * crop_pad + 1, (B,), generator=g)
        ox = torch.randint(0, 2 * crop_pad + 1, (B,), generator=g)
        img = torch.stack([padded[i, :, oy[i]:oy[i] + h, ox[i]:ox[i] + w] for i in range(B)])
    if mean is not None:
        img = (img - torch.tensor(mean).view(1, c, 1, 1)) / torch.tensor(std).view(1, c, 1, 1)
    if noise > 0:
        img = img + noise * torch.randn(img.shape, generator=g)
    return img.reshape(B, -1)

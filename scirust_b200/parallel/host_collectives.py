"""Host-side collectives with fixed reduction order (the reference's only "distributed" layer:
scirust-core/src/distributed.rs:29-231, tree_allreduce.rs:33-366, autodiff/data_parallel.rs:91-192).

* ``WorkerGroup`` / ``DistributedContext``: threads as ranks sharing a barrier and a keyed slot table.
  ``all_reduce`` publishes, waits, then every rank adds the slots in ascending rank order and
  multiplies once by 1/world; a key or length mismatch raises on every rank. ``broadcast`` and
  ``barrier`` complete the surface.
* ``tree_all_reduce``: fixed binary tree (children of r are 2r+1, 2r+2). A rank always combines
  *self, left, right* in that order, whatever order the messages arrive in (early ones are parked),
  so timing never changes the bits. ``FixedOrderSum`` adds fp32 in tree order (bits depend on the
  world size); ``ExactSum`` carries exact long accumulators (topology-independent, correctly rounded).
  Engines: in-process threads with optional adversarial jitter, and a TCP transport on 127.0.0.1
  or real hosts (frame = ``u32 rank | u64 len | payload`` little-endian, 1 GiB cap, a frame from an
  unexpected rank is an error). The transport is unauthenticated: use it inside a trusted network.
* ``DataParallelTrainer``: splits a batch over workers, computes per-worker gradients (optionally on
  threads) and reduces them in worker-index order, so the update is bit-identical for any thread
  count.
These run on CPU ranks; the GPU counterparts with the same order contract are
``parallel/fused_allreduce.py`` and ``parallel/tensor_parallel.py``.
"""
from __future__ import annotations

import random
import socket
import struct
import threading
import time

import numpy as np

from ..numerics.reproducible import ExactAccumulator

MAX_FRAME = 1 << 30


class CollectiveError(RuntimeError):
    pass


# ----------------------------------------------------------------------------- thread ranks
class WorkerGroup:
    def __init__(self, world: int):
        if world < 1:
            raise ValueError("world size must be positive")
        self.world = world
        self.barrier = threading.Barrier(world)
        self.lock = threading.Lock()
        self.slots: dict = {}
        self.errors: dict = {}

    def context(self, rank: int) -> "DistributedContext":
        return DistributedContext(self, rank)


class DistributedContext:
    def __init__(self, group: WorkerGroup, rank: int):
        if not 0 <= rank < group.world:
            raise ValueError("rank out of range")
        self.group, self.rank, self.world = group, rank, group.world

    @staticmethod
    def single() -> "DistributedContext":
        return DistributedContext(WorkerGroup(1), 0)

    def barrier(self) -> None:
        self.group.barrier.wait()

    def all_reduce(self, key: str, values) -> np.ndarray:
        g = self.group
        v = np.asarray(values, dtype=np.float32).copy()
        with g.lock:
            g.slots.setdefault(key, [None] * g.world)[self.rank] = v
        g.barrier.wait()
        slots = g.slots.get(key)
        err = None
        if slots is None or any(s is None for s in slots):
            err = f"all_reduce: key {key!r} was not published by every rank"
        elif any(s.shape != slots[0].shape for s in slots):
            err = f"all_reduce: length mismatch for key {key!r}"
        out = None
        if err is None:
            acc = np.zeros_like(slots[0])
            for r in range(g.world):                 # ascending rank order on every rank
                acc = (acc + slots[r]).astype(np.float32)
            out = (acc * np.float32(1.0 / g.world)).astype(np.float32)
        g.barrier.wait()
        if self.rank == 0:
            with g.lock:
                g.slots.pop(key, None)
        g.barrier.wait()
        if err is not None:
            raise CollectiveError(err)
        return out

    def all_reduce_dict(self, grads: dict) -> dict:
        keys = sorted(grads)
        mine = "\x00".join(keys)
        sig = self.gather_obj("__keys__", mine)
        if any(s != mine for s in sig):
            raise CollectiveError("all_reduce: ranks disagree on the set of keys")
        return {k: self.all_reduce(k, grads[k]) for k in keys}

    def gather_obj(self, key: str, obj) -> list:
        g = self.group
        with g.lock:
            g.slots.setdefault(key, [None] * g.world)[self.rank] = obj
        g.barrier.wait()
        out = list(g.slots[key])
        g.barrier.wait()
        if self.rank == 0:
            with g.lock:
                g.slots.pop(key, None)
        g.barrier.wait()
        return out

    def broadcast(self, key: str, values=None) -> np.ndarray:
        g = self.group
        if self.rank == 0:
            with g.lock:
                g.slots[key] = np.asarray(values, dtype=np.float32).copy()
        g.barrier.wait()
        out = g.slots[key].copy()
        g.barrier.wait()
        if self.rank == 0:
            with g.lock:
                g.slots.pop(key, None)
        g.barrier.wait()
        return out
    broadcast_f32 = broadcast


def run_ranks(world: int, fn):
    """Run ``fn(ctx)`` on ``world`` threads; returns results by rank; re-raises the first error."""
    group = WorkerGroup(world)
    out, errs = [None] * world, [None] * world

    def work(r):
        try:
            out[r] = fn(group.context(r))
        except BaseException as e:  # noqa: BLE001
            errs[r] = e
            try:
                group.barrier.abort()
            except Exception:  # noqa: BLE001
                pass
    ts = [threading.Thread(target=work, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    real = [e for e in errs if e is not None and not isinstance(e, threading.BrokenBarrierError)]
    if real:
        raise real[0]
    if any(errs):
        raise next(e for e in errs if e is not None)
    return out


# ----------------------------------------------------------------------------- combiners
class FixedOrderSum:
    """fp32 element-wise sum; the value of a subtree is ((self + left) + right)."""
    @staticmethod
    def lift(x):
        return np.asarray(x, dtype=np.float32).copy()

    @staticmethod
    def combine(a, b):
        return (a + b).astype(np.float32)

    @staticmethod
    def finish(a):
        return a

    @staticmethod
    def to_bytes(a):
        return np.asarray(a, dtype="<f4").tobytes()

    @staticmethod
    def from_bytes(b):
        return np.frombuffer(b, dtype="<f4").copy()


class ExactSum:
    """Exact long accumulators per element: the result is the correctly rounded true sum and does not
    depend on the tree shape or the world size."""
    @staticmethod
    def lift(x):
        accs = []
        for v in np.asarray(x, dtype=np.float32).tolist():
            a = ExactAccumulator()
            a.add(v)
            accs.append(a)
        return accs

    @staticmethod
    def combine(a, b):
        if len(a) != len(b):
            raise CollectiveError("ExactSum: length mismatch")
        for x, y in zip(a, b):
            x.merge(y)
        return a

    @staticmethod
    def finish(a):
        return np.array([x.round_f32() for x in a], dtype=np.float32)

    @staticmethod
    def to_bytes(a):
        parts = [struct.pack("<I", len(a))]
        for x in a:
            b = x.to_bytes()
            parts.append(struct.pack("<I", len(b)) + b)
        return b"".join(parts)

    @staticmethod
    def from_bytes(b):
        (n,) = struct.unpack_from("<I", b, 0)
        p, out = 4, []
        for _ in range(n):
            (ln,) = struct.unpack_from("<I", b, p)
            out.append(ExactAccumulator.from_bytes(b[p + 4:p + 4 + ln]))
            p += 4 + ln
        return out


def _children(r, world):
    return [c for c in (2 * r + 1, 2 * r + 2) if c < world]


# ----------------------------------------------------------------------------- in-process tree engine
def tree_all_reduce(inputs, combine=FixedOrderSum, jitter_seed=None):
    """All-reduce ``inputs[rank]`` over a fixed binary tree with one thread per rank. ``jitter_seed``
    injects random delays before every send to scramble arrival order."""
    world = len(inputs)
    boxes = [dict() for _ in range(world)]
    conds = [threading.Condition() for _ in range(world)]
    results = [None] * world
    rnd = random.Random(jitter_seed) if jitter_seed is not None else None
    delays = [[rnd.random() * 0.003 for _ in range(4)] for _ in range(world)] if rnd else None

    def send(dst, tag, payload, src):
        if delays:
            time.sleep(delays[src][hash(tag) % 4])
        with conds[dst]:
            boxes[dst][tag] = payload
            conds[dst].notify_all()

    def recv(me, tag):
        with conds[me]:
            while tag not in boxes[me]:       # messages for later steps stay parked in the box
                if not conds[me].wait(timeout=30):
                    raise CollectiveError(f"rank {me}: timed out waiting for {tag}")
            return boxes[me].pop(tag)

    def work(r):
        acc = combine.lift(inputs[r])
        for c in _children(r, world):          # always left then right
            acc = combine.combine(acc, recv(r, ("up", c)))
        if r != 0:
            send((r - 1) // 2, ("up", r), acc, r)
            total = recv(r, ("down", r))
        else:
            total = combine.finish(acc)
        for c in _children(r, world):
            send(c, ("down", c), total, r)
        results[r] = total

    errs = []

    def guarded(r):
        try:
            work(r)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=guarded, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    if errs:
        raise errs[0]
    return results


# ----------------------------------------------------------------------------- TCP transport
def _recv_exact(sock, n):
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(1 << 20, n - len(buf)))
        if not chunk:
            raise CollectiveError("connection closed mid-frame")
        buf += chunk
    return bytes(buf)


def send_frame(sock, rank: int, payload: bytes) -> None:
    if len(payload) > MAX_FRAME:
        raise CollectiveError("frame larger than 1 GiB")
    sock.sendall(struct.pack("<IQ", rank, len(payload)) + payload)


def recv_frame(sock, expected_ranks):
    rank, ln = struct.unpack("<IQ", _recv_exact(sock, 12))
    if ln > MAX_FRAME:
        raise CollectiveError(f"frame of {ln} bytes exceeds the 1 GiB cap")
    if rank not in expected_ranks:
        raise CollectiveError(f"frame from unexpected rank {rank}")
    return rank, _recv_exact(sock, ln)


def tcp_tree_all_reduce_rank(rank: int, world: int, addrs, values, combine=FixedOrderSum, timeout: float = 30.0):
    """One rank of the TCP tree all-reduce. ``addrs[r] = (host, port)`` is rank r's listener. Every
    rank listens for its children, connects to its parent, and returns the reduced vector."""
    kids = _children(rank, world)
    srv = None
    if kids:
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind(addrs[rank])
        srv.listen(len(kids))
        srv.settimeout(timeout)
    try:
        acc = combine.lift(values)
        conns = {}
        for _ in kids:
            c, _a = srv.accept()
            c.settimeout(timeout)
            r, payload = recv_frame(c, set(kids) - set(conns))
            conns[r] = (c, combine.from_bytes(payload))
        for k in kids:                          # combine in fixed order, not arrival order
            acc = combine.combine(acc, conns[k][1])
        if rank != 0:
            parent = (rank - 1) // 2
            deadline = time.time() + timeout
            while True:
                try:
                    up = socket.create_connection(addrs[parent], timeout=timeout)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise CollectiveError(f"rank {rank}: cannot reach parent {parent}") from None
                    time.sleep(0.02)
            up.settimeout(timeout)
            send_frame(up, rank, combine.to_bytes(acc))
            _r, payload = recv_frame(up, {parent})
            total = np.frombuffer(payload, dtype="<f4").copy()
            up.close()
        else:
            total = combine.finish(acc)
        out = np.asarray(total, dtype="<f4").tobytes()
        for k in kids:
            send_frame(conns[k][0], rank, out)
            conns[k][0].close()
        return np.asarray(total, dtype=np.float32)
    finally:
        if srv is not None:
            srv.close()


def tcp_tree_all_reduce_native(rank: int, world: int, addrs, values, timeout: float = 30.0) -> np.ndarray:
    """Same all-reduce (fp32 fixed-order sum) through the native transport (csrc/rt_collectives.cpp):
    sockets, framing and the child-ordered sum run in C++ without the interpreter lock, so ranks living
    in threads of one process overlap. Bitwise identical to ``tcp_tree_all_reduce_rank`` with
    ``FixedOrderSum``; addresses must be IPv4 literals."""
    import ctypes as C
    from ..ops import _lib
    lib = _lib.rt()
    fn = lib.sbrt_tcp_tree_allreduce_f32
    fn.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.c_void_p, C.c_int64, C.c_int]
    fn.restype = C.c_int
    buf = np.ascontiguousarray(values, dtype=np.float32).copy()
    hosts = (C.c_char_p * world)(*[a[0].encode() for a in addrs])
    ports = (C.c_int * world)(*[int(a[1]) for a in addrs])
    rc = fn(rank, world, hosts, ports, buf.ctypes.data, buf.size, int(timeout * 1000))
    if rc != 0:
        what = {1: "bad argument", 2: "socket error", 3: "timed out", 4: "protocol error / unexpected rank",
                5: "out of memory", 6: "peer closed the connection"}.get(rc, str(rc))
        raise CollectiveError(f"rank {rank}: native tree all-reduce failed: {what}")
    return buf


# ----------------------------------------------------------------------------- data-parallel trainer
class DataParallelTrainer:
    """``grad_fn(params, x, y) -> (loss, grads)`` is evaluated on ``workers`` contiguous slices of the
    batch; gradients are summed in worker-index order and divided by the worker count, then
    ``update_fn(params, grads)`` applies them. ``train_batch_threaded`` computes the slices on
    threads; the reduction order, hence every bit of the update, is the same."""

    def __init__(self, workers: int, grad_fn, update_fn):
        self.workers, self.grad_fn, self.update_fn = workers, grad_fn, update_fn

    def _slices(self, n):
        per = (n + self.workers - 1) // self.workers
        return [(i * per, min(n, (i + 1) * per)) for i in range(self.workers) if i * per < n]

    def _reduce(self, results):
        k = len(results)
        loss = np.float32(0)
        grads = None
        for l, g in results:                    # worker-index order
            loss = np.float32(loss + np.float32(l))
            grads = [x.astype(np.float32).copy() for x in g] if grads is None else \
                [(a + b).astype(np.float32) for a, b in zip(grads, g)]
        inv = np.float32(1.0 / k)
        return float(loss * inv), [(g * inv).astype(np.float32) for g in grads]

    def train_batch(self, params, x, y):
        res = [self.grad_fn(params, x[a:b], y[a:b]) for a, b in self._slices(len(x))]
        loss, grads = self._reduce(res)
        self.update_fn(params, grads)
        return loss

    def train_batch_threaded(self, params, x, y):
        sl = self._slices(len(x))
        res = [None] * len(sl)

        def work(i, a, b):
            res[i] = self.grad_fn(params, x[a:b], y[a:b])
        ts = [threading.Thread(target=work, args=(i, a, b)) for i, (a, b) in enumerate(sl)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        loss, grads = self._reduce(res)
        self.update_fn(params, grads)
        return loss

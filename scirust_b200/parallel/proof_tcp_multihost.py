"""Self-verifying proof of the fixed-tree all-reduce over real TCP between separate processes (or machines).

One process per rank:

    python -m scirust_b200.parallel.proof_tcp_multihost --rank R --n N --seed SEED [--dim D]
        [--combine fixed|exact] [--my-addr HOST:PORT] [--parent-addr HOST:PORT] [--native 1]

``--my-addr`` is required exactly when the rank has children (2R + 1 < N): the address its listener binds.
``--parent-addr`` is required for every rank but 0: the reachable address of rank (R - 1) // 2. Every rank derives its
contribution locally from Philox(seed, stream = rank), so no data has to be shipped beforehand; after the all-reduce
rank 0 regenerates all N contributions, runs the in-process tree engine on them and compares bit for bit. It prints
``verdict=PASS`` (exit 0) or ``verdict=FAIL`` (exit 1). Ranks on different architectures that print PASS show the
reduction to be bit-exact across them and across a real network.

Counterpart of scirust-core/src/bin/proof_tcp_multihost.rs:1-272.
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np

from ..nn.rng import Philox4x32
from .host_collectives import (CollectiveError, ExactSum, FixedOrderSum, tcp_tree_all_reduce_native,
                               tcp_tree_all_reduce_rank, tree_all_reduce)


def rank_input(seed: int, rank: int, dim: int) -> np.ndarray:
    """Rank ``rank``'s contribution: a pure function of (seed, rank, dim), identical on every machine."""
    return Philox4x32(seed).fill_f32(rank, 0, dim)


def _addr(text: str):
    host, _, port = text.rpartition(":")
    return host, int(port)


def run(rank: int, n: int, seed: int, dim: int, combine_name: str, my_addr, parent_addr, native: bool = False,
        timeout: float = 30.0) -> int:
    combine = {"fixed": FixedOrderSum, "exact": ExactSum}[combine_name]
    has_children = 2 * rank + 1 < n
    if has_children and my_addr is None:
        print(f"rank {rank} has children: --my-addr is required", file=sys.stderr)
        return 2
    if rank > 0 and parent_addr is None:
        print(f"rank {rank} is not the root: --parent-addr is required", file=sys.stderr)
        return 2
    addrs = [None] * n
    if my_addr is not None:
        addrs[rank] = my_addr
    if rank > 0:
        addrs[(rank - 1) // 2] = parent_addr
    x = rank_input(seed, rank, dim)
    t0 = time.time()
    try:
        if native and combine is FixedOrderSum:
            filled = [a if a is not None else ("127.0.0.1", 1) for a in addrs]
            got = tcp_tree_all_reduce_native(rank, n, filled, x, timeout=timeout)
        else:
            got = tcp_tree_all_reduce_rank(rank, n, addrs, x, combine=combine, timeout=timeout)
    except (CollectiveError, OSError) as e:
        print(f"rank {rank}: all-reduce failed: {e}", file=sys.stderr)
        return 1
    dt = time.time() - t0
    if rank != 0:
        print(f"rank={rank} n={n} dim={dim} combine={combine_name} done in {dt:.3f}s "
              f"fingerprint={_fingerprint(got):016x}")
        return 0
    ref = tree_all_reduce([rank_input(seed, r, dim) for r in range(n)], combine=combine)[0]
    ok = np.array_equal(np.asarray(got, dtype=np.float32).view(np.uint32),
                        np.asarray(ref, dtype=np.float32).view(np.uint32))
    print(f"rank=0 n={n} dim={dim} seed={seed} combine={combine_name} time={dt:.3f}s "
          f"fingerprint={_fingerprint(got):016x} reference={_fingerprint(ref):016x} verdict={'PASS' if ok else 'FAIL'}")
    return 0 if ok else 1


def _fingerprint(v) -> int:
    h = 0xCBF29CE484222325
    for b in np.asarray(v, dtype="<f4").tobytes():
        h = ((h ^ b) * 0x100000001B3) & ((1 << 64) - 1)
    return h


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dim", type=int, default=100_352)
    ap.add_argument("--combine", default="fixed", choices=["fixed", "exact"])
    ap.add_argument("--my-addr", default=None)
    ap.add_argument("--parent-addr", default=None)
    ap.add_argument("--native", type=int, default=0, help="1: C++ transport (fixed-order sum only)")
    ap.add_argument("--timeout", type=float, default=30.0)
    a = ap.parse_args(argv)
    if not (0 <= a.rank < a.n):
        print("--rank must be in [0, n)", file=sys.stderr)
        return 2
    return run(a.rank, a.n, a.seed, a.dim, a.combine, _addr(a.my_addr) if a.my_addr else None,
               _addr(a.parent_addr) if a.parent_addr else None, bool(a.native), a.timeout)


if __name__ == "__main__":
    sys.exit(main())

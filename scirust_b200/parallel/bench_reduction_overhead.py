"""What does a deterministic reduction cost? Pinned-order against arrival-order gradient reduction on threads.

    python -m scirust_b200.parallel.bench_reduction_overhead [--dim 100352] [--threads 1,2,4,8] [--iters 50]

N worker threads each hold a gradient of ``dim`` floats. *Pinned*: the results are added in worker order 0..N-1 after
all have arrived (the data-parallel trainer's rule: bit-identical for any scheduling). *Arrival*: each worker adds its
gradient into the shared accumulator under a lock as soon as it is done, in whatever order the scheduler produces
(the non-deterministic baseline). Both do the same N vector additions; the table shows the median time of each and
how many distinct results (bit patterns) arrival order produced over the iterations.

Counterpart of scirust-core/src/bin/bench_reduction_overhead.rs:1-204 (results: docs/evidence/o1-bench).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import threading
import time

import numpy as np


def _inputs(n: int, dim: int, seed: int):
    rng = np.random.default_rng(seed)
    # wide dynamic range, so that the order of fp32 additions shows in the low bits
    return [(rng.standard_normal(dim) * 10.0 ** rng.integers(-3, 4, dim)).astype(np.float32) for _ in range(n)]


def reduce_pinned(grads) -> np.ndarray:
    results = [None] * len(grads)

    def work(i):
        results[i] = grads[i] * np.float32(1.0)        # stands for "worker i computed its gradient"
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(grads))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    acc = np.zeros_like(grads[0])
    for r in results:                                  # worker order, whatever the arrival order was
        acc += r
    return acc


def reduce_arrival(grads) -> np.ndarray:
    acc = np.zeros_like(grads[0])
    lock = threading.Lock()

    def work(i):
        g = grads[i] * np.float32(1.0)
        with lock:
            acc.__iadd__(g)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(grads))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return acc


def bench(dim: int, threads, iters: int, seed: int = 0):
    rows = []
    for n in threads:
        grads = _inputs(n, dim, seed)
        tp, ta, pats_p, pats_a = [], [], set(), set()
        for _ in range(iters):
            t0 = time.perf_counter()
            a = reduce_pinned(grads)
            tp.append(time.perf_counter() - t0)
            pats_p.add(a.tobytes())
            t0 = time.perf_counter()
            b = reduce_arrival(grads)
            ta.append(time.perf_counter() - t0)
            pats_a.add(b.tobytes())
        rows.append({"threads": n, "dim": dim, "pinned_us": statistics.median(tp) * 1e6,
                     "arrival_us": statistics.median(ta) * 1e6, "pinned_distinct_results": len(pats_p),
                     "arrival_distinct_results": len(pats_a)})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--dim", type=int, default=100_352)
    ap.add_argument("--threads", default="1,2,4,8")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    rows = bench(a.dim, [int(t) for t in a.threads.split(",")], a.iters)
    if a.json:
        print(json.dumps(rows))
        return 0
    print(f"{'threads':>7} {'pinned us':>10} {'arrival us':>11} {'overhead':>9} {'distinct (pinned / arrival)':>28}")
    for r in rows:
        print(f"{r['threads']:>7} {r['pinned_us']:>10.0f} {r['arrival_us']:>11.0f} "
              f"{r['pinned_us'] / r['arrival_us']:>8.2f}x {r['pinned_distinct_results']:>12} / "
              f"{r['arrival_distinct_results']}")
    return 0 if all(r["pinned_distinct_results"] == 1 for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())

"""Elastic BPE tokenizer: one semantic (canonical rank-priority BPE), several execution kernels, a router that picks
the kernel by piece length, and an auto-tuner that fits the routing profile to the host.

Semantics (``CanonicalBpeOracle``): a merge rule's rank is its position in the ordered merge table; on every
iteration the adjacent pair with the globally lowest rank is merged, the left-most occurrence on ties, until no pair
has a rule. A piece is never chunked: routing changes HOW a piece is encoded, never WHICH ids come out, so two hosts
with different profiles produce identical tokens. A table that names the same pair twice is refused
(``DuplicateMergeRule``).

Kernels, all parity-gated against the oracle:

* ``reference``  the O(n^2) oracle itself;
* ``tiny_scan``  the same scan on a fixed small array without allocation per step, for pieces of a few bytes;
* ``indexed``    ranks of all adjacent pairs kept in an array beside a doubly linked list; one O(n) arg-min per merge
                 and O(1) local repair, no hashing in the loop;
* ``heap``       a binary heap of (rank, position, generation) over the linked list with lazy invalidation:
                 O(n log n), for long pieces.

``ElasticThresholds`` split piece lengths into six classes (S, M, L, XL, XXL, XXXL); an ``ElasticProfile`` maps each
class to a kernel; ``autotune`` times every kernel on representative pieces of every class, discards any kernel whose
output differs from the oracle, and returns the fastest per class.

Counterparts: scirust-sciagent/src/elastic_tokenizer.rs:16-260 (classes, profile, oracle), elastic_tiny.rs,
elastic_indexed.rs, elastic_heap.rs (kernels), elastic_autotune.rs / elastic_profile_fit.rs (calibration).
"""
from __future__ import annotations

import heapq
import time
from dataclasses import dataclass

CLASSES = ("S", "M", "L", "XL", "XXL", "XXXL")
KERNELS = ("reference", "tiny_scan", "indexed", "heap")


class DuplicateMergeRule(ValueError):
    def __init__(self, left, right):
        super().__init__(f"duplicate BPE merge rule for pair ({left}, {right})")
        self.left, self.right = left, right


@dataclass(frozen=True)
class ElasticThresholds:
    s_max: int = 16
    m_max: int = 64
    l_max: int = 256
    xl_max: int = 1024
    xxl_max: int = 4096

    def __post_init__(self):
        if not (self.s_max < self.m_max < self.l_max < self.xl_max < self.xxl_max):
            raise ValueError("elastic tokenizer thresholds must be strictly increasing")

    def classify(self, piece_len: int) -> str:
        for name, lim in zip(CLASSES, (self.s_max, self.m_max, self.l_max, self.xl_max, self.xxl_max)):
            if piece_len <= lim:
                return name
        return "XXXL"


@dataclass(frozen=True)
class ElasticProfile:
    thresholds: ElasticThresholds
    kernels: tuple            # one kernel name per class

    def __post_init__(self):
        if len(self.kernels) != 6 or any(k not in KERNELS for k in self.kernels):
            raise ValueError("a profile names one known kernel for each of the six classes")

    @staticmethod
    def reference_only(thresholds: ElasticThresholds | None = None) -> "ElasticProfile":
        return ElasticProfile(thresholds or ElasticThresholds(), ("reference",) * 6)

    def kernel_for(self, piece_len: int) -> str:
        return self.kernels[CLASSES.index(self.thresholds.classify(piece_len))]


class CanonicalBpeOracle:
    def __init__(self, ordered_merges):
        self.rules: dict = {}
        for rank, (l, r, out) in enumerate(ordered_merges):
            if (l, r) in self.rules:
                raise DuplicateMergeRule(l, r)
            self.rules[(l, r)] = (rank, out)

    def __len__(self):
        return len(self.rules)

    # ---- reference: the auditable statement
    def encode_ids(self, ids) -> list:
        ids = list(ids)
        rules = self.rules
        while len(ids) >= 2:
            best = None
            for pos in range(len(ids) - 1):
                rule = rules.get((ids[pos], ids[pos + 1]))
                if rule is not None and (best is None or (rule[0], pos) < (best[0], best[1])):
                    best = (rule[0], pos, rule[1])
            if best is None:
                break
            ids[best[1]] = best[2]
            del ids[best[1] + 1]
        return ids

    # ---- tiny scan: in place on one list, ranks looked up once per surviving pair per step
    def encode_tiny(self, ids) -> list:
        ids = list(ids)
        n = len(ids)
        get = self.rules.get
        none = (1 << 62, 0)
        while n >= 2:
            best_rank, best_pos, best_out = 1 << 62, -1, 0
            for pos in range(n - 1):
                rank, out = get((ids[pos], ids[pos + 1]), none)
                if rank < best_rank:
                    best_rank, best_pos, best_out = rank, pos, out
            if best_pos < 0:
                break
            ids[best_pos] = best_out
            ids[best_pos + 1:n - 1] = ids[best_pos + 2:n]
            n -= 1
        return ids[:n]

    # ---- indexed: pair ranks beside a linked list, repaired locally after each merge
    def encode_indexed(self, ids) -> list:
        n = len(ids)
        if n < 2:
            return list(ids)
        tok = list(ids)
        nxt = list(range(1, n + 1))
        prv = list(range(-1, n - 1))
        get = self.rules.get
        big = 1 << 62
        rank = [big] * n            # rank[i]: rule of (tok[i], tok[next(i)]), big when none or i is dead / last
        out = [0] * n
        for i in range(n - 1):
            r = get((tok[i], tok[i + 1]))
            if r is not None:
                rank[i], out[i] = r
        while True:
            best = min(rank)
            if best == big:
                break
            i = rank.index(best)      # left-most position of the lowest rank (positions keep their order)
            j = nxt[i]
            tok[i] = out[i]
            k = nxt[j]
            nxt[i] = k
            if k < n:
                prv[k] = i
            rank[j] = big
            r = get((tok[i], tok[k])) if k < n else None
            rank[i], out[i] = r if r is not None else (big, 0)
            p = prv[i]
            if p >= 0:
                r = get((tok[p], tok[i]))
                rank[p], out[p] = r if r is not None else (big, 0)
        res, i = [], 0
        while i < n:
            res.append(tok[i])
            i = nxt[i]
        return res

    # ---- heap: (rank, position) candidates with lazy invalidation
    def encode_heap(self, ids) -> list:
        n = len(ids)
        if n < 2:
            return list(ids)
        tok = list(ids)
        nxt = list(range(1, n + 1))
        prv = list(range(-1, n - 1))
        alive = [True] * n
        gen = [0] * n               # bumped whenever the pair starting at i changes: stale heap entries are skipped
        get = self.rules.get
        heap = []
        for i in range(n - 1):
            r = get((tok[i], tok[i + 1]))
            if r is not None:
                heap.append((r[0], i, 0, r[1]))
        heapq.heapify(heap)
        while heap:
            _, i, g, out = heapq.heappop(heap)
            if not alive[i] or g != gen[i]:
                continue
            j = nxt[i]
            tok[i] = out
            alive[j] = False
            k = nxt[j]
            nxt[i] = k
            if k < n:
                prv[k] = i
            gen[i] += 1
            if k < n:
                r = get((tok[i], tok[k]))
                if r is not None:
                    heapq.heappush(heap, (r[0], i, gen[i], r[1]))
            p = prv[i]
            if p >= 0:
                gen[p] += 1
                r = get((tok[p], tok[i]))
                if r is not None:
                    heapq.heappush(heap, (r[0], p, gen[p], r[1]))
        res, i = [], 0
        while i < n:
            res.append(tok[i])
            i = nxt[i]
        return res

    def kernel(self, name: str):
        return {"reference": self.encode_ids, "tiny_scan": self.encode_tiny, "indexed": self.encode_indexed,
                "heap": self.encode_heap}[name]


class ElasticTokenizer:
    """Routes every complete piece to the kernel its length class is mapped to."""

    def __init__(self, ordered_merges, profile: ElasticProfile | None = None):
        self.oracle = CanonicalBpeOracle(ordered_merges)
        self.profile = profile or ElasticProfile(ElasticThresholds(), ("tiny_scan", "indexed", "indexed", "heap", "heap", "heap"))
        self.routed = {k: 0 for k in KERNELS}

    def encode_piece(self, ids, piece_len: int | None = None) -> list:
        name = self.profile.kernel_for(len(ids) if piece_len is None else piece_len)
        self.routed[name] += 1
        return self.oracle.kernel(name)(ids)

    def encode_bytes(self, data: bytes, byte_ids=None) -> list:
        ids = list(data) if byte_ids is None else [byte_ids[b] for b in data]
        return self.encode_piece(ids, len(data))


@dataclass
class CalibrationReport:
    profile: ElasticProfile
    ns_per_piece: dict          # class -> {kernel: median nanoseconds}
    rejected: dict              # class -> [kernels whose output differed from the oracle]


def autotune(oracle: CanonicalBpeOracle, cases: dict, thresholds: ElasticThresholds | None = None, repeats: int = 5,
             clock=time.perf_counter_ns) -> CalibrationReport:
    """``cases``: class name -> list of complete pieces (id lists) representative of that class. Every kernel is run on
    every piece; a kernel that disagrees with the oracle on ANY piece of a class is rejected for that class, however fast
    it was. Classes without cases keep the reference kernel."""
    thresholds = thresholds or ElasticThresholds()
    chosen, timings, rejected = [], {}, {}
    for cls in CLASSES:
        pieces = cases.get(cls, [])
        if not pieces:
            chosen.append("reference")
            continue
        want = [oracle.encode_ids(p) for p in pieces]
        timings[cls], rejected[cls] = {}, []
        for name in KERNELS:
            fn = oracle.kernel(name)
            if any(fn(p) != w for p, w in zip(pieces, want)):
                rejected[cls].append(name)
                continue
            samples = []
            for _ in range(repeats):
                t0 = clock()
                for p in pieces:
                    fn(p)
                samples.append((clock() - t0) // max(len(pieces), 1))
            timings[cls][name] = sorted(samples)[len(samples) // 2]
        chosen.append(min(timings[cls], key=lambda k: (timings[cls][k], KERNELS.index(k))))
    return CalibrationReport(ElasticProfile(thresholds, tuple(chosen)), timings, rejected)

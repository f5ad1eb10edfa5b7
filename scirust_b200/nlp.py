"""Classical text processing: tokenisation, bag-of-words / TF-IDF vectorisers (dense tensors, so similarity matrices are
one matrix product), multinomial naive Bayes, MinHash + banded LSH for near-duplicate detection, keyword extraction
(TF-IDF, RAKE, TextRank), latent Dirichlet allocation by collapsed Gibbs sampling, gazetteer / rule NER with BIO tags,
Bloom filter, trie, canonical Huffman coding and string distances.
Reference counterpart: scirust-nlp-advanced/src/{tokenize,classify,similarity,lsh,keyword,topic,ner,bloom,trie,huffman}.rs.
"""
from __future__ import annotations

import hashlib
import heapq
import math
import re
from collections import Counter, defaultdict

import torch

_TOKEN = re.compile(r"[A-Za-z0-9]+(?:'[A-Za-z]+)?")
STOP_WORDS = frozenset("""a an and are as at be but by for from had has have he her his i if in into is it its me my no not of on or our
she so that the their them then there these they this to was we were what when which who will with you your
about after again all also am any been before being both can could did do does down each few here him how just may more most now
off once other out over own same should some such than too under up us very where why would""".split())


def tokenize(text: str) -> list:
    return _TOKEN.findall(text)


def normalize_token(tok: str) -> str:
    return tok.lower().strip("'")


def tokenize_normalized(text: str, drop_stop_words: bool = False) -> list:
    toks = [normalize_token(t) for t in tokenize(text)]
    return [t for t in toks if t and not (drop_stop_words and t in STOP_WORDS)]


# ------------------------------------------------------------------ vectorisers and similarity
class BagOfWords:
    def __init__(self, docs, min_count: int = 1):
        cnt = Counter(t for d in docs for t in tokenize_normalized(d))
        self.vocab = {w: i for i, w in enumerate(sorted(w for w, c in cnt.items() if c >= min_count))}

    def __len__(self):
        return len(self.vocab)

    def vectorize(self, docs, binary: bool = False) -> torch.Tensor:
        docs = [docs] if isinstance(docs, str) else list(docs)
        out = torch.zeros(len(docs), len(self.vocab), dtype=torch.float64)
        for r, d in enumerate(docs):
            for w, c in Counter(tokenize_normalized(d)).items():
                if w in self.vocab:
                    out[r, self.vocab[w]] = 1.0 if binary else float(c)
        return out


class TfidfVectorizer:
    """Smoothed idf ``ln((1 + n) / (1 + df)) + 1``, rows L2-normalised."""

    def __init__(self, docs):
        docs = list(docs)
        self.bow = BagOfWords(docs)
        df = (self.bow.vectorize(docs, binary=True)).sum(0)
        self.idf = torch.log((1 + len(docs)) / (1 + df)) + 1.0

    def transform(self, docs) -> torch.Tensor:
        x = self.bow.vectorize(docs) * self.idf
        return x / x.norm(dim=1, keepdim=True).clamp_min(1e-12)


def cosine_similarity_matrix(x: torch.Tensor) -> torch.Tensor:
    n = x / x.norm(dim=1, keepdim=True).clamp_min(1e-12)
    return n @ n.t()


def jaccard_similarity(a, b) -> float:
    a, b = set(a), set(b)
    return len(a & b) / len(a | b) if a | b else 1.0


def weighted_jaccard(a: dict, b: dict) -> float:
    keys = set(a) | set(b)
    den = sum(max(a.get(k, 0.0), b.get(k, 0.0)) for k in keys)
    return sum(min(a.get(k, 0.0), b.get(k, 0.0)) for k in keys) / den if den else 1.0


def levenshtein(a: str, b: str) -> int:
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


def most_similar(x: torch.Tensor, row: int, k: int = 5):
    s = cosine_similarity_matrix(x)[row]
    s[row] = -math.inf
    top = s.topk(min(k, x.shape[0] - 1))
    return list(zip(top.indices.tolist(), top.values.tolist()))


# ------------------------------------------------------------------ naive Bayes
class NaiveBayes:
    """Multinomial model with Laplace smoothing ``alpha``; prediction is one matrix product with the log-likelihoods."""

    def __init__(self, alpha: float = 1.0):
        self.alpha = alpha

    def train(self, docs, labels):
        docs, labels = list(docs), list(labels)
        if len(docs) != len(labels) or not docs:
            raise ValueError("one label per document, at least one document")
        self.bow = BagOfWords(docs)
        self.classes = sorted(set(labels))
        x = self.bow.vectorize(docs)
        onehot = torch.tensor([[float(l == c) for c in self.classes] for l in labels], dtype=torch.float64)
        counts = onehot.t() @ x + self.alpha
        self.log_lik = torch.log(counts / counts.sum(1, keepdim=True))
        self.log_prior = torch.log(onehot.sum(0) / len(docs))
        return self

    def _scores(self, docs):
        return self.bow.vectorize(docs) @ self.log_lik.t() + self.log_prior

    def predict(self, docs):
        single = isinstance(docs, str)
        out = [self.classes[i] for i in self._scores(docs).argmax(1).tolist()]
        return out[0] if single else out

    def predict_proba(self, docs) -> torch.Tensor:
        return torch.softmax(self._scores(docs), 1)


# ------------------------------------------------------------------ MinHash + LSH
_MERSENNE = (1 << 61) - 1


def _h64(s: str) -> int:
    return int.from_bytes(hashlib.blake2b(s.encode(), digest_size=8).digest(), "little")


class MinHash:
    def __init__(self, num_hashes: int = 128, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.a = [int(v) | 1 for v in torch.randint(1, 1 << 31, (num_hashes,), generator=g)]
        self.b = [int(v) for v in torch.randint(0, 1 << 31, (num_hashes,), generator=g)]

    def signature(self, items) -> list:
        hs = [_h64(str(i)) % _MERSENNE for i in set(items)]
        if not hs:
            return [_MERSENNE] * len(self.a)
        return [min((a * h + b) % _MERSENNE for h in hs) for a, b in zip(self.a, self.b)]

    @staticmethod
    def estimate_jaccard(s1, s2) -> float:
        return sum(x == y for x, y in zip(s1, s2)) / len(s1)


def shingles(text: str, k: int = 3) -> set:
    toks = tokenize_normalized(text)
    return {" ".join(toks[i:i + k]) for i in range(max(1, len(toks) - k + 1))}


class MinHashLsh:
    def __init__(self, bands: int = 32, rows: int = 4, seed: int = 0):
        self.bands, self.rows = bands, rows
        self.mh = MinHash(bands * rows, seed)
        self.tables = [defaultdict(list) for _ in range(bands)]
        self.signatures: dict = {}

    def estimated_threshold(self) -> float:
        return (1.0 / self.bands) ** (1.0 / self.rows)

    def _band_keys(self, sig):
        return [hash(tuple(sig[b * self.rows:(b + 1) * self.rows])) for b in range(self.bands)]

    def insert(self, key, items) -> None:
        sig = self.mh.signature(items)
        self.signatures[key] = sig
        for t, k in zip(self.tables, self._band_keys(sig)):
            t[k].append(key)

    def insert_doc(self, key, text: str, k: int = 3) -> None:
        self.insert(key, shingles(text, k))

    def query(self, items) -> list:
        sig = self.mh.signature(items)
        cands = {c for t, k in zip(self.tables, self._band_keys(sig)) for c in t.get(k, ())}
        return sorted(((c, MinHash.estimate_jaccard(sig, self.signatures[c])) for c in cands), key=lambda kv: (-kv[1], str(kv[0])))

    def query_doc(self, text: str, k: int = 3) -> list:
        return self.query(shingles(text, k))

    def duplicate_pairs(self, threshold: float = 0.8) -> list:
        seen = set()
        for t in self.tables:
            for bucket in t.values():
                for i, a in enumerate(bucket):
                    for b in bucket[i + 1:]:
                        seen.add((a, b) if str(a) <= str(b) else (b, a))
        out = [(a, b, MinHash.estimate_jaccard(self.signatures[a], self.signatures[b])) for a, b in seen]
        return sorted((p for p in out if p[2] >= threshold), key=lambda p: (-p[2], str(p[0]), str(p[1])))


# ------------------------------------------------------------------ keywords
def keyword_tfidf(doc: str, corpus, k: int = 5) -> list:
    vec = TfidfVectorizer(list(corpus) + [doc])
    row = vec.transform([doc])[0]
    inv = {i: w for w, i in vec.bow.vocab.items()}
    top = row.topk(min(k, int((row > 0).sum())))
    return [(inv[i], float(s)) for i, s in zip(top.indices.tolist(), top.values.tolist()) if inv[i] not in STOP_WORDS]


class Rake:
    """Candidate phrases = maximal runs of non-stop words inside a sentence; word score = degree / frequency; a phrase
    scores the sum of its words."""

    def __init__(self, stop_words=STOP_WORDS, max_words: int = 4):
        self.stop, self.max_words = stop_words, max_words

    def extract(self, text: str, k: int = 5) -> list:
        phrases = []
        for sentence in re.split(r"[.!?,;:()\n]+", text):
            cur = []
            for t in tokenize_normalized(sentence) + [None]:
                if t is None or t in self.stop:
                    if 0 < len(cur) <= self.max_words:
                        phrases.append(tuple(cur))
                    cur = []
                else:
                    cur.append(t)
        freq, degree = Counter(), Counter()
        for p in phrases:
            for w in p:
                freq[w] += 1
                degree[w] += len(p)
        scored = {p: sum(degree[w] / freq[w] for w in p) for p in set(phrases)}
        return [(" ".join(p), s) for p, s in sorted(scored.items(), key=lambda kv: (-kv[1], kv[0]))[:k]]


class TextRank:
    def __init__(self, window: int = 4, damping: float = 0.85, iters: int = 50):
        self.window, self.damping, self.iters = window, damping, iters

    def extract(self, text: str, k: int = 5) -> list:
        toks = tokenize_normalized(text, drop_stop_words=True)
        vocab = sorted(set(toks))
        if not vocab:
            return []
        idx = {w: i for i, w in enumerate(vocab)}
        adj = torch.zeros(len(vocab), len(vocab), dtype=torch.float64)
        for i, w in enumerate(toks):
            for u in toks[i + 1:i + self.window]:
                if u != w:
                    adj[idx[w], idx[u]] += 1
                    adj[idx[u], idx[w]] += 1
        trans = adj / adj.sum(0, keepdim=True).clamp_min(1e-12)
        r = torch.full((len(vocab),), 1.0 / len(vocab), dtype=torch.float64)
        for _ in range(self.iters):
            r = (1 - self.damping) / len(vocab) + self.damping * (trans @ r)
        top = r.topk(min(k, len(vocab)))
        return [(vocab[i], float(s)) for i, s in zip(top.indices.tolist(), top.values.tolist())]


# ------------------------------------------------------------------ LDA (collapsed Gibbs)
class LdaModel:
    def __init__(self, vocab, n_dk, n_kw, alpha, beta):
        self.vocab, self.n_dk, self.n_kw, self.alpha, self.beta = vocab, n_dk, n_kw, alpha, beta

    def topic_term_dist(self) -> torch.Tensor:
        x = self.n_kw + self.beta
        return x / x.sum(1, keepdim=True)

    def doc_topic_dist(self) -> torch.Tensor:
        x = self.n_dk + self.alpha
        return x / x.sum(1, keepdim=True)

    def top_words(self, topic: int, k: int = 5) -> list:
        return [self.vocab[i] for i in self.topic_term_dist()[topic].topk(k).indices.tolist()]

    def perplexity(self, docs_ids) -> float:
        phi, theta = self.topic_term_dist(), self.doc_topic_dist()
        ll, n = 0.0, 0
        for d, ids in enumerate(docs_ids):
            if ids:
                ll += float(torch.log(theta[d] @ phi[:, ids]).sum())
                n += len(ids)
        return math.exp(-ll / max(1, n))


def fit_lda_from_text(docs, topics: int, iters: int = 200, alpha: float = 0.1, beta: float = 0.01, seed: int = 0):
    """-> (model, docs as word-id lists). Stop words are dropped; each Gibbs sweep resamples every token's topic from
    ``(n_dk + alpha) (n_kw + beta) / (n_k + V beta)``."""
    toks = [tokenize_normalized(d, drop_stop_words=True) for d in docs]
    vocab = sorted({t for d in toks for t in d})
    if not vocab or topics < 1:
        raise ValueError("empty vocabulary or no topics")
    wid = {w: i for i, w in enumerate(vocab)}
    ids = [[wid[t] for t in d] for d in toks]
    g = torch.Generator().manual_seed(seed)
    v = len(vocab)
    n_dk = torch.zeros(len(docs), topics, dtype=torch.float64)
    n_kw = torch.zeros(topics, v, dtype=torch.float64)
    n_k = torch.zeros(topics, dtype=torch.float64)
    z = [[int(t) for t in torch.randint(topics, (len(d),), generator=g)] for d in ids]
    for d, (ws, zs) in enumerate(zip(ids, z)):
        for w, t in zip(ws, zs):
            n_dk[d, t] += 1
            n_kw[t, w] += 1
            n_k[t] += 1
    for _ in range(iters):
        for d, ws in enumerate(ids):
            u = torch.rand(len(ws), generator=g, dtype=torch.float64).tolist()
            for i, w in enumerate(ws):
                t = z[d][i]
                n_dk[d, t] -= 1
                n_kw[t, w] -= 1
                n_k[t] -= 1
                p = (n_dk[d] + alpha) * (n_kw[:, w] + beta) / (n_k + v * beta)
                c = torch.cumsum(p, 0)
                t = min(int(torch.searchsorted(c, u[i] * c[-1])), topics - 1)
                z[d][i] = t
                n_dk[d, t] += 1
                n_kw[t, w] += 1
                n_k[t] += 1
    return LdaModel(vocab, n_dk, n_kw, alpha, beta), ids


def coherence_umass(model: LdaModel, docs_ids, topic: int, k: int = 5) -> float:
    top = model.topic_term_dist()[topic].topk(k).indices.tolist()
    sets = [set(d) for d in docs_ids]
    score = 0.0
    for i in range(1, len(top)):
        for j in range(i):
            dj = sum(1 for s in sets if top[j] in s)
            dij = sum(1 for s in sets if top[j] in s and top[i] in s)
            score += math.log((dij + 1) / max(dj, 1))
    return score


# ------------------------------------------------------------------ named entities
class Gazetteer:
    def __init__(self):
        self.entries: dict = {}

    def add(self, phrase: str, entity_type: str) -> None:
        self.entries[tuple(tokenize_normalized(phrase))] = entity_type

    def add_many(self, phrases, entity_type: str) -> None:
        for p in phrases:
            self.add(p, entity_type)

    def max_entry_words(self) -> int:
        return max((len(k) for k in self.entries), default=0)

    def lookup(self, words):
        return self.entries.get(tuple(w.lower() for w in words))


class RuleBasedNer:
    """Longest gazetteer match first, then regular-expression patterns on the raw text (dates, e-mail, money, ...);
    ``bio_tags`` gives one B-/I-/O tag per token."""

    DEFAULT_PATTERNS = (("DATE", r"\b\d{4}-\d{2}-\d{2}\b"), ("EMAIL", r"\b[\w.+-]+@[\w-]+\.[\w.]+\b"),
                        ("MONEY", r"[$€£]\s?\d+(?:[.,]\d+)*"), ("PERCENT", r"\b\d+(?:\.\d+)?\s?%"))

    def __init__(self, gazetteer: Gazetteer | None = None):
        self.gaz = gazetteer or Gazetteer()
        self.patterns = [(t, re.compile(p)) for t, p in self.DEFAULT_PATTERNS]

    def add_pattern(self, entity_type: str, pattern: str) -> None:
        self.patterns.append((entity_type, re.compile(pattern)))

    def extract(self, text: str) -> list:
        """-> [(surface text, type, start char, end char)] without overlaps, in text order."""
        spans = []
        toks = [(m.group(), m.start(), m.end()) for m in _TOKEN.finditer(text)]
        i, longest = 0, self.gaz.max_entry_words()
        while i < len(toks):
            for n in range(min(longest, len(toks) - i), 0, -1):
                t = self.gaz.lookup([normalize_token(w) for w, _, _ in toks[i:i + n]])
                if t:
                    spans.append((text[toks[i][1]:toks[i + n - 1][2]], t, toks[i][1], toks[i + n - 1][2]))
                    i += n - 1
                    break
            i += 1
        for t, rx in self.patterns:
            for m in rx.finditer(text):
                if all(m.end() <= s or m.start() >= e for _, _, s, e in spans):
                    spans.append((m.group(), t, m.start(), m.end()))
        return sorted(spans, key=lambda s: s[2])

    def bio_tags(self, text: str) -> list:
        ents = self.extract(text)
        out = []
        for m in _TOKEN.finditer(text):
            tag = "O"
            for _, t, s, e in ents:
                if s <= m.start() < e:
                    tag = ("B-" if m.start() == s else "I-") + t
            out.append((m.group(), tag))
        return out


def word_shape(tok: str) -> str:
    """``Xxxx``-style shape with runs collapsed: "McDonald's" -> "XxXx'x", "2024" -> "d"."""
    out = []
    for c in tok:
        s = "X" if c.isupper() else "x" if c.islower() else "d" if c.isdigit() else c
        if not out or out[-1] != s:
            out.append(s)
    return "".join(out)


# ------------------------------------------------------------------ Bloom filter, trie, Huffman
class BloomFilter:
    def __init__(self, expected_items: int, fpr: float = 0.01):
        if expected_items < 1 or not 0 < fpr < 1:
            raise ValueError("expected_items >= 1 and 0 < fpr < 1")
        self.m = max(8, math.ceil(-expected_items * math.log(fpr) / math.log(2) ** 2))
        self.k = max(1, round(self.m / expected_items * math.log(2)))
        self.bits = bytearray((self.m + 7) // 8)
        self.count = 0

    def _positions(self, item: bytes):
        d = hashlib.blake2b(item, digest_size=16).digest()
        h1, h2 = int.from_bytes(d[:8], "little"), int.from_bytes(d[8:], "little") | 1
        return [(h1 + i * h2) % self.m for i in range(self.k)]

    def insert(self, item) -> None:
        for p in self._positions(item if isinstance(item, bytes) else str(item).encode()):
            self.bits[p >> 3] |= 1 << (p & 7)
        self.count += 1

    def contains(self, item) -> bool:
        return all(self.bits[p >> 3] >> (p & 7) & 1 for p in self._positions(item if isinstance(item, bytes) else str(item).encode()))

    __contains__ = contains

    def bits_set(self) -> int:
        return sum(bin(b).count("1") for b in self.bits)

    def estimated_fpr(self) -> float:
        return (self.bits_set() / self.m) ** self.k

    def merge(self, other: "BloomFilter") -> None:
        if (self.m, self.k) != (other.m, other.k):
            raise ValueError("filters differ in size or hash count")
        self.bits = bytearray(a | b for a, b in zip(self.bits, other.bits))
        self.count += other.count


class Trie:
    def __init__(self):
        self.root: dict = {}
        self.size = 0

    def insert(self, word: str) -> None:
        node = self.root
        for c in word:
            node = node.setdefault(c, {})
        if "" not in node:
            node[""] = True
            self.size += 1

    def __len__(self):
        return self.size

    def __contains__(self, word: str) -> bool:
        node = self.root
        for c in word:
            node = node.get(c)
            if node is None:
                return False
        return "" in node

    def longest_prefix(self, text: str) -> str:
        node, best = self.root, ""
        for i, c in enumerate(text):
            node = node.get(c)
            if node is None:
                break
            if "" in node:
                best = text[:i + 1]
        return best

    def with_prefix(self, prefix: str) -> list:
        node = self.root
        for c in prefix:
            node = node.get(c)
            if node is None:
                return []
        out, stack = [], [(prefix, node)]
        while stack:
            p, n = stack.pop()
            for c, child in n.items():
                if c == "":
                    out.append(p)
                else:
                    stack.append((p + c, child))
        return sorted(out)

    def node_count(self) -> int:
        n, stack = 0, [self.root]
        while stack:
            node = stack.pop()
            n += 1
            stack += [c for k, c in node.items() if k != ""]
        return n


class HuffmanCodebook:
    """Canonical Huffman code over bytes: only the code LENGTHS need storing; codes are assigned in (length, symbol) order."""

    def __init__(self, lengths: dict):
        self.lengths = dict(lengths)
        code, prev, self.codes = 0, 0, {}
        for sym, ln in sorted(self.lengths.items(), key=lambda kv: (kv[1], kv[0])):
            code <<= ln - prev
            self.codes[sym] = (code, ln)
            code, prev = code + 1, ln
        self.decode_map = {(ln, c): s for s, (c, ln) in self.codes.items()}

    @staticmethod
    def from_data(data: bytes) -> "HuffmanCodebook":
        freq = Counter(data)
        if not freq:
            raise ValueError("empty input")
        if len(freq) == 1:
            return HuffmanCodebook({next(iter(freq)): 1})
        heap = [(f, s, (s,)) for s, f in freq.items()]
        heapq.heapify(heap)
        depth = Counter()
        while len(heap) > 1:
            fa, sa, a = heapq.heappop(heap)
            fb, sb, b = heapq.heappop(heap)
            for s in a + b:
                depth[s] += 1
            heapq.heappush(heap, (fa + fb, min(sa, sb), a + b))
        return HuffmanCodebook(depth)

    def encode(self, data: bytes):
        """-> (packed bytes, number of valid bits)."""
        acc, n = 0, 0
        for b in data:
            c, ln = self.codes[b]
            acc, n = (acc << ln) | c, n + ln
        pad = (-n) % 8
        return (acc << pad).to_bytes((n + pad) // 8, "big"), n

    def decode(self, packed: bytes, bits: int) -> bytes:
        acc = int.from_bytes(packed, "big") >> ((-bits) % 8)
        out, code, ln = bytearray(), 0, 0
        for i in range(bits - 1, -1, -1):
            code, ln = (code << 1) | ((acc >> i) & 1), ln + 1
            s = self.decode_map.get((ln, code))
            if s is not None:
                out.append(s)
                code, ln = 0, 0
        if ln:
            raise ValueError("trailing bits do not form a code word")
        return bytes(out)

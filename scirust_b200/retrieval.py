"""Vector and lexical retrieval for retrieval-augmented generation. Dense scoring is one matrix product and a top-k on
the device that holds the index (``[queries, dim] @ [dim, items]``), so a batch of queries costs one GEMM, not a loop.

* ``DenseIndex``: exact inner-product / cosine search over a growing matrix (chunked append, optional bf16 storage).
* ``IvfIndex``: inverted file: k-means coarse centroids, each item listed under its nearest centroid; a query scans the
  ``nprobe`` nearest lists only. ``nprobe = nlist`` is exact.
* ``LshIndex``: random-hyperplane signatures in several tables; candidates that share a bucket are re-scored exactly.
* ``Bm25Index``: Okapi BM25 over lower-cased alphanumeric tokens; ``reciprocal_rank_fusion`` merges rankings;
  ``HybridRetriever`` fuses the dense and the lexical ranking.
* ``maxsim`` / ``rerank``: late-interaction scoring (sum over query tokens of the best document-token similarity).
* metrics: recall@k, precision@k, reciprocal rank, MRR, average precision, nDCG@k.
* vector-symbolic algebra: circular convolution / correlation (FFT), superposition, a clean-up memory.
* ``ProjectionHead`` + ``infonce_loss`` + ``train_contrastive``: a linear head on frozen embeddings trained on positive pairs.
* ``RagContext``: index chunks, retrieve for a question, assemble a prompt under a character or chunk budget.
An encoder is any object with ``embed_batch(list[str]) -> [n, dim]`` (``scirust_b200.embed.EmbeddingEngine`` is one).
Reference counterpart: scirust-retrieval/src/{index,ivf,ann,hybrid,rerank,metrics,vsa,contrastive,rag,vector}.rs.
"""
from __future__ import annotations

import math
import re
from collections import Counter, defaultdict
from dataclasses import dataclass

import torch


def normalized(v: torch.Tensor) -> torch.Tensor:
    return v / v.norm(dim=-1, keepdim=True).clamp_min(1e-12)


def cosine(a, b) -> torch.Tensor:
    return (normalized(torch.as_tensor(a, dtype=torch.float32)) * normalized(torch.as_tensor(b, dtype=torch.float32))).sum(-1)


def _rows(v, dim=None):
    v = torch.as_tensor(v, dtype=torch.float32)
    v = v[None] if v.dim() == 1 else v
    if dim is not None and v.shape[1] != dim:
        raise ValueError(f"expected vectors of dimension {dim}, got {v.shape[1]}")
    return v


# ------------------------------------------------------------------ dense indexes
class DenseIndex:
    def __init__(self, dim: int, metric: str = "cosine", device="cpu", storage_dtype=torch.float32):
        if metric not in ("cosine", "dot"):
            raise ValueError("metric is cosine or dot")
        self.dim, self.metric, self.device, self.dtype = dim, metric, torch.device(device), storage_dtype
        self._buf = torch.empty(0, dim, dtype=storage_dtype, device=self.device)
        self._n = 0
        self.ids: list = []

    def __len__(self):
        return self._n

    def add(self, vectors, ids=None) -> None:
        v = _rows(vectors, self.dim)
        if not bool(torch.isfinite(v).all()):
            raise ValueError("vectors must be finite")
        if self.metric == "cosine":
            v = normalized(v)
        n = v.shape[0]
        if self._n + n > self._buf.shape[0]:                                  # amortised growth: no re-copy per insert
            grown = torch.empty(max(2 * self._buf.shape[0], self._n + n, 64), self.dim, dtype=self.dtype, device=self.device)
            grown[:self._n] = self._buf[:self._n]
            self._buf = grown
        self._buf[self._n:self._n + n] = v.to(self.device, self.dtype)
        self.ids += list(ids) if ids is not None else list(range(self._n, self._n + n))
        self._n += n
        if len(self.ids) != self._n:
            raise ValueError("one id per vector")

    @property
    def matrix(self):
        return self._buf[:self._n]

    def search(self, queries, k: int = 10):
        """-> (scores [q, k'], ids: list of lists), best first, k' = min(k, len)."""
        q = _rows(queries, self.dim).to(self.device)
        if self.metric == "cosine":
            q = normalized(q)
        if self._n == 0:
            return torch.empty(q.shape[0], 0), [[] for _ in range(q.shape[0])]
        scores = (q.to(self.dtype) @ self.matrix.t()).float()
        top = scores.topk(min(k, self._n), dim=1)
        return top.values.cpu(), [[self.ids[j] for j in row] for row in top.indices.tolist()]


class IvfIndex:
    def __init__(self, vectors, nlist: int = 16, metric: str = "cosine", iters: int = 20, seed: int = 0, ids=None):
        v = _rows(vectors)
        self.dim, self.metric = v.shape[1], metric
        v = normalized(v) if metric == "cosine" else v
        nlist = max(1, min(nlist, v.shape[0]))
        g = torch.Generator().manual_seed(seed)
        c = v[torch.randperm(v.shape[0], generator=g)[:nlist]].clone()
        assign = None
        for _ in range(iters):
            new = torch.cdist(v, c).argmin(1)
            if assign is not None and torch.equal(new, assign):
                break
            assign = new
            one = torch.nn.functional.one_hot(assign, nlist).float()
            cnt = one.sum(0)
            c = torch.where(cnt[:, None] > 0, (one.t() @ v) / cnt.clamp_min(1)[:, None], c)
        self.centroids, self.vectors = c, v
        self.lists = [torch.nonzero(assign == j)[:, 0] for j in range(nlist)]
        self.ids = list(ids) if ids is not None else list(range(v.shape[0]))

    def __len__(self):
        return self.vectors.shape[0]

    @property
    def nlist(self):
        return len(self.lists)

    def search(self, query, k: int = 10, nprobe: int = 4):
        q = _rows(query, self.dim)[0]
        q = normalized(q) if self.metric == "cosine" else q
        probe = torch.cdist(q[None], self.centroids)[0].topk(min(nprobe, self.nlist), largest=False).indices
        cand = torch.cat([self.lists[int(j)] for j in probe])
        if cand.numel() == 0:
            return torch.empty(0), []
        top = (self.vectors[cand] @ q).topk(min(k, cand.numel()))
        return top.values, [self.ids[int(cand[j])] for j in top.indices]


class LshIndex:
    def __init__(self, dim: int, bits: int = 12, tables: int = 8, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        self.dim, self.planes = dim, torch.randn(tables, bits, dim, generator=g)
        self.pow = (2 ** torch.arange(bits)).long()
        self.buckets = [defaultdict(list) for _ in range(tables)]
        self.vectors: list = []

    def __len__(self):
        return len(self.vectors)

    def _keys(self, v):
        return ((torch.einsum("tbd,d->tb", self.planes, v) > 0).long() * self.pow).sum(1).tolist()

    def add(self, vector) -> int:
        v = normalized(_rows(vector, self.dim)[0])
        i = len(self.vectors)
        self.vectors.append(v)
        for t, key in enumerate(self._keys(v)):
            self.buckets[t][key].append(i)
        return i

    def search(self, query, k: int = 10):
        q = normalized(_rows(query, self.dim)[0])
        cand = sorted({i for t, key in enumerate(self._keys(q)) for i in self.buckets[t].get(key, ())})
        if not cand:
            return torch.empty(0), []
        top = (torch.stack([self.vectors[i] for i in cand]) @ q).topk(min(k, len(cand)))
        return top.values, [cand[j] for j in top.indices.tolist()]


# ------------------------------------------------------------------ lexical + fusion
_WORD = re.compile(r"[a-z0-9]+")


def tokenize(text: str):
    return _WORD.findall(text.lower())


class Bm25Index:
    def __init__(self, k1: float = 1.2, b: float = 0.75):
        self.k1, self.b = k1, b
        self.docs: list = []
        self.df: Counter = Counter()
        self.total_len = 0

    def __len__(self):
        return len(self.docs)

    def add(self, text: str) -> int:
        tf = Counter(tokenize(text))
        self.docs.append(tf)
        self.df.update(tf.keys())
        self.total_len += sum(tf.values())
        return len(self.docs) - 1

    def search(self, query: str, k: int = 10):
        """-> [(doc id, score)], best first; documents that share no term with the query are left out."""
        n = len(self.docs)
        if n == 0:
            return []
        avg = self.total_len / n
        scores = defaultdict(float)
        for term in set(tokenize(query)):
            df = self.df.get(term, 0)
            if not df:
                continue
            idf = math.log(1 + (n - df + 0.5) / (df + 0.5))
            for i, tf in enumerate(self.docs):
                f = tf.get(term, 0)
                if f:
                    scores[i] += idf * f * (self.k1 + 1) / (f + self.k1 * (1 - self.b + self.b * sum(tf.values()) / avg))
        return sorted(scores.items(), key=lambda kv: (-kv[1], kv[0]))[:k]


def reciprocal_rank_fusion(rankings, k: int = 60):
    """Rankings are lists of ids, best first -> [(id, score)] with score = sum 1 / (k + rank)."""
    score = defaultdict(float)
    for r in rankings:
        for rank, i in enumerate(r, 1):
            score[i] += 1.0 / (k + rank)
    return sorted(score.items(), key=lambda kv: (-kv[1], kv[0]))


class HybridRetriever:
    def __init__(self, encoder, dim: int | None = None, device="cpu"):
        self.encoder = encoder
        self.dense = DenseIndex(dim or encoder.dimension(), device=device)
        self.lexical = Bm25Index()
        self.texts: list = []

    def __len__(self):
        return len(self.texts)

    def index_texts(self, texts) -> None:
        texts = list(texts)
        self.dense.add(self.encoder.embed_batch(texts), ids=range(len(self.texts), len(self.texts) + len(texts)))
        for t in texts:
            self.lexical.add(t)
        self.texts += texts

    def index_text(self, text: str) -> int:
        self.index_texts([text])
        return len(self.texts) - 1

    def retrieve(self, query: str, k: int = 5, pool: int = 20):
        dense_ids = self.dense.search(self.encoder.embed_batch([query]), pool)[1][0]
        lex_ids = [i for i, _ in self.lexical.search(query, pool)]
        return [(i, s, self.texts[i]) for i, s in reciprocal_rank_fusion([dense_ids, lex_ids])[:k]]


# ------------------------------------------------------------------ late interaction
def maxsim(query_tokens, doc_tokens) -> torch.Tensor:
    """``[q, d]`` x ``[..., t, d]`` token embeddings -> sum over query tokens of the best cosine with a document token."""
    q, d = normalized(torch.as_tensor(query_tokens, dtype=torch.float32)), normalized(torch.as_tensor(doc_tokens, dtype=torch.float32))
    return (q @ d.transpose(-1, -2)).max(-1).values.sum(-1)


def rerank(query_tokens, docs_tokens, candidates):
    """Re-order candidate ids by ``maxsim``; ``docs_tokens[id]`` = that document's token matrix."""
    scored = [(i, float(maxsim(query_tokens, docs_tokens[i]))) for i in candidates]
    return sorted(scored, key=lambda kv: (-kv[1], kv[0]))


# ------------------------------------------------------------------ metrics
def recall_at_k(retrieved, relevant, k):
    rel = set(relevant)
    return len(rel & set(retrieved[:k])) / len(rel) if rel else 0.0


def precision_at_k(retrieved, relevant, k):
    return len(set(relevant) & set(retrieved[:k])) / k if k else 0.0


def reciprocal_rank(retrieved, relevant):
    rel = set(relevant)
    return next((1.0 / r for r, i in enumerate(retrieved, 1) if i in rel), 0.0)


def mean_reciprocal_rank(runs):
    runs = list(runs)
    return sum(reciprocal_rank(a, b) for a, b in runs) / len(runs) if runs else 0.0


def average_precision(retrieved, relevant):
    rel, hits, total = set(relevant), 0, 0.0
    for r, i in enumerate(retrieved, 1):
        if i in rel:
            hits += 1
            total += hits / r
    return total / len(rel) if rel else 0.0


def ndcg_at_k(retrieved, gains: dict, k):
    dcg = sum(gains.get(i, 0.0) / math.log2(r + 1) for r, i in enumerate(retrieved[:k], 1))
    ideal = sum(g / math.log2(r + 1) for r, g in enumerate(sorted(gains.values(), reverse=True)[:k], 1))
    return dcg / ideal if ideal > 0 else 0.0


# ------------------------------------------------------------------ vector-symbolic algebra
def circular_convolution(a, b):
    a, b = torch.as_tensor(a, dtype=torch.float64), torch.as_tensor(b, dtype=torch.float64)
    return torch.fft.irfft(torch.fft.rfft(a) * torch.fft.rfft(b), n=a.shape[-1])


def involution(a):
    a = torch.as_tensor(a, dtype=torch.float64)
    return torch.cat([a[..., :1], a[..., 1:].flip(-1)], -1)


def circular_correlation(a, b):
    """Approximate unbinding: ``correlation(a, convolution(a, b)) ~ b`` for random unit-variance/d vectors."""
    return circular_convolution(involution(a), b)


def superpose(vectors):
    return normalized(torch.stack([torch.as_tensor(v, dtype=torch.float64) for v in vectors]).sum(0))


class CleanupMemory:
    def __init__(self, dim: int):
        self.dim, self.names, self.rows = dim, [], []

    def __len__(self):
        return len(self.names)

    def insert(self, name: str, vector) -> None:
        v = torch.as_tensor(vector, dtype=torch.float64)
        if v.shape != (self.dim,):
            raise ValueError(f"expected a vector of dimension {self.dim}")
        self.names.append(name)
        self.rows.append(normalized(v))

    def clean(self, noisy):
        """-> (name, cosine, margin to the runner-up) of the nearest stored item, or None when empty."""
        if not self.rows:
            return None
        s = torch.stack(self.rows) @ normalized(torch.as_tensor(noisy, dtype=torch.float64))
        top = s.topk(min(2, len(self.rows)))
        margin = float(top.values[0] - top.values[1]) if len(self.rows) > 1 else float(top.values[0])
        return self.names[int(top.indices[0])], float(top.values[0]), margin


# ------------------------------------------------------------------ contrastive projection head
class ProjectionHead(torch.nn.Module):
    def __init__(self, dim_in: int, dim_out: int, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.w = torch.nn.Parameter(torch.randn(dim_in, dim_out, generator=g) / math.sqrt(dim_in))

    def forward(self, x):
        return normalized(torch.as_tensor(x, dtype=torch.float32) @ self.w)

    project = forward


def infonce_loss(anchors, positives, temperature: float = 0.07):
    """Row i of ``positives`` is the match of row i of ``anchors``; every other row of the batch is a negative."""
    logits = normalized(anchors) @ normalized(positives).t() / temperature
    return torch.nn.functional.cross_entropy(logits, torch.arange(logits.shape[0], device=logits.device))


def train_contrastive(head: ProjectionHead, anchors, positives, steps: int = 200, lr: float = 1e-2, temperature: float = 0.07):
    opt = torch.optim.Adam(head.parameters(), lr=lr)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = infonce_loss(head(anchors), head(positives), temperature)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


class ProjectedEncoder:
    def __init__(self, encoder, head: ProjectionHead):
        self.encoder, self.head = encoder, head

    def dimension(self) -> int:
        return self.head.w.shape[1]

    @torch.no_grad()
    def embed_batch(self, texts):
        return self.head(self.encoder.embed_batch(texts))


# ------------------------------------------------------------------ retrieval-augmented prompts
@dataclass
class AugmentedPrompt:
    prompt: str
    sources: list
    truncated: bool


class RagContext:
    def __init__(self, retriever: HybridRetriever, template: str = "Context:\n{context}\n\nQuestion: {question}\nAnswer:"):
        self.retriever, self.template = retriever, template

    def index_chunk(self, text: str) -> int:
        return self.retriever.index_text(text)

    def augment(self, question: str, k: int = 3, max_chars: int | None = None, max_chunks: int | None = None) -> AugmentedPrompt:
        hits = self.retriever.retrieve(question, k)
        if max_chunks is not None:
            hits = hits[:max_chunks]
        parts, used, truncated = [], 0, False
        for n, (i, _, text) in enumerate(hits, 1):
            piece = f"[{n}] {text}"
            if max_chars is not None and used + len(piece) > max_chars:
                room = max_chars - used
                if room > 8:
                    parts.append(piece[:room])
                truncated = True
                break
            parts.append(piece)
            used += len(piece) + 1
        return AugmentedPrompt(self.template.format(context="\n".join(parts), question=question), [i for i, _, _ in hits[:len(parts)]], truncated)

    def generate_with(self, question: str, generate, **kw):
        """``generate(prompt) -> str`` is any text generator; -> (answer, the prompt that was used)."""
        p = self.augment(question, **kw)
        return generate(p.prompt), p

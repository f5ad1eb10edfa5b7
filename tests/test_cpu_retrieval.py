"""Dense / inverted-file / LSH / BM25 retrieval, fusion, late interaction, metrics, vector-symbolic algebra, contrastive
head and retrieval-augmented prompts (CPU)."""
import math

import pytest
import torch

from scirust_b200 import retrieval as R


class BagEncoder:
    """Deterministic hashed bag-of-words embedding: enough structure for ranking tests without a trained model."""

    def __init__(self, dim=64):
        self.dim = dim

    def dimension(self):
        return self.dim

    def embed_batch(self, texts):
        out = torch.zeros(len(texts), self.dim)
        for r, t in enumerate(texts):
            for w in R.tokenize(t):
                h = sum((i + 1) * ord(c) for i, c in enumerate(w))
                out[r, h % self.dim] += 1.0
                out[r, (h * 31 + 7) % self.dim] += 0.5
        return R.normalized(out)


def _data(n=2000, d=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, d, generator=g), torch.randn(20, d, generator=g)


def test_dense_index_is_exact_and_grows():
    x, q = _data()
    idx = R.DenseIndex(32)
    for s in range(0, 2000, 300):                                             # several appends: the buffer regrows
        idx.add(x[s:s + 300])
    assert len(idx) == 2000
    scores, ids = idx.search(q, 5)
    ref = (R.normalized(q) @ R.normalized(x).t()).topk(5, dim=1)
    assert [list(r) for r in ref.indices.tolist()] == ids and torch.allclose(scores, ref.values, atol=1e-6)
    dot = R.DenseIndex(32, metric="dot")
    dot.add(x, ids=[f"doc{i}" for i in range(2000)])
    assert dot.search(q[0], 1)[1][0][0] == f"doc{int((x @ q[0]).argmax())}"
    assert R.DenseIndex(4).search(torch.zeros(4), 3)[1] == [[]]
    with pytest.raises(ValueError):
        idx.add(torch.zeros(3, 8))
    with pytest.raises(ValueError):
        idx.add(torch.full((1, 32), float("nan")))


def test_inverted_file_and_lsh_trade_recall_for_work():
    x, q = _data()
    exact = R.DenseIndex(32)
    exact.add(x)
    truth = exact.search(q, 10)[1]
    ivf = R.IvfIndex(x, nlist=16)
    assert sum(len(l) for l in ivf.lists) == 2000 and ivf.nlist == 16
    full = [ivf.search(q[i], 10, nprobe=16)[1] for i in range(20)]
    assert full == truth                                                       # probing every list is exact
    rec = lambda res: sum(R.recall_at_k(res[i], truth[i], 10) for i in range(20)) / 20
    r1, r4 = rec([ivf.search(q[i], 10, nprobe=1)[1] for i in range(20)]), rec([ivf.search(q[i], 10, nprobe=6)[1] for i in range(20)])
    assert r1 < r4 and r4 > 0.6
    lsh = R.LshIndex(32, bits=8, tables=12)
    for v in x[:500]:
        lsh.add(v)
    near = x[17] + 0.05 * torch.randn(32, generator=torch.Generator().manual_seed(1))
    assert lsh.search(near, 3)[1][0] == 17 and len(lsh) == 500


def test_bm25_fusion_and_hybrid_retrieval():
    docs = ["the cat sat on the mat", "dogs chase cats in the park", "quantum circuits use qubits and gates",
            "tensor cores multiply matrices quickly", "the mat was red"]
    bm = R.Bm25Index()
    for d in docs:
        bm.add(d)
    hits = bm.search("cat mat", 3)
    assert hits[0][0] == 0 and {i for i, _ in hits} == {0, 4} and bm.search("zebra") == []
    assert bm.search("the")[0][1] < bm.search("qubits")[0][1]                  # common words weigh less
    fused = R.reciprocal_rank_fusion([[1, 2, 3], [3, 1, 4]])
    assert [i for i, _ in fused][:2] == [1, 3] and fused[0][1] == pytest.approx(1 / 61 + 1 / 62)
    hy = R.HybridRetriever(BagEncoder())
    hy.index_texts(docs)
    top = hy.retrieve("which gates act on qubits", 2)
    assert top[0][0] == 2 and top[0][2] == docs[2] and len(hy) == 5


def test_late_interaction_and_ranking_metrics():
    g = torch.Generator().manual_seed(2)
    qtok = torch.randn(4, 16, generator=g)
    docs = {0: torch.randn(9, 16, generator=g), 1: torch.cat([qtok + 0.01 * torch.randn(4, 16, generator=g), torch.randn(5, 16, generator=g)]),
            2: torch.randn(9, 16, generator=g)}
    order = R.rerank(qtok, docs, [0, 1, 2])
    assert order[0][0] == 1 and abs(order[0][1] - 4.0) < 0.01                  # every query token finds its twin
    assert R.maxsim(qtok, torch.stack([docs[0], docs[1]])).shape == (2,)
    got, rel = [3, 1, 7, 2, 9], [1, 2, 5]
    assert R.recall_at_k(got, rel, 3) == pytest.approx(1 / 3) and R.precision_at_k(got, rel, 4) == 0.5
    assert R.reciprocal_rank(got, rel) == 0.5 and R.mean_reciprocal_rank([(got, rel), ([5], [5])]) == 0.75
    assert R.average_precision(got, rel) == pytest.approx((1 / 2 + 2 / 4) / 3)
    gains = {1: 3.0, 2: 1.0}
    assert R.ndcg_at_k([1, 2], gains, 2) == 1.0 and R.ndcg_at_k([2, 1], gains, 2) == pytest.approx((1 + 3 / math.log2(3)) / (3 + 1 / math.log2(3)))
    assert R.ndcg_at_k([8], {}, 3) == 0.0 and R.recall_at_k([1], [], 1) == 0.0


def test_vector_symbolic_binding_and_cleanup():
    d = 1024
    g = torch.Generator().manual_seed(3)
    vec = {n: torch.randn(d, generator=g, dtype=torch.float64) / math.sqrt(d) for n in ("role_a", "role_b", "x", "y", "z")}
    mem = R.CleanupMemory(d)
    for n in ("x", "y", "z"):
        mem.insert(n, vec[n])
    record = R.circular_convolution(vec["role_a"], vec["x"]) + R.circular_convolution(vec["role_b"], vec["y"])
    name, cos, margin = mem.clean(R.circular_correlation(vec["role_a"], record))
    assert name == "x" and cos > 0.5 and margin > 0.3
    assert mem.clean(R.circular_correlation(vec["role_b"], record))[0] == "y"
    a, b = vec["x"], vec["y"]
    direct = torch.stack([sum(a[j] * b[(i - j) % d] for j in range(d)) for i in range(4)])
    assert torch.allclose(R.circular_convolution(a, b)[:4], direct, atol=1e-12)
    assert torch.allclose(R.circular_convolution(a, b), R.circular_convolution(b, a))
    assert abs(float(R.superpose([a, b, vec["z"]]).norm()) - 1) < 1e-12 and R.CleanupMemory(4).clean(torch.zeros(4)) is None


def test_contrastive_head_and_augmented_prompts():
    g = torch.Generator().manual_seed(4)
    signal = torch.randn(32, 8, generator=g)
    anchors = torch.cat([signal, torch.randn(32, 24, generator=g) * 3], 1)      # 8 shared dims buried under 24 nuisance dims
    positives = torch.cat([signal, torch.randn(32, 24, generator=g) * 3], 1)
    head = R.ProjectionHead(32, 8)
    before = float(R.infonce_loss(head(anchors), head(positives)))
    losses = R.train_contrastive(head, anchors, positives, steps=150, lr=5e-2)
    assert losses[-1] < 0.2 * before
    hits = (head(anchors) @ head(positives).t()).argmax(1)
    assert float((hits == torch.arange(32)).float().mean()) > 0.9
    enc = R.ProjectedEncoder(BagEncoder(32), R.ProjectionHead(32, 8))
    assert enc.embed_batch(["a b", "c"]).shape == (2, 8) and enc.dimension() == 8
    rag = R.RagContext(R.HybridRetriever(BagEncoder()))
    for t in ("Blackwell tensor cores keep accumulators in tensor memory.", "NVLink connects the GPUs through a switch.",
              "Cats sleep most of the day."):
        rag.index_chunk(t)
    p = rag.augment("where do tensor cores keep accumulators", k=2)
    assert "[1] Blackwell tensor cores" in p.prompt and p.prompt.endswith("Answer:") and p.sources[0] == 0 and not p.truncated
    short = rag.augment("where do tensor cores keep accumulators", k=2, max_chars=30)
    assert short.truncated and len(short.sources) == 1
    answer, used = rag.generate_with("what connects the GPUs", lambda prompt: "NVLink" if "NVLink" in prompt else "?", k=1)
    assert answer == "NVLink" and used.sources == [1]

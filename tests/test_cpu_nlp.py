"""Classical text processing (CPU)."""
import math

import pytest
import torch

from scirust_b200 import nlp as N

SPORT = ["the team won the football match", "a great goal in the second half", "the striker scored twice in the match",
         "fans cheered the team after the goal"]
TECH = ["the new gpu has faster tensor cores", "the compiler emits tensor core instructions", "memory bandwidth limits the kernel",
        "the kernel uses shared memory and the gpu cache"]


def test_tokens_vectorisers_and_similarity():
    assert N.tokenize("Don't panic: it's 42!") == ["Don't", "panic", "it's", "42"]
    assert N.tokenize_normalized("The GPU and the CPU", drop_stop_words=True) == ["gpu", "cpu"]
    bow = N.BagOfWords(SPORT + TECH)
    v = bow.vectorize("the team the team")
    assert float(v[0, bow.vocab["team"]]) == 2.0 and float(bow.vectorize("the team the team", binary=True).sum()) == 2.0
    tf = N.TfidfVectorizer(SPORT + TECH)
    x = tf.transform(SPORT + TECH)
    assert torch.allclose(x.norm(dim=1), torch.ones(8, dtype=torch.float64))
    assert float(tf.idf[tf.bow.vocab["the"]]) < float(tf.idf[tf.bow.vocab["striker"]])
    sim = N.cosine_similarity_matrix(x)
    assert float(sim[:4, :4].mean()) > float(sim[:4, 4:].mean()) and N.most_similar(x, 4, 1)[0][0] in (5, 6, 7)
    assert N.jaccard_similarity("abc", "bcd") == 0.5 and N.weighted_jaccard({"a": 2, "b": 1}, {"a": 1, "c": 1}) == 0.25
    assert N.levenshtein("kitten", "sitting") == 3 and N.levenshtein("", "abc") == 3
    assert N.word_shape("McDonald's") == "XxXx'x" and N.word_shape("2024") == "d"


def test_naive_bayes_separates_topics():
    nb = N.NaiveBayes().train(SPORT + TECH, ["sport"] * 4 + ["tech"] * 4)
    assert nb.predict("the striker scored a goal") == "sport" and nb.predict(["gpu memory kernel"]) == ["tech"]
    p = nb.predict_proba(["the match", "tensor cores"])
    assert torch.allclose(p.sum(1), torch.ones(2, dtype=torch.float64)) and float(p[0, 0]) > 0.5 and float(p[1, 1]) > 0.5
    with pytest.raises(ValueError):
        N.NaiveBayes().train(["a"], [])


def test_minhash_lsh_finds_near_duplicates():
    a = set(range(100))
    b = set(range(20, 120))                                                   # Jaccard 80 / 120
    mh = N.MinHash(256)
    assert abs(N.MinHash.estimate_jaccard(mh.signature(a), mh.signature(b)) - 2 / 3) < 0.1
    lsh = N.MinHashLsh(bands=32, rows=4)
    base = "the quick brown fox jumps over the lazy dog near the quiet river bank at dawn"
    lsh.insert_doc("orig", base)
    lsh.insert_doc("near", base.replace("quiet", "silent"))
    lsh.insert_doc("other", "tensor cores multiply matrices while the memory system streams operands from cache")
    hits = lsh.query_doc(base)
    assert hits[0] == ("orig", 1.0) and hits[1][0] == "near" and all(k != "other" for k, _ in hits)
    pairs = lsh.duplicate_pairs(0.5)
    assert [(a_, b_) for a_, b_, _ in pairs] == [("near", "orig")] and 0.3 < lsh.estimated_threshold() < 0.5


def test_keyword_extractors():
    text = ("Compatibility of systems of linear constraints over the set of natural numbers. Criteria of compatibility of a "
            "system of linear Diophantine equations are considered.")
    rake = N.Rake().extract(text, 3)
    assert rake[0][0] == "linear diophantine equations" and rake[0][1] == pytest.approx(8.5)
    tr = [w for w, _ in N.TextRank().extract(text, 5)]
    assert "linear" in tr and "compatibility" in tr
    kw = [w for w, _ in N.keyword_tfidf(TECH[0], SPORT + TECH[1:], 3)]
    assert "faster" in kw or "new" in kw


def test_lda_recovers_two_planted_topics():
    docs = ["goal match team striker goal team"] * 6 + ["gpu kernel memory tensor gpu kernel"] * 6
    model, ids = N.fit_lda_from_text(docs, topics=2, iters=60, seed=1)
    dt = model.doc_topic_dist()
    first, second = int(dt[0].argmax()), int(dt[6].argmax())
    assert first != second and float(dt[:6, first].min()) > 0.8 and float(dt[6:, second].min()) > 0.8
    assert set(model.top_words(first, 4)) == {"goal", "match", "team", "striker"}
    assert model.perplexity(ids) < 5.0 and N.coherence_umass(model, ids, first, 3) > -0.5
    assert torch.allclose(model.topic_term_dist().sum(1), torch.ones(2, dtype=torch.float64))


def test_rule_based_entities_and_bio_tags():
    gaz = N.Gazetteer()
    gaz.add_many(["New York", "Paris"], "LOC")
    gaz.add("New York Times", "ORG")
    ner = N.RuleBasedNer(gaz)
    text = "The New York Times wrote on 2024-05-17 that rents in Paris rose 4.5% to $1,200; mail ed@nyt.com"
    ents = ner.extract(text)
    assert [(s, t) for s, t, _, _ in ents] == [("New York Times", "ORG"), ("2024-05-17", "DATE"), ("Paris", "LOC"), ("4.5%", "PERCENT"),
                                               ("$1,200", "MONEY"), ("ed@nyt.com", "EMAIL")]
    assert all(text[s:e] == surface for surface, _, s, e in ents)
    tags = dict(ner.bio_tags("She moved to New York"))
    assert tags["New"] == "B-LOC" and tags["York"] == "I-LOC" and tags["She"] == "O"
    ner.add_pattern("VERSION", r"\bv\d+\.\d+\b")
    assert ("v2.1", "VERSION") in [(s, t) for s, t, _, _ in ner.extract("upgrade to v2.1 now")]


def test_bloom_filter_trie_and_huffman_code():
    bf = N.BloomFilter(1000, 0.01)
    for i in range(1000):
        bf.insert(f"item{i}")
    assert all(f"item{i}" in bf for i in range(1000))                          # never a false negative
    fp = sum(f"other{i}" in bf for i in range(5000)) / 5000
    assert fp < 0.03 and abs(bf.estimated_fpr() - 0.01) < 0.01
    other = N.BloomFilter(1000, 0.01)
    other.insert("zzz")
    bf.merge(other)
    assert "zzz" in bf
    with pytest.raises(ValueError):
        bf.merge(N.BloomFilter(10, 0.1))
    t = N.Trie()
    for w in ("car", "card", "care", "cat", "dog", "car"):
        t.insert(w)
    assert len(t) == 5 and "car" in t and "ca" not in t and t.with_prefix("car") == ["car", "card", "care"]
    assert t.longest_prefix("cards are here") == "card" and t.longest_prefix("xyz") == "" and t.node_count() == 10
    data = b"abracadabra alakazam " * 20
    book = N.HuffmanCodebook.from_data(data)
    packed, bits = book.encode(data)
    assert book.decode(packed, bits) == data and len(packed) < 0.5 * len(data)
    assert book.lengths[ord("a")] == min(book.lengths.values())                 # the most frequent symbol has the shortest code
    assert sum(2.0 ** -l for l in book.lengths.values()) == pytest.approx(1.0)  # Kraft equality: the code is complete
    rebuilt = N.HuffmanCodebook(book.lengths)
    assert rebuilt.codes == book.codes and N.HuffmanCodebook.from_data(b"aaaa").encode(b"aaaa")[1] == 4

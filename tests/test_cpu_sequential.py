"""Hidden Markov models, linear-chain CRFs, labelling helpers, alignment and matching (CPU)."""
import itertools
import math

import pytest
import torch

from scirust_b200 import sequential as Q


def _hmm():
    return Q.Hmm([0.6, 0.4], [[0.7, 0.3], [0.4, 0.6]], [[0.5, 0.4, 0.1], [0.1, 0.3, 0.6]])


def test_hmm_recursions_agree_with_brute_force_enumeration():
    h = _hmm()
    obs = [0, 1, 2, 2, 0]
    pi, a, b = h.log_pi.exp(), h.log_a.exp(), h.log_b.exp()
    total, best = 0.0, (None, -1.0)
    for path in itertools.product(range(2), repeat=5):
        p = float(pi[path[0]] * b[path[0], obs[0]])
        for t in range(1, 5):
            p *= float(a[path[t - 1], path[t]] * b[path[t], obs[t]])
        total += p
        best = max(best, (list(path), p), key=lambda x: x[1])
    assert float(h.log_probability(obs)) == pytest.approx(math.log(total), abs=1e-12)
    path, lp = h.viterbi(obs)
    assert path == best[0] and lp == pytest.approx(math.log(best[1]), abs=1e-12)
    la, lb = h.forward(obs), h.backward(obs)
    for t in range(5):                                                         # alpha_t . beta_t is the likelihood at every t
        assert float(torch.logsumexp(la[0, t] + lb[0, t], 0)) == pytest.approx(math.log(total), abs=1e-12)
    batch = torch.tensor([obs, [2, 2, 2, 1, 0]])
    assert torch.allclose(h.log_probability(batch), torch.stack([h.log_probability(obs), h.log_probability(batch[1])]))
    with pytest.raises(ValueError):
        Q.Hmm([0.5, 0.6], [[0.7, 0.3], [0.4, 0.6]], [[1.0], [1.0]])


def test_baum_welch_increases_the_likelihood_and_recovers_the_emissions():
    truth = Q.Hmm([0.5, 0.5], [[0.9, 0.1], [0.1, 0.9]], [[0.8, 0.15, 0.05], [0.05, 0.15, 0.8]])
    seqs = torch.tensor([truth.sample(60, seed=s)[1] for s in range(40)])
    model = Q.Hmm([0.6, 0.4], [[0.6, 0.4], [0.3, 0.7]], [[0.5, 0.3, 0.2], [0.2, 0.3, 0.5]])
    hist = model.baum_welch(seqs, iters=60)
    assert all(b >= a - 1e-7 for a, b in zip(hist, hist[1:])) and hist[-1] > hist[0] + 50
    em = model.log_b.exp()
    assert float((em - truth.log_b.exp()).abs().max()) < 0.08 and float(model.log_a.exp()[0, 0]) > 0.8
    assert hist[-1] >= float(truth.log_probability(seqs).sum()) - 1e-6              # the fit is at least as likely as the truth
    states, obs = truth.sample(200, seed=99)
    acc = sum(int(a == b) for a, b in zip(model.viterbi(obs)[0], states)) / 200
    assert acc > 0.85


def test_crf_partition_marginals_and_training():
    torch.manual_seed(0)
    crf = Q.LinearChainCrf(3, 2)
    with torch.no_grad():
        for p in crf.parameters():
            p.copy_(torch.randn_like(p))
    feats = torch.randn(4, 3, dtype=torch.float64)
    scores = torch.stack([crf.score(feats, list(y))[0] for y in itertools.product(range(2), repeat=4)])
    assert float(crf.log_partition(feats)[0]) == pytest.approx(float(torch.logsumexp(scores, 0)), abs=1e-12)
    best = max(itertools.product(range(2), repeat=4), key=lambda y: float(crf.score(feats, list(y))[0]))
    assert crf.decode(feats) == list(best)
    marg = crf.marginals(feats)[0]
    probs = torch.softmax(scores, 0)
    for t in range(4):
        want = sum(float(p) for p, y in zip(probs, itertools.product(range(2), repeat=4)) if y[t] == 1)
        assert float(marg[t, 1]) == pytest.approx(want, abs=1e-10)
    # sticky labels seen through noisy features: the transitions must carry part of the evidence
    g = torch.Generator().manual_seed(1)

    def draw(n, t):
        stay = torch.rand(n, t, generator=g) < 0.9
        lab = torch.zeros(n, t, dtype=torch.long)
        lab[:, 0] = (torch.rand(n, generator=g) < 0.5).long()
        for k in range(1, t):
            lab[:, k] = torch.where(stay[:, k], lab[:, k - 1], 1 - lab[:, k - 1])
        x = torch.nn.functional.one_hot(lab, 2).double() + 0.9 * torch.randn(n, t, 2, generator=g, dtype=torch.float64)
        return x, lab
    x, labels = draw(64, 20)
    model = Q.LinearChainCrf(2, 2)
    hist = model.fit(x, labels, steps=150, lr=0.1, l2=1e-4)
    assert hist[-1] < 0.6 * hist[0]
    tr = model.trans.detach()
    assert float(tr[0, 0] + tr[1, 1] - tr[0, 1] - tr[1, 0]) > 2.0                # staying is rewarded
    xt, lt = draw(40, 20)
    chain = sum(sum(int(a == b) for a, b in zip(model.decode(xt[i]), lt[i].tolist())) for i in range(40)) / 800
    pointwise = float(((xt @ model.w.detach()).argmax(2) == lt).double().mean())
    assert chain > pointwise + 0.04 and chain > 0.85


def test_bio_spans_alignment_and_matching():
    tags = ["O", "B-PER", "I-PER", "O", "B-LOC", "B-LOC", "I-ORG", "O"]
    assert Q.extract_spans(tags) == [("PER", 1, 3), ("LOC", 4, 5), ("LOC", 5, 6), ("ORG", 6, 7)]
    assert Q.validate_bio(tags) == [6] and Q.validate_bio(["I-X"]) == [0] and Q.validate_bio(["B-X", "I-X", "O"]) == []
    score, a, b = Q.needleman_wunsch("GATTACA", "GCATGCU")
    assert score == 0.0 and len(a) == len(b) and [c for c in a if c] == list("GATTACA") and [c for c in b if c] == list("GCATGCU")
    assert Q.edit_distance("kitten", "sitting") == 3 and Q.edit_distance([], [1, 2]) == 2
    assert "".join(Q.longest_common_subsequence("AGGTAB", "GXTXAYB")) == "GTAB"
    assert Q.dynamic_time_warping([1, 2, 3], [1, 2, 2, 3]) == 0.0
    cost, path = Q.dynamic_time_warping([0, 1, 2], [0, 2], with_path=True)
    assert cost == 1.0 and path[0] == (0, 0) and path[-1] == (2, 1)
    text = "abracadabra abracadabra"
    for fn in (Q.kmp, Q.boyer_moore):
        assert fn(text, "abra") == [0, 7, 12, 19] and fn("aaaa", "aa") == [0, 1, 2] and fn(text, "xyz") == [] and fn("ab", "") == [0, 1, 2]

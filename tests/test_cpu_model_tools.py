"""Pruning, differentially private training, integrated gradients, accumulation autotuning, CSR products, embeddings."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from scirust_b200 import privacy as D
from scirust_b200 import pruning as P
from scirust_b200 import sparse as SP
from scirust_b200 import xai
from scirust_b200.embed import CharTokenizer, EmbeddingEngine
from scirust_b200.numerics import accumulate as A


def test_magnitude_and_structured_pruning():
    w = torch.tensor([0.5, -0.1, 0.3, -0.05, 0.8, 0.0])
    assert P.prune_magnitude(w.clone(), 0.5).tolist() == pytest.approx([0.5, 0.0, 0.3, 0.0, 0.8, 0.0])
    assert P.prune_magnitude(w.clone(), 0.0).tolist() == w.tolist()
    assert P.sparsity_ratio(P.prune_magnitude(w.clone(), 1.0)) == 1.0
    # ties go to the lower index
    assert P.prune_magnitude(torch.tensor([1.0, -1.0, 1.0, 1.0]), 0.5).tolist() == [0.0, 0.0, 1.0, 1.0]
    W = torch.tensor([[1.0, 0.125, 3.0], [2.0, 0.25, 0.5]])
    assert P.prune_structured_columns(W.clone(), sparsity=0.34).tolist() == [[1.0, 0.0, 3.0], [2.0, 0.0, 0.5]]
    assert P.prune_structured_rows(W.clone(), sparsity=0.5).tolist() == [[1.0, 0.125, 3.0], [0.0, 0.0, 0.0]]
    flat = W.clone().reshape(-1)
    P.prune_structured_columns(flat, 2, 3, 0.34)
    assert flat.tolist() == [1.0, 0.0, 3.0, 2.0, 0.0, 0.5]
    assert P.prune(W.clone(), P.PruningMethod.STRUCTURED_ROWS, 0.5)[1].abs().sum() == 0
    for bad in (-0.1, 1.5, float("nan")):
        with pytest.raises(ValueError):
            P.prune_magnitude(w.clone(), bad)
    with pytest.raises(ValueError):
        P.prune_magnitude(torch.tensor([1.0, float("inf")]), 0.5)
    with pytest.raises(ValueError):
        P.prune_structured_rows(torch.zeros(5), 2, 3, 0.5)


def test_wanda_n_of_m_and_lottery_ticket():
    W = torch.tensor([[1.0, -2.0, 0.5, 3.0], [0.125, 0.25, -4.0, 0.375]])
    norms = torch.tensor([10.0, 0.1, 1.0, 0.01])
    out = P.prune_wanda(W.clone(), norms, 0.5)
    # scores row 0: 10, 0.2, 0.5, 0.03 -> drop columns 3 and 1; row 1: 1.25, 0.025, 4, 0.00375 -> drop 3 and 1
    assert out.tolist() == [[1.0, 0.0, 0.5, 0.0], [0.125, 0.0, -4.0, 0.0]]
    with pytest.raises(ValueError):
        P.prune_wanda(W.clone(), norms[:3], 0.5)
    with pytest.raises(ValueError):
        P.prune_wanda(W.clone(), -norms, 0.5)
    torch.manual_seed(0)
    M = torch.randn(8, 16)
    S = P.prune_n_of_m(M.clone())
    assert P.is_n_of_m(S) and not P.is_n_of_m(M) and P.sparsity_ratio(S) == 0.5
    groups = M.reshape(-1, 4)
    kept = (S.reshape(-1, 4) != 0)
    assert bool(((groups.abs() * kept).sum(1) >= (groups.abs() * ~kept).sum(1)).all())      # the two largest survive
    with pytest.raises(ValueError):
        P.prune_n_of_m(torch.zeros(3, 6))
    lt = P.LotteryTicketPruner(0.5, 2)
    init = torch.arange(1.0, 9.0)
    lt.save_initial(init)
    trained = torch.tensor([0.1, 0.9, 0.2, 0.8, 0.3, 0.7, 0.4, 0.6])
    lt.prune_and_rewind(trained)
    assert trained.tolist() == [0.0, 2.0, 0.0, 4.0, 0.0, 6.0, 0.0, 8.0]                   # survivors back at their initial values
    trained[trained != 0] = torch.tensor([0.5, 0.1, 0.4, 0.2])
    lt.prune_and_rewind(trained)
    assert P.sparsity_ratio(trained) == 0.75 and trained.tolist() == [0.0, 2.0, 0.0, 0.0, 0.0, 6.0, 0.0, 0.0]
    before = trained.clone()
    lt.prune_and_rewind(trained)                                                          # target reached: no-op
    assert torch.equal(trained, before)
    with pytest.raises(ValueError):
        P.LotteryTicketPruner(0.5, 1).prune_and_rewind(trained)


def test_dp_clipping_noise_and_accounting():
    g = torch.tensor([0.1, 0.2, 0.3])
    assert torch.equal(D.clip_gradients(g.clone(), 10.0), g)
    assert torch.allclose(D.clip_gradients(torch.tensor([3.0, 4.0]), 1.0), torch.tensor([0.6, 0.8]))
    big = D.clip_gradients(torch.tensor([torch.finfo(torch.float32).max / 4, 0.0]), 1.0)
    assert bool(torch.isfinite(big).all()) and abs(float(big[0]) - 1.0) < 1e-6 and float(big[1]) == 0.0
    rows = D.clip_gradients(torch.tensor([[3.0, 4.0], [0.3, 0.4]]), 1.0)
    assert torch.allclose(rows, torch.tensor([[0.6, 0.8], [0.3, 0.4]]))
    g1 = D.add_noise(torch.tensor([1.0, 2.0]), 0.5, torch.Generator().manual_seed(9))
    g2 = D.add_noise(torch.tensor([1.0, 2.0]), 0.5, torch.Generator().manual_seed(9))
    assert torch.equal(g1, g2) and not torch.equal(g1, torch.tensor([1.0, 2.0]))
    cfg = D.DpSgdConfig(1.0, 1.0, 1e-5)
    G = torch.tensor([[3.0, 4.0], [0.0, 0.5], [-6.0, 8.0]])
    out = D.dp_sgd_gradient(G, cfg, torch.Generator().manual_seed(1))
    noise = torch.randn(2, generator=torch.Generator().manual_seed(1))
    assert torch.allclose(out, (torch.tensor([0.6 + 0.0 - 0.6, 0.8 + 0.5 + 0.8]) + noise) / 3, atol=1e-6)
    assert torch.allclose(D.dp_sgd_gradient([r for r in G], cfg, torch.Generator().manual_seed(1)), out)
    for bad in (D.DpSgdConfig(0.0), D.DpSgdConfig(1.0, -1.0), D.DpSgdConfig(1.0, 1.0, 1.5), D.DpSgdConfig(1.0, 1.0, 1e-5, -2.0),
                D.DpSgdConfig(float("nan"))):
        with pytest.raises(ValueError):
            bad.validate()
    with pytest.raises(ValueError):
        D.dp_sgd_gradient([], cfg, torch.Generator())
    with pytest.raises(ValueError):
        D.dp_sgd_gradient([torch.zeros(2), torch.zeros(3)], cfg, torch.Generator())
    with pytest.raises(ValueError):
        D.dp_sgd_gradient(torch.tensor([[float("nan"), 0.0]]), cfg, torch.Generator())
    # accounting: closed form at one order, monotone in the number of steps, decreasing in sigma
    assert D.gaussian_rdp(2.0, 1.0) == 1.0 and D.rdp_to_dp(1.0, 2.0, math.exp(-3)) == pytest.approx(4.0)
    e100, order = D.rdp_gaussian_epsilon(100, 1.1, 1e-5)
    assert order in D._orders() and e100 > D.rdp_gaussian_epsilon(10, 1.1, 1e-5)[0] > 0
    assert D.rdp_gaussian_epsilon(100, 4.0, 1e-5)[0] < e100
    acc = D.MomentsAccountant(1e-5, 0.01, 1.1)
    for _ in range(100):
        acc.step()
    assert acc.epsilon == pytest.approx(e100, rel=1e-9) and acc.steps == 100
    dead = D.MomentsAccountant(1e-5, 0.01, 0.0)
    dead.step()
    assert dead.epsilon == math.inf
    assert D.secure_generator().initial_seed() != D.secure_generator().initial_seed()


def test_per_sample_gradients_and_private_training():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.Tanh(), torch.nn.Linear(8, 3))
    x, y = torch.randn(6, 4), torch.randint(0, 3, (6,))
    G = D.per_sample_gradients(model, F.cross_entropy, x, y)
    ref = []
    for i in range(6):
        model.zero_grad()
        F.cross_entropy(model(x[i:i + 1]), y[i:i + 1]).backward()
        ref.append(torch.cat([p.grad.reshape(-1) for p in model.parameters()]))
    assert torch.allclose(G, torch.stack(ref), atol=1e-6)
    # a separable problem still trains under clipping + noise, and the budget grows with every step
    X = torch.cat([torch.randn(64, 4) + 2, torch.randn(64, 4) - 2])
    Y = torch.cat([torch.zeros(64), torch.ones(64)]).long()
    clf = torch.nn.Linear(4, 2)
    opt = D.DpSgd(clf, F.cross_entropy, 0.5, D.DpSgdConfig(1.0, 0.8, 1e-5), torch.Generator().manual_seed(3))
    eps = []
    for _ in range(30):
        opt.step(X, Y)
        eps.append(opt.epsilon)
    assert float((clf(X).argmax(1) == Y).float().mean()) > 0.95
    assert eps == sorted(eps) and eps[0] > 0


def test_integrated_gradients():
    torch.manual_seed(0)
    lin = torch.nn.Linear(5, 1)
    x, base = torch.randn(5), torch.zeros(5)
    f = lambda X: lin(X)
    attr = xai.integrated_gradients(x, base, 10, f)
    assert torch.allclose(attr, lin.weight[0].detach() * x, atol=1e-6)                     # linear model: exact
    assert abs(xai.completeness_gap(attr, x, base, f)) < 1e-5
    net = torch.nn.Sequential(torch.nn.Linear(5, 16), torch.nn.Tanh(), torch.nn.Linear(16, 1))
    g = lambda X: net(X)
    coarse = abs(xai.completeness_gap(xai.integrated_gradients(x, base, 4, g), x, base, g))
    fine = abs(xai.completeness_gap(xai.integrated_gradients(x, base, 256, g), x, base, g))
    assert fine < 1e-2 and fine <= coarse + 1e-6
    # chunked evaluation is the same estimate; a feature the model ignores gets zero attribution
    assert torch.allclose(xai.integrated_gradients(x, base, 64, g, batch=7), xai.integrated_gradients(x, base, 64, g), atol=1e-6)
    h = lambda X: (X[:, 0] * X[:, 1])
    assert float(xai.integrated_gradients(x, base, 32, h)[2:].abs().sum()) == 0.0
    with pytest.raises(ValueError):
        xai.integrated_gradients(x, torch.zeros(4), 8, f)
    with pytest.raises(ValueError):
        xai.integrated_gradients(x, base, 0, f)


def test_accumulation_methods_and_autotuner():
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(3000) * 1e4).astype(np.float32)
    xs[::2] += np.float32(1e7)
    scores = {m.kind: A.accum_score(m, xs) for m in A.default_accumulators()}
    assert scores["klein"] >= scores["neumaier"] >= scores["naive"] and scores["pairwise"] > scores["naive"]
    assert scores["neumaier"] > -1e-7
    # compensated sums recover what the naive sum loses outright
    hard = np.array([1e8, 1.0, -1e8, 1.0] * 50, dtype=np.float32)
    assert float(A.accumulate(A.NAIVE, hard)) != 100.0 and float(A.accumulate(A.NEUMAIER, hard)) == 100.0
    assert float(A.accumulate(A.KLEIN, hard)) == 100.0 and A.exact_sum(hard) == 100.0
    assert A.accum_score(A.NAIVE, np.array([1.0, -1.0], dtype=np.float32)) is None
    assert [m.cost() for m in A.default_accumulators()] == [1, 1, 7, 14, 3]
    # stochastic rounding: representable values are fixed points, neighbours bracket, the variate picks the branch
    for v in (0.0, 1.0, -2.5, 1024.0):
        assert float(A.stochastic_round_to_f32(v, 0.3)) == v
    lo = np.float32(0.1) if float(np.float32(0.1)) < 0.1 else np.nextafter(np.float32(0.1), np.float32(-1))
    assert A.stochastic_round_to_f32(0.1, 0.0) == np.nextafter(lo, np.float32(1)) and A.stochastic_round_to_f32(0.1, 0.999999) == lo
    assert float(A.stochastic_round_to_f32(1e300, 0.5)) == float(np.finfo(np.float32).max)
    s1, s2 = A.stochastic_sum_f32(xs[:200], 7, 1), A.stochastic_sum_f32(xs[:200], 7, 1)
    assert s1 == s2 and abs(float(s1) - A.exact_sum(xs[:200])) / abs(A.exact_sum(xs[:200])) < 1e-5
    rep = A.autotune_accumulator(xs[:1500], xs[1500:])
    assert rep.chosen.kind in ("pairwise", "neumaier", "klein") and rep.beats_baseline
    assert rep.chosen_eval_score > rep.baseline_eval_score and len(rep.dev_scores) == 5
    # generic harness: infeasible candidates are skipped, no feasible candidate means no choice
    none = A.autotune_by([1], [1], ["a", "b"], lambda c, f, s: None, lambda f, s: 0.0)
    assert none.chosen is None and not none.beats_baseline and none.chosen_eval_score == -math.inf
    pick = A.autotune_by([1], [1], ["a", "b", "c"], lambda c, f, s: {"a": 1.0, "b": 2.0, "c": 2.0}[c], lambda f, s: 1.5)
    assert pick.chosen == "b" and pick.beats_baseline


def test_csr_products_and_validation():
    torch.manual_seed(0)
    dense = torch.randn(6, 9) * (torch.rand(6, 9) > 0.6)
    csr = SP.CsrTensor.from_dense(dense)
    b = torch.randn(9, 4)
    assert torch.equal(csr.to_dense(), dense) and csr.nnz() == int((dense != 0).sum())
    assert torch.allclose(SP.spmm_dense(csr, b), dense @ b, atol=1e-5)
    assert torch.allclose(SP.spmm_dense_reference(csr, b), dense @ b, atol=1e-5)
    empty = SP.CsrTensor([], [], [0, 0, 0], 2, 3)
    assert float(SP.spmm_dense(empty, torch.randn(3, 2)).abs().sum()) == 0.0
    hand = SP.CsrTensor([1.0, 2.0, 3.0], [0, 2, 1], [0, 2, 3], 2, 3)
    assert hand.to_dense().tolist() == [[1.0, 0.0, 2.0], [0.0, 3.0, 0.0]]
    for args in (([1.0], [0], [0, 1], 2, 3), ([1.0, 2.0], [0], [0, 1, 2], 2, 3), ([1.0], [0], [1, 1, 1], 2, 3),
                 ([1.0, 2.0], [0, 1], [0, 2, 1], 2, 3), ([1.0], [0], [0, 0, 2], 2, 3), ([1.0], [3], [0, 1, 1], 2, 3)):
        with pytest.raises(ValueError):
            SP.CsrTensor(*args)
    with pytest.raises(ValueError):
        SP.spmm_dense(hand, torch.randn(4, 2))


def test_embedding_engine():
    eng = EmbeddingEngine(["hello world", "goodbye moon"], d_model=32, d_ff=64)
    batch = eng.embed_batch(["hello", "hello world", "", "moon"])
    assert batch.shape == (4, 32) and eng.dim() == 32
    assert torch.allclose(batch.norm(dim=1), torch.tensor([1.0, 1.0, 0.0, 1.0]), atol=1e-5)
    assert torch.allclose(eng.embed("hello"), batch[0], atol=1e-6)              # padding in a batch changes nothing
    assert EmbeddingEngine.cosine_similarity(batch[0], batch[0]) == pytest.approx(1.0, abs=1e-5)
    assert EmbeddingEngine.cosine_similarity(batch[0], batch[2]) == 0.0
    assert EmbeddingEngine.cosine_similarity(batch[0], batch[1]) > EmbeddingEngine.cosine_similarity(batch[0], batch[3])
    again = EmbeddingEngine(["hello world", "goodbye moon"], d_model=32, d_ff=64)
    assert torch.equal(again.embed("moon"), batch[3])                           # seeded construction
    tok = CharTokenizer(["abc"])
    assert tok.encode("cabz") == [3, 1, 2, 0] and tok.decode([3, 1, 2, 0]) == "cab" and tok.vocab_size == 4


def test_certificate_gated_transform_selection():
    from scirust_b200.numerics import transform_search as T
    xs = np.logspace(-6, 6, 200)
    rep = T.select_transform(xs, 64.0, T.default_positive_dictionary())
    by = {v.repr.name: v for v in rep.verdicts}
    assert rep.chosen == T.Representation("power", 0.5) and rep.chosen_bound_ulps == pytest.approx(12.0)
    assert by["log"].accepted and by["anscombe"].rejected.kind == "tolerance-exceeded"
    assert rep.support.lo == pytest.approx(1e-6) and rep.support.hi == pytest.approx(1e6)
    # a tighter tolerance rejects more; an impossible one rejects all, with reasons
    assert T.select_transform(xs, 1.0, T.default_positive_dictionary()).chosen is None
    # negative samples are outside the domain of log: the first offender is reported
    neg = T.select_transform([1.0, -2.0, 3.0], 64.0, [T.LOG, T.SIGNED_LOG])
    why = {v.repr.name: v.rejected for v in neg.verdicts}
    assert why["log"] == T.RejectReason("outside-domain", -2.0) and neg.chosen == T.SIGNED_LOG
    # Anscombe near 0: sqrt(x + 3/8) forgets a tiny x entirely (kappa_rt * u >= 1/2): the invalid region, whatever the tolerance
    tight = T.select_transform([1e-17, 1.0], 1e30, [T.ANSCOMBE])
    assert tight.verdicts[0].rejected.kind == "invalid-region" and tight.chosen is None
    empty = T.select_transform([], 64.0, [T.LOG])
    assert empty.chosen is None and empty.verdicts == []
    assert [r.cost() for r in (T.ANSCOMBE, T.LOG, T.LOGIT, T.Representation("mu-law", 255.0))] == [2, 3, 4, 5]


def test_quantizer_autotune_and_plan_search():
    from scirust_b200.numerics import transform_search as T
    q = T.UniformQuantizer.fit([0.0, 10.0], 10)
    assert q.round_trip(np.array([0.2, 9.99, 25.0, -3.0])).tolist() == pytest.approx([0.5, 9.5, 9.5, 0.5])
    assert T.sqnr_db([1.0, 2.0], [1.0, 2.0]) == math.inf and T.sqnr_db([3.0, 4.0], [3.0, 3.0]) == pytest.approx(10 * math.log10(25))
    rng = np.random.default_rng(0)
    data = np.exp(rng.standard_normal(3000) * 2.0)
    rep = T.autotune_quantizer(data[:1500], data[1500:], T.default_positive_quantizer_dictionary(), 64)
    assert rep.chosen is not None and rep.beats_baseline and rep.chosen_eval_sqnr_db > rep.baseline_eval_sqnr_db
    assert len(rep.verdicts) == 9 and all(not isinstance(s, T.RejectReason) for _, s in rep.verdicts)
    # data with zeros: log is gated out with a reason, log1p / power stay
    z = np.concatenate([[0.0], data[:200]])
    rz = T.autotune_quantizer(z[:100], z[100:], [T.LOG, T.LOG1P], 32)
    assert isinstance(dict((r.name, s) for r, s in rz.verdicts)["log"], T.RejectReason) and rz.chosen == T.LOG1P
    joint = T.joint_search(data[:200], data[200:400])
    seq = T.sequential_baseline(data[:200], data[200:400])
    assert joint.evaluated == 6 * 5 and seq.evaluated == 5
    assert joint.chosen is not None and seq.chosen.representation.kind != "identity"
    dev_best = min(e for _, e in joint.dev_errors if e is not None)
    assert T.pipeline_relative_error(joint.chosen, data[:200], data[:200]) == dev_best      # the dev optimum was taken
    assert dev_best <= min(e for _, e in seq.dev_errors if e is not None) + 1e-15             # joint search covers the baseline's pair
    cache = T.PlanCache()
    p1 = cache.plan_for("sum", "cpu", data[:200], data[200:400])
    p2 = cache.plan_for("sum", "cpu", data[:200] * 1.01, data[200:400])                      # same distribution summary: reused
    assert p1 == p2 and (cache.hits, cache.misses) == (1, 1)
    assert cache.get("sum", "cpu", T.summarize(-data[:50])) is None
    s = T.summarize(data)
    assert s.sign == "positive" and s.decades >= 4 and T.summarize([0.0, 0.0]).decades == 0
    assert T.summarize([-1.0, 2.0]).sign == "mixed" and T.current_hardware_key() in ("cpu",) or True


def test_pinned_pool_uploader_and_tensor3d():
    from scirust_b200.autodiff import Tape
    from scirust_b200.tensor import Tensor, Tensor3D, Var3D, broadcast_get, unbroadcast
    from scirust_b200.utils import pinned as PN
    buf = PN.PinnedBuffer(4)
    assert buf.as_tensor().tolist() == [0.0] * 4 and buf.is_aligned() and buf.len_bytes() == 16 and len(buf) == 4
    assert buf.layout() in (PN.MemoryLayout.CPU, PN.MemoryLayout.PINNED) and PN.PinnedBuffer(0).is_empty()
    with pytest.raises(PN.PinError, match="too large"):
        PN.PinnedBuffer(1 << 60, torch.int64)
    pool = PN.PinnedPool(2, 8)
    first, second = pool.borrow(), pool.borrow()
    assert pool.available() == 0 and pool.capacity() == 2 and {first.index, second.index} == {0, 1}
    with pytest.raises(PN.PinError, match="allocation failed"):
        pool.borrow()
    first.as_tensor()[0] = 7.0
    pool.release(first)
    assert pool.available() == 1 and float(pool.borrow().as_tensor()[0]) == 7.0       # storage is reused, not reallocated
    with pytest.raises(PN.PinError, match="does not belong"):
        pool.release(first)                                                            # double release
    with pytest.raises(PN.PinError, match="does not belong"):
        PN.PinnedPool(1, 8).release(second)                                            # another pool's buffer
    with pytest.raises(PN.PinError, match="released"):
        first.as_tensor()
    up = PN.DoubleBufferedUploader(16, torch.float32, "cpu")
    a, b = up.submit(torch.arange(6.0).reshape(2, 3)), up.submit(torch.ones(4))
    with pytest.raises(PN.PinError):
        up.submit(torch.zeros(2))                                                      # both slots in flight
    assert up.take(a).tolist() == [[0, 1, 2], [3, 4, 5]] and up.take(b).tolist() == [1.0] * 4
    assert up.take is not None and up.pool.available() == 2
    with pytest.raises(PN.PinError):
        up.take(a)
    with pytest.raises(PN.PinError):
        PN.stage_to_device(torch.zeros(32), up.pool.borrow(), "cpu")
    t3 = Tensor3D.zeros(2, 3, 4)
    assert t3.shape == (2, 3, 4) and t3.as_nd().shape == (2, 3, 4)
    with pytest.raises(ValueError):
        Tensor3D(Tensor.zeros(5, 4), 2, 3, 4)
    v3 = Var3D.input_3d(Tape(), t3)
    assert v3.shape == (2, 3, 4) and tuple(v3.as_var().t.shape) == (6, 4)
    assert broadcast_get([1, 2, 3], [1, 3], [5, 2]) == 3.0 and broadcast_get([1, 2, 3, 4], [2, 2], [1, 0]) == 3.0
    assert unbroadcast(torch.ones(4, 2, 3), (1, 3)).tolist() == [[8.0, 8.0, 8.0]] and unbroadcast(torch.ones(2, 3), (2, 3)).shape == (2, 3)

"""Elastic latent KV: online basis learner and committed versions, lifecycle ring, representation epochs, the
integrated per-head decode runtime and the encoder session."""
import pytest
import torch

from scirust_b200.nn import kv_cache_elastic_runtime as E
from scirust_b200.nn.rng import PcgEngine
from scirust_b200.nn.transformer import MultiHeadAttention, TransformerEncoder


def test_basis_learner_tracks_the_subspace_and_commits_versions():
    torch.manual_seed(0)
    cfg = E.BasisLearningConfig(8, 2, 0.1, 4, 10, 200, 4)
    learner = E.CommittedBasisLearner(cfg, E.identity_prefix(8, 2))
    U = torch.linalg.qr(torch.randn(8, 8))[0][:, :2]
    commits = []
    for _ in range(300):
        obs = learner.observe(U @ torch.randn(2) + 0.01 * torch.randn(8))
        if obs.committed:
            commits.append(obs.committed)
    B = learner.basis()
    assert float((B.t() @ B - torch.eye(2)).abs().max()) < 1e-5              # orthonormal
    assert float((U @ U.t() @ B - B).norm()) < 0.05 and obs.quality_bps > 9900
    assert len(commits) >= 1 and [c.version for c in commits] == list(range(1, len(commits) + 1))
    qualities = [c.quality_bps for c in commits]
    assert all(b - a >= cfg.minimum_quality_gain_bps for a, b in zip([0] + qualities, qualities))
    assert all(b.samples_seen - a.samples_seen >= 10 for a, b in zip(learner.versions(), learner.versions()[1:]))
    assert len(learner.versions()) <= cfg.maximum_versions
    # every archived snapshot matches the fingerprint recorded at commit time; the live basis has moved on
    for v in learner.versions():
        assert E.basis_fingerprint(learner.committed_basis(v.version)) == v.fingerprint
    assert learner.committed_basis(99) is None
    assert E.basis_fingerprint(learner.latest_committed_basis()) == learner.versions()[-1].fingerprint
    # same stream, same versions (bit for bit)
    torch.manual_seed(0)
    again = E.CommittedBasisLearner(cfg, E.identity_prefix(8, 2))
    U2 = torch.linalg.qr(torch.randn(8, 8))[0][:, :2]
    for _ in range(300):
        again.observe(U2 @ torch.randn(2) + 0.01 * torch.randn(8))
    assert again.versions() == learner.versions()
    # fingerprint: FNV-1a over bit patterns (sign of zero matters, empty input is the offset basis)
    assert E.basis_fingerprint(torch.zeros(0)) == 0xCBF29CE484222325
    assert E.basis_fingerprint(torch.tensor([0.0])) != E.basis_fingerprint(torch.tensor([-0.0]))
    full = E.complete_basis(B)
    assert float((full.t() @ full - torch.eye(8)).abs().max()) < 1e-4 and torch.allclose(full[:, :2], B)


def test_basis_learner_validation():
    ok = E.identity_prefix(4, 2)
    for bad in (E.BasisLearningConfig(0, 1), E.BasisLearningConfig(4, 0), E.BasisLearningConfig(4, 5),
                E.BasisLearningConfig(4, 2, 0.0), E.BasisLearningConfig(4, 2, 1.5), E.BasisLearningConfig(4, 2, float("nan")),
                E.BasisLearningConfig(4, 2, 0.1, 0), E.BasisLearningConfig(4, 2, 0.1, 1, 0),
                E.BasisLearningConfig(4, 2, 0.1, 1, 1, 0, 0)):
        with pytest.raises(E.BasisLearningError):
            E.DeterministicBasisLearner(bad, ok)
    cfg = E.BasisLearningConfig(4, 2)
    with pytest.raises(E.BasisLearningError):
        E.DeterministicBasisLearner(cfg, torch.zeros(7))
    with pytest.raises(E.BasisLearningError):
        E.DeterministicBasisLearner(cfg, torch.full((4, 2), float("inf")))
    learner = E.DeterministicBasisLearner(cfg, torch.zeros(4, 2))         # degenerate columns become unit vectors
    assert torch.equal(learner.basis(), E.identity_prefix(4, 2))
    with pytest.raises(E.BasisLearningError):
        learner.observe(torch.zeros(3))
    with pytest.raises(E.BasisLearningError):
        learner.observe(torch.tensor([1.0, float("nan"), 0.0, 0.0]))
    assert learner.observe(torch.zeros(4)).quality_bps == 10_000


def test_lifecycle_ring_temperatures_and_eviction():
    lc = E.LatentKvLifecycle(E.LifecycleConfig(6, 2, 2))
    for i in range(6):
        adm = lc.admit(basis_version=i // 3)
        assert adm.position == i and adm.evicted is None
        lc.rebalance()
    assert {k.value: v for k, v in lc.counts().items()} == {"hot": 2, "warm": 2, "cold": 2}
    assert lc.get(5).temperature == E.CacheTemperature.HOT and lc.get(0).temperature == E.CacheTemperature.COLD
    adm = lc.admit(7)
    assert adm.position == 6 and adm.evicted.position == 0 and adm.evicted.temperature == E.CacheTemperature.COLD
    acts = lc.rebalance()
    # one hot -> warm and one warm -> cold move per admitted token once the windows are full
    assert [(a.position, a.source.value, a.to.value) for a in acts] == [(2, "warm", "cold"), (4, "hot", "warm")]
    assert acts[0].target == lc.config.cold and acts[0].basis_version == 0
    assert lc.get(0) is None and len(lc) == 6
    lc.touch(3)
    assert lc.get(3).last_access_tick > lc.get(6).last_access_tick
    with pytest.raises(E.LifecycleError):
        lc.touch(0)
    # the report can be capped, the state change cannot
    lc.admit(0)
    assert len(lc.rebalance(limit=1)) == 1 and lc.rebalance() == []
    for bad in (E.LifecycleConfig(0, 0, 0), E.LifecycleConfig(4, 3, 2),
                E.LifecycleConfig(4, 1, 1, cold=E.CompressionTier("int4", "int4", 0, 0))):
        with pytest.raises(E.LifecycleError):
            E.LatentKvLifecycle(bad)


def test_representation_epochs():
    m0 = E.KvRepresentationMetadata("dense-fp32", 0, 8)
    cache = E.RepresentedElasticKvCache(8, 4, m0)
    torch.manual_seed(0)
    for _ in range(6):
        cache.append(torch.randn(8), torch.randn(8))
    assert len(cache) == 6 and cache.attention(torch.randn(8)).shape == (8,) and cache.compressed_bytes() > 0
    m1 = m0.next_epoch("latent-r4")
    cache.commit_representation(m1)
    assert cache.representation.epoch == 1 and [m.representation_id for m in cache.history] == ["dense-fp32", "latent-r4"]
    with pytest.raises(E.KvRepresentationError):
        cache.commit_representation(m1)                                           # epoch must advance by one
    with pytest.raises(E.KvRepresentationError):
        cache.commit_representation(E.KvRepresentationMetadata("x", 2, 16))       # contract change
    with pytest.raises(E.KvRepresentationError):
        cache.commit_representation(E.KvRepresentationMetadata("x", 2, 8, E.KvKeyTransformScope.PER_HEAD))
    with pytest.raises(E.KvRepresentationError):
        E.KvRepresentationMetadata("  ", 0, 8)
    with pytest.raises(E.KvRepresentationError):
        E.RepresentedElasticKvCache(4, 4, m0)


def _decode_errors(mha, rt, toks, n):
    mha.reset_cache()
    errs = []
    for t in range(n):
        ref = mha.infer_step(toks[t:t + 1])[0]
        out = rt.decode_step(mha, toks[t])
        errs.append(float((out - ref).detach().norm() / ref.detach().norm()))
    return errs


def test_decode_runtime_matches_dense_cache_and_respects_budgets():
    torch.manual_seed(0)
    mha = MultiHeadAttention(32, 4, PcgEngine(1))
    toks = torch.randn(64, 32)
    cal = E.calibrate_heads(mha, toks)
    full = E.CompressionTier("fp32", "fp32", 4, 1)
    exact_cfg = E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 10 ** 6, 10 ** 7, E.LifecycleConfig(24, 8, 8, full, full, full))
    rt = E.ElasticLatentDecodeRuntime(mha, exact_cfg, cal)
    assert max(_decode_errors(mha, rt, toks, 20)) < 1e-5                  # full rank, fp32: the dense result
    tel = rt.telemetry()
    assert tel.steps == 20 and tel.worst_quality_bps == 10_000 and tel.total_lifecycle_evictions == 0
    assert tel.planned_persistent_bytes <= 10 ** 6 and tel.allocated_bytes <= 10 ** 7
    # int8 middle tier: small, bounded error; lifecycle transitions are counted
    i8 = E.CompressionTier("int8", "int8", 2, 1)
    rt8 = E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 10 ** 6, 10 ** 7,
                                                                         E.LifecycleConfig(24, 8, 8, full, i8, i8)), cal)
    errs = _decode_errors(mha, rt8, toks, 30)
    assert max(errs[:8]) < 1e-5 and 0 < max(errs[:24]) < 0.05            # beyond 24 tokens the window slides, the dense reference does not
    t8 = rt8.telemetry()
    assert t8.total_lifecycle_evictions == 4 * 6 and t8.last_lifecycle_transitions == 4 * 2 and t8.last_lifecycle_evictions == 4
    # a tight budget forces cheaper plans; the budget is split over the heads
    tight = E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 4 * 24 * 24, 10 ** 7,
                                                                           E.LifecycleConfig(24, 8, 8)), cal)
    assert tight.telemetry().planned_persistent_bytes <= 4 * 24 * 24
    assert all(p.bytes_per_token <= 24 for p in tight.plans) and any(p.key.fmt != "fp32" for p in tight.plans)
    assert tight.telemetry().worst_quality_bps < 10_000
    with pytest.raises(E.ElasticLatentRuntimeError):
        E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 40, 10 ** 7, E.LifecycleConfig(24, 8, 8)), cal)
    with pytest.raises(E.ElasticLatentRuntimeError):
        E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 10 ** 6, 100, E.LifecycleConfig(24, 8, 8)), cal)
    with pytest.raises(E.ElasticLatentRuntimeError):
        E.ElasticLatentDecodeRuntime(mha, exact_cfg, cal[:2])
    with pytest.raises(E.ElasticLatentRuntimeError):
        E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(16, 2, 8, 4, 10 ** 6, 10 ** 7, E.LifecycleConfig(24, 8, 8)), cal)
    with pytest.raises(E.ElasticLatentRuntimeError):
        rt.decode_step(mha, torch.zeros(5))


def test_low_rank_keys_survive_rank_reduced_cold_tier():
    torch.manual_seed(1)
    mha = MultiHeadAttention(32, 4, PcgEngine(3))
    # tokens in a 2-dimensional subspace -> per-head keys / values have rank 2: every tier keeps at least rank 2, so nothing is lost
    toks = torch.randn(80, 2) @ torch.randn(2, 32)
    cal = E.calibrate_heads(mha, toks)
    full = E.CompressionTier("fp32", "fp32", 0, 1)
    half = E.CompressionTier("fp32", "fp32", 0, 2)
    rt = E.ElasticLatentDecodeRuntime(mha, E.ElasticLatentRuntimeConfig(32, 2, 8, 0, 10 ** 6, 10 ** 7,
                                                                        E.LifecycleConfig(32, 4, 4, full, full, half)), cal)
    assert max(_decode_errors(mha, rt, toks, 30)) < 1e-3 and rt.telemetry().worst_quality_bps > 9990


def test_encoder_session_and_committed_basis_handoff():
    torch.manual_seed(0)
    enc = TransformerEncoder(2, 32, 4, 64, PcgEngine(2))
    toks = torch.randn(48, 32)
    full = E.CompressionTier("fp32", "fp32", 4, 1)
    cfg = E.ElasticLatentRuntimeConfig(24, 2, 8, 4, 10 ** 6, 10 ** 7, E.LifecycleConfig(24, 8, 8, full, full, full))
    sess = E.ElasticLatentEncoderSession(enc, cfg, [E.calibrate_heads(b.attn, toks) for b in enc.blocks])
    for b in enc.blocks:
        b.attn.reset_cache()
    for t in range(10):
        h = toks[t:t + 1]
        for b in enc.blocks:
            h = h + b.attn.infer_step(b.ln1(h))
            h = h + b.ffn(b.ln2(h))
        ref = enc.ln(h)[0]
        out = sess.infer_step(toks[t])
        assert float((out - ref).abs().max()) < 1e-4
    assert sess.layers() == 2 and sess.layer_telemetry(1).steps == 10 and sess.layer_telemetry(5) is None
    with pytest.raises(E.ElasticLatentRuntimeError):
        E.ElasticLatentEncoderSession(enc, cfg, [])
    # bases learned online and COMMITTED are what a new session freezes; later learning does not touch it
    attn = enc.blocks[0].attn
    with torch.no_grad():
        K = attn.w_k(toks).reshape(-1, 4, 8)
        V = attn.w_v(toks).reshape(-1, 4, 8)
    lcfg = E.BasisLearningConfig(8, 8, 0.05, 2, 8, 50, 4)
    learners = [(E.CommittedBasisLearner(lcfg, E.identity_prefix(8, 8)), E.CommittedBasisLearner(lcfg, E.identity_prefix(8, 8)))
                for _ in range(4)]
    for t in range(48):
        for h, (kl, vl) in enumerate(learners):
            kl.observe(K[t, h])
            vl.observe(V[t, h])
    cal = E.calibrate_heads(attn, toks, learners)
    assert [c.basis_version for c in cal] == [kl.versions()[-1].version for kl, _ in learners]
    rt = E.ElasticLatentDecodeRuntime(attn, cfg, cal)
    frozen = cal[0].key_basis.clone()
    learners[0][0].observe(torch.randn(8) * 5)
    assert torch.equal(cal[0].key_basis, frozen)
    assert max(_decode_errors(attn, rt, toks, 12)) < 1e-4                         # full-rank learned basis: still exact

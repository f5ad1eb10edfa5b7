"""Static-pipeline generator, additively homomorphic encryption, quaternion chart search (CPU)."""
import numpy as np
import pytest
import torch

from scirust_b200 import aot
from scirust_b200 import homomorphic as H
from scirust_b200.numerics import quaternion_search as S
from scirust_b200.numerics.accumulate import NAIVE, NEUMAIER


def test_static_pipeline_matches_reference_bitwise_and_torch_closely(tmp_path):
    torch.manual_seed(0)
    seq = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.ReLU(), torch.nn.Linear(7, 3))
    layers, wb = aot.from_torch_sequential(seq)
    assert len(wb) == aot.expected_weight_bytes(layers) == 4 * (5 * 7 + 7 + 7 * 3 + 3)
    src = aot.generate_static_pipeline(layers, wb)
    assert "static_model_forward" in src and "weight_0[5][7]" in src and "bias_2[3]" in src
    cp = aot.compile_pipeline(layers, wb, out_dir=str(tmp_path))
    assert (cp.in_dim, cp.out_dim) == (5, 3)
    x = np.random.default_rng(1).standard_normal((6, 5)).astype(np.float32)
    y = cp(x)
    assert np.array_equal(y, aot.reference_forward(layers, wb, x))
    assert np.abs(y - seq(torch.from_numpy(x)).detach().numpy()).max() < 1e-5
    with pytest.raises(ValueError):
        cp(np.zeros((2, 4), np.float32))


def test_static_pipeline_rejects_bad_streams_and_shapes():
    layers = [aot.Linear(2, 3), aot.ReLU(), aot.Linear(3, 1)]
    good = bytes(aot.expected_weight_bytes(layers))
    with pytest.raises(ValueError):
        aot.generate_static_pipeline(layers, good[:-4])                       # the biases are part of the stream
    with pytest.raises(ValueError):
        aot.generate_static_pipeline([aot.Linear(2, 3), aot.Linear(4, 1)], bytes(4 * (6 + 3 + 4 + 1)))
    with pytest.raises(ValueError):
        aot.generate_static_pipeline([aot.ReLU()], b"")
    bad = bytearray(good)
    bad[0:4] = np.float32(np.inf).tobytes()
    with pytest.raises(ValueError):
        aot.generate_static_pipeline(layers, bytes(bad))


def test_paillier_is_additively_homomorphic_and_probabilistic():
    src = H.UnsafeSeededSource(7)
    pk, sk = H.generate_keypair(256, src)
    assert 250 <= pk.n.bit_length() <= 256 and pk.nn == pk.n * pk.n
    a, b = 123456789, 987654321
    ca, cb = H.encrypt(a, pk), H.encrypt(b, pk)
    assert H.decrypt(ca, sk) == a
    assert H.decrypt(H.add_encrypted(ca, cb, pk), sk) == a + b
    assert H.decrypt(H.mul_plain(ca, 7, pk), sk) == 7 * a
    assert H.encrypt(a, pk) != H.encrypt(a, pk)                               # fresh blinding factor every time
    assert H.decrypt(H.encrypt(pk.n + 5, pk), sk) == 5                         # plaintexts live in Z_n
    assert H.is_probable_prime(2 ** 61 - 1) and not H.is_probable_prime(2 ** 61 + 1) and not H.is_probable_prime(561)


def test_encrypted_sum_of_signed_fixed_point_vectors():
    pk, sk = H.generate_keypair(128, H.UnsafeSeededSource(3))
    g1, g2, g3 = [0.5, -1.25, 3.0], [0.25, -2.0, -3.0], [-1.0, 0.125, 1e-3]
    total = H.encrypt_vector(g1, pk)
    for g in (g2, g3):
        total = H.add_vectors(total, H.encrypt_vector(g, pk), pk)
    got = H.decrypt_vector(total, sk)
    assert np.allclose(got, np.sum([g1, g2, g3], 0), atol=3 * 2.0 ** -24)
    with pytest.raises(ValueError):
        H.encode_fixed(float("nan"), pk)
    with pytest.raises(ValueError):
        H.add_vectors(total, total[:-1], pk)


def test_quaternion_charts_recover_a_noise_free_orientation_and_ignore_sign_flips():
    truth = S.q_from_axis_angle([1.0, 1.0, 1.0], 0.7)
    for chart in S.default_chart_dictionary():
        est = S.average(chart, NEUMAIER, truth.expand(10, 4))
        assert float(S.angular_error_degrees(est, truth)) < 1e-3, chart.name()
    ident = torch.tensor([1.0, 0, 0, 0], dtype=torch.float64)
    flipped = torch.stack([ident, -ident, ident, -ident, -ident, ident])
    assert float(S.angular_error_degrees(S.average(S.COMPONENTWISE, NAIVE, flipped), ident)) < 1e-6
    ref, q = S.q_from_axis_angle([0.0, 1.0, 0.0], 0.3), S.q_from_axis_angle([1.0, 0.0, 0.0], 0.9)
    assert float(S.angular_error_degrees(S.exp_relative(ref, S.log_relative(ref, q)), q)) < 1e-4
    assert S.Chart("log", 2).cost() == 8 and S.COMPONENTWISE.cost() == 0


def test_joint_chart_search_dominates_sequential_on_dev_and_wins_at_high_noise():
    truth = S.q_from_axis_angle([1.0, 1.0, 1.0], 0.7)
    dev, held = S.noisy_trials(truth, 1.5, 12, 100, 10), S.noisy_trials(truth, 1.5, 12, 100, 11)
    seq, joint = S.sequential_baseline(truth, dev, held), S.joint_search(truth, dev, held)
    assert S.score_plan(joint.plan, truth, dev, dev) >= S.score_plan(seq.plan, truth, dev, dev) - 1e-9
    assert joint.plan.chart.kind == "log"
    assert joint.eval_mean_error_degrees < 0.8 * seq.eval_mean_error_degrees   # at least 20 % less angular error
    assert S.score_plan(joint.plan, truth, dev, held[:0]) is None

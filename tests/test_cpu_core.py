"""CPU tests: RNG streams, formats, tape/optimizers, numerics, quantisation, tokenizer, caches,
data, deterministic MLP, CLI exit codes."""
import json
import math
import os
import struct

import numpy as np
import pytest
import torch

from scirust_b200 import nn, quantization as Q
from scirust_b200.autodiff import Adam, AdamW, Sgd, Tape, WarmupCosine
from scirust_b200.io import artifacts as A
from scirust_b200.io import checkpoint as CK
from scirust_b200.io import proof, safetensors as ST
from scirust_b200.nn.rng import PcgEngine, Philox4x32
from scirust_b200.numerics import lowprec as L
from scirust_b200.numerics import portable as P
from scirust_b200.numerics import reproducible as R

# golden files of the reference implementation: a checkout beside this repository, or SCIRUST_REFERENCE_DIR
REF = os.environ.get("SCIRUST_REFERENCE_DIR") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
need_ref = pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not mounted")


# ------------------------------------------------------------------ RNG
def test_pcg_is_deterministic_and_in_range():
    a, b = PcgEngine(42), PcgEngine(42)
    assert [a.next_u32() for _ in range(100)] == [b.next_u32() for _ in range(100)]
    assert PcgEngine(1).next_u32() != PcgEngine(2).next_u32()
    f = PcgEngine(7).fill_float((1000,))
    assert 0.0 <= float(f.min()) and float(f.max()) < 1.0
    n = PcgEngine(3).fill_normal((20000,), 1.0, 2.0)
    assert abs(float(n.mean()) - 1.0) < 0.05 and abs(float(n.std()) - 2.0) < 0.05


def test_philox_known_answers_and_fingerprint():
    z = Philox4x32(0)
    assert z.block([0, 0, 0, 0]).tolist() == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = Philox4x32(0xFFFFFFFFFFFFFFFF)
    assert f.block([0xFFFFFFFF] * 4).tolist() == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    p = Philox4x32((0x299F31D0 << 32) | 0xA4093822)
    assert p.block([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344]).tolist() == [0xD16CFE09, 0x94FDCCEB, 0x5001E420,
                                                                                  0x24126EA1]
    rng = Philox4x32(20260710)
    fp = 0xCBF29CE484222325
    for i in range(4096):
        fp = ((fp ^ rng.u32_at(0, i)) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert fp == 0xF96C6B6AECA699F5


# ------------------------------------------------------------------ formats
def test_safetensors_layout_and_errors():
    t = {"b": torch.arange(6.0).reshape(2, 3), "a": torch.ones(1, 2)}
    raw = ST.serialize([("b", t["b"]), ("a", t["a"])])
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert raw[8:8 + hlen].decode() == ('{"b":{"dtype":"F32","shape":[2,3],"data_offsets":[0,24]},'
                                        '"a":{"dtype":"F32","shape":[1,2],"data_offsets":[24,32]}}')
    back = ST.deserialize(raw)
    assert torch.equal(back["b"], t["b"]) and torch.equal(back["a"], t["a"])
    for bad in (b"", raw[:20], struct.pack("<Q", 1 << 40) + b"{}", struct.pack("<Q", 2) + b"[]"):
        with pytest.raises(ValueError):
            ST.deserialize(bad)


@need_ref
def test_safetensors_roundtrip_of_shipped_checkpoint_is_byte_identical():
    raw = open(f"{REF}/scirust-sciagent/checkpoints/small-20M/final/model.safetensors", "rb").read()
    sd = ST.deserialize(raw)
    assert len(sd) == 38 and tuple(sd["sciagent.embed.weight"].shape) == (8192, 128)
    assert ST.serialize([(k, sd[k]) for k in ST.header_order(raw)]) == raw


def test_srt1_manifest_qsr1_proof():
    sd = {"1.weight": torch.randn(3, 2), "0.bias": torch.randn(1, 3)}
    raw = A.srt1_to_bytes(sd)
    assert raw[:4] == b"SRT1" and raw[8:12] == struct.pack("<I", 6)  # keys sorted: "0.bias" first
    back = A.srt1_from_bytes(raw)
    assert all(torch.equal(back[k], sd[k]) for k in sd)
    with pytest.raises(ValueError):
        A.srt1_from_bytes(raw[:-3])
    specs = [A.LayerSpec("conv2d", (1, 8, 3, 1, True, 28, 28)), A.LayerSpec("relu"), A.LayerSpec("maxpool2d", (2, 2, 8, 28, 28)),
             A.LayerSpec("linear", (1568, 10)), A.LayerSpec("layernorm", (10, 1e-5))]
    text = A.write_manifest(specs)
    assert text.splitlines()[0] == "conv2d 1 8 3 1 same 28 28" and text.splitlines()[-1] == "layernorm 10 0.00001"
    assert A.parse_manifest("# c\n\n" + text) == specs
    with pytest.raises(ValueError):
        A.parse_manifest("linear 3")
    m = A.QModel([A.QLinear(3, 2, 0.01, True, np.array([0.002, 0.003], np.float32), np.array([1, -2, 3, 4, -5, 6], np.int8),
                            np.array([10, -20], np.int32)),
                  A.QLinear(2, 2, 0.05, False, np.array([0.01, 0.02], np.float32), np.array([1, 2, -3, 4], np.int8),
                            np.array([0, 5], np.int32))])
    b = m.to_bytes()
    m2 = A.QModel.from_bytes(b)
    assert m2.to_bytes() == b
    x = [0.5, -0.25, 0.125]
    assert np.array_equal(m.infer(x, 1), m2.infer(x, 1))
    for cut in (3, 9, 20, len(b) - 1):
        with pytest.raises(ValueError):
            A.QModel.from_bytes(b[:cut])
    bundle = proof.build_bundle(b, 2, [1, 2])
    assert proof.verify_bundle(bundle, b) == []
    tampered = bytearray(b)
    tampered[-1] ^= 1
    assert proof.verify_bundle(bundle, bytes(tampered))
    cert = proof.resource_certificate(m, 2)
    assert cert["mac_count"] == 2 * (3 * 2 + 2 * 2)


def test_quantize_multiplier_and_requant():
    m, s = A.quantize_multiplier(0.3)
    assert 2 ** 30 <= m < 2 ** 31 and abs(m / 2 ** 31 / 2 ** s - 0.3) < 1e-9
    assert A.quantize_multiplier(0.0) == (0, 0)
    assert int(A.requant_i32(np.array([1000], dtype=np.int64), m, s)[0]) == 300
    assert A.quantize_tensor(np.array([0.5, -0.5, 1.5, 2.5, 500.0], np.float32), 1.0).tolist() == [1, -1, 2, 3, 127]


def test_core_checkpoint_json(tmp_path):
    CK.save_checkpoint(tmp_path / "e3", {"w": torch.ones(2, 2)}, {"learning_rate": 0.1, "m": {"w": torch.zeros(4)}}, 3, 30)
    CK.save_checkpoint(tmp_path / "e1", {"w": torch.ones(2, 2)}, {}, 1, 10)
    ck = CK.load_checkpoint(tmp_path / "e3")
    assert ck["weights"]["w"] == [1.0] * 4 and ck["optimizer_state"]["learning_rate"] == pytest.approx(0.1)
    assert [e for e, _ in CK.list_checkpoints(tmp_path)] == [1, 3]


# ------------------------------------------------------------------ tape and optimizers
def test_tape_gradients_match_finite_differences():
    torch.manual_seed(0)
    x0, w0 = torch.randn(5, 4), torch.randn(4, 3)

    def f(w):
        t = Tape()
        x, wv = t.constant(x0), t.input(w)
        y = x.matmul(wv).tanh().softmax().log().sum_axis(1).mean()
        return t, wv, y
    t, wv, y = f(w0)
    t.backward(y)
    g = t.grad(wv.idx).t
    num = torch.zeros_like(w0)
    for i in range(4):
        for j in range(3):
            d = torch.zeros_like(w0)
            d[i, j] = 1e-3
            num[i, j] = (f(w0 + d)[2].item() - f(w0 - d)[2].item()) / 2e-3
    assert torch.allclose(g, num, atol=2e-3)
    with pytest.raises(Exception):
        Tape().input(torch.ones(1, 1)).add(wv)


def test_optimizer_formulas():
    for opt, expect in ((Sgd(0.1).with_momentum(0.9), None), (Adam(0.01), None), (AdamW(0.01, weight_decay=0.1), None)):
        t = Tape()
        w = t.input(torch.tensor([[1.0, -2.0]]))
        t.backward(w.mul(w).sum())
        p0 = w.t.detach().clone()
        opt.step([w.idx], t)
        g = 2 * p0
        if isinstance(opt, Sgd):
            ref = p0 - 0.1 * g
        else:
            m, v = 0.1 * g, 0.001 * g * g
            upd = 0.01 * (m / 0.1) / (torch.sqrt(v / 0.001) + 1e-8)
            ref = p0 - upd - (0.01 * 0.1 * p0 if isinstance(opt, AdamW) else 0)
        assert torch.allclose(w.t.detach(), ref, atol=1e-6)
    s = WarmupCosine(1.0, 0.1, 10, 110)
    assert s.lr_at(0) == 0 and s.lr_at(10) == pytest.approx(1.0) and s.lr_at(110) == 0.1 and s.lr_at(60) == pytest.approx(0.55)


# ------------------------------------------------------------------ numerics
def test_reproducible_sum_is_order_independent_and_correctly_rounded():
    xs = (np.random.RandomState(0).randn(500) * 10.0 ** np.random.RandomState(1).randint(-6, 7, 500)).astype(np.float32)
    a = R.reproducible_sum(xs)
    assert a == R.reproducible_sum(xs[::-1]) == R.reproducible_sum(np.random.RandomState(2).permutation(xs))
    assert a == float(np.float32(math.fsum(float(v) for v in xs)))
    acc1, acc2 = R.ExactAccumulator().add_all(xs[:200]), R.ExactAccumulator().add_all(xs[200:])
    acc1.merge(R.ExactAccumulator.from_bytes(acc2.to_bytes()))
    assert acc1.round_f32() == a


def test_portable_functions():
    import decimal
    for x in (0.0, 1.0, -3.5, 10.25, 88.0, -100.0):
        want = float(np.float32(float(decimal.Context(prec=50).exp(decimal.Decimal(x)))))
        assert float(P.exp_f32(x)) == want
    assert float(P.ln_f32(1.0)) == 0.0 and np.isnan(P.ln_f32(-1.0)) and P.exp_f32(200.0) == np.inf
    sm = P.softmax_f32([1.0, 2.0, 3.0])
    assert abs(float(sm.sum()) - 1.0) < 1e-6
    a, b = torch.randn(6, 9), torch.randn(9, 4)
    assert torch.equal(P.gemm_f32(a, b), (a.double() @ b.double()).float()) or torch.allclose(P.gemm_f32(a, b), a @ b, atol=1e-5)


def test_lowprec():
    assert L.to_bf16([1.00390625])[0] == 1.0 and L.to_bf16([1.01171875])[0] == np.float32(1.015625)
    sr = L.stochastic_round_bf16(np.full(2000, 1.00390625, np.float32), seed=5)
    frac = float((sr > 1.0).mean())
    assert 0.4 < frac < 0.6
    assert np.array_equal(sr[:100], L.stochastic_round_bf16(np.full(100, 1.00390625, np.float32), seed=5))
    sc = L.DynamicLossScaler(init_scale=8.0, growth_interval=2)
    assert not sc.update(True) and sc.scale == 4.0
    assert sc.update(False) and sc.update(False) and sc.scale == 8.0


# ------------------------------------------------------------------ quantisation
def test_quantization_core_vectors():
    q, s = Q.quantize_per_channel([1.0, -2.0, 0.5, 4.0, 1.0, -0.25], 2, 3)
    assert np.allclose(s, [4 / 127, 2 / 127, 0.5 / 127]) and q.tolist() == [32, -127, 127, 127, 64, -64]
    assert Q.matmul_int8([1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], 2, 3, 2).tolist() == [58, 64, 139, 154]
    assert Q.quantize_tensor([500.0, -500.0, 0.0], Q.compute_scale([500.0, -500.0, 0.0])).tolist() == [127, -127, 0]
    x = np.random.RandomState(0).randn(4, 8).astype(np.float32)
    w = np.random.RandomState(1).randn(8, 5).astype(np.float32)
    wq, ws = Q.quantize_per_channel(w, 8, 5)
    y = Q.quantized_linear_forward(x, 4, 8, wq, ws, np.zeros(5, np.float32), 5).reshape(4, 5)
    assert np.abs(y - x @ w).max() < 0.15
    with pytest.raises(ValueError):
        Q.quantized_linear_forward(x, 4, 8, wq[:-1], ws, np.zeros(5), 5)


def test_quantization_methods():
    torch.manual_seed(0)
    W, X = torch.randn(32, 16), torch.randn(128, 32)
    rtn = Q._rtn(W, 4, W.abs().amax(0) / 7)
    assert ((X @ Q.gptq_quantize(W, X)) - X @ W).pow(2).mean() < ((X @ rtn) - X @ W).pow(2).mean()
    wq, s = Q.awq_quantize(W, X)
    assert ((X @ wq) - X @ W).pow(2).mean() <= ((X @ rtn) - X @ W).pow(2).mean() * 1.05
    codes, scale = Q.ternary_quantize(W)
    assert set(codes.unique().tolist()) <= {-1, 0, 1}
    assert (Q.nf4_dequantize(*Q.nf4_quantize(W)) - W).abs().max() < 0.6
    assert (Q.int4_group_dequantize(*Q.int4_group_quantize(W)) - W).abs().max() < 0.35
    xs, wsm, sm = Q.smoothquant_apply(X, W)
    assert torch.allclose(xs @ wsm, X @ W, atol=1e-4)


# ------------------------------------------------------------------ tokenizer, caches, data
def test_bpe_train_encode_decode(tmp_path):
    from scirust_b200.tokenizer import BpeTokenizer, BpeTrainer
    text = "fn alpha<T>() { alpha::<T>(); } // café — ✅\n" * 40
    tok = BpeTrainer(400).train([text])
    tok2 = BpeTrainer(400).train([text])
    assert tok.merges == tok2.merges
    for src in ["Vec<T>", "fn main() {}", "a < b && b << 2", "", "rms → √(mean(x²)+eps) · wᵀ ✅ é"]:
        assert tok.decode(tok.encode(src)) == src
    tok.save_json(tmp_path / "t.json")
    back = BpeTokenizer.load_json(tmp_path / "t.json")
    assert back.encode("fn alpha") == tok.encode("fn alpha")
    assert tok.encode_with_special("x", True, True)[0] == 1 and tok.encode_with_special("x", True, True)[-1] == 2
    with pytest.raises(ValueError):
        BpeTokenizer.from_json_str("{}")


def test_kv_caches_against_plain():
    from scirust_b200.nn.kv_cache import (ElasticKvCache, LatentKvCache, PagedKvCache, PlainKvCache, QuantKvCache,
                                          TieredKvCache)
    torch.manual_seed(0)
    d = 16
    caches = {"plain": PlainKvCache(d), "paged": PagedKvCache(d, 4, 16), "q8": QuantKvCache(d, 8),
              "elastic": ElasticKvCache(d, window=8), "latent": LatentKvCache(d, d, residual_bits=0),
              "tiered": TieredKvCache(d, d, hot=4, warm=8)}
    for _ in range(37):
        k, v = torch.randn(d), torch.randn(d)
        for c in caches.values():
            c.append(k, v)
    q = torch.randn(d)
    ref = caches["plain"].decode_step(q)
    assert torch.equal(caches["paged"].decode_step(q), ref)      # paged == contiguous, bit for bit
    assert (caches["q8"].decode_step(q) - ref).abs().max() < 0.05
    assert (caches["elastic"].decode_step(q) - ref).abs().max() < 0.5
    assert (caches["latent"].decode_step(q) - ref).abs().max() < 1e-4   # full-rank basis is lossless
    assert (caches["tiered"].decode_step(q) - ref).abs().max() < 0.05
    small = ElasticKvCache(d, window=4, budget_bytes=4 * d * 8 + 10 * (d // 2 + 4) * 2)
    for _ in range(64):
        small.append(torch.randn(d), torch.randn(d))
        small.decode_step(q)
    assert small.evicted > 0 and small.nbytes() <= small.budget
    caches["paged"].release()
    assert len(caches["paged"].free) == 16


def test_data_loading_is_a_function_of_seed_and_epoch(tmp_path):
    from scirust_b200.data import DataLoader, TokenShardDataset, gaussian_clusters, write_token_shard
    ds = gaussian_clusters()
    a, b = DataLoader(ds, 16, seed=3), DataLoader(ds, 16, seed=3)
    assert torch.equal(a.order(5), b.order(5)) and not torch.equal(a.order(5), a.order(6))
    assert sum(x.shape[0] for x, _ in a) == 150 and a.epoch == 1
    write_token_shard(tmp_path / "s.bin", np.arange(5000) % 300)
    ts = TokenShardDataset([tmp_path / "s.bin"], 32, vocab_size=256, val_frac=0.1, seed=1)
    assert int(ts.tokens.max()) < 256 and (ts.tokens == 3).any()      # ids >= vocab map to <unk>
    assert len(ts.val_windows) > 0 and len(ts.train_windows) + len(ts.val_windows) == (5000 - 1) // 32
    b1 = ts.batch(7, 4)
    assert b1.shape == (4, 33) and torch.equal(b1, TokenShardDataset([tmp_path / "s.bin"], 32, 256, 0.1, 1).batch(7, 4))


def test_deterministic_mlp_is_bit_reproducible():
    from scirust_b200.models.mlp_cpu import train_gaussian_mlp
    m1, h1 = train_gaussian_mlp(epochs=30)
    m2, h2 = train_gaussian_mlp(epochs=30)
    assert m1.fingerprint() == m2.fingerprint() and h1 == h2
    assert h1[-1][1] >= 0.95 and h1[-1][0] < h1[0][0]
    m3, _ = train_gaussian_mlp(epochs=30, fma=True)
    assert m3.fingerprint() != m1.fingerprint()       # fused multiply-add is a different rounding order


def test_cli_exit_codes(tmp_path, capsys):
    from scirust_b200 import cli
    assert cli.run(["version"]) == 0
    assert cli.run(["nonsense"]) == 2
    assert cli.run(["sciagent", "info", "--checkpoint", str(tmp_path / "missing")]) == 3
    assert cli.run(["train", "--model", "debug", "--steps", "2", "--checkpoint-dir", str(tmp_path / "ck")]) == 0
    assert (tmp_path / "ck" / "step_2" / "meta.json").exists()
    assert not list((tmp_path / "ck").glob(".*partial"))
    assert cli.run(["infer", "--checkpoint", str(tmp_path / "ck" / "step_2"), "--prompt", "5 6 7", "--max-new", "4"]) == 0
    out1 = capsys.readouterr().out
    assert cli.run(["infer", "--checkpoint", str(tmp_path / "ck" / "step_2"), "--prompt", "5 6 7", "--max-new", "4"]) == 0
    assert capsys.readouterr().out.splitlines()[-1] == out1.splitlines()[-1]


def test_nd_tape_surface_gradients_and_errors():
    """N-D tape: finite-difference check through gather / rope / bmm / softmax / rmsnorm / layernorm / causal_conv /
    cross_entropy, lag-ordered convolution equals the direct loop bit for bit, tapes do not mix."""
    from scirust_b200.autodiff import NdTape, NdTapeError
    torch.manual_seed(0)
    E0, W0, H0 = torch.randn(10, 8) * 0.3, torch.randn(8, 10) * 0.3, torch.randn(4, 8) * 0.1

    def loss_of(Ev):
        t = NdTape()
        E = t.input(Ev)
        x = E.gather([1, 2, 3, 4])
        q = x.reshape([1, 4, 8]).rope(10000.0)
        a = q.bmm(q.transpose_last2()).softmax().bmm(x.reshape([1, 4, 8])).reshape([4, 8]).rmsnorm(1e-5)
        y = a.causal_conv(t.input(H0)).add(x.layernorm(1e-5)).relu().add(x.sigmoid().mul(0.1))
        loss = y.matmul(t.input(W0)).cross_entropy([2, 3, 4, 5])
        return t, E, loss

    t, E, loss = loss_of(E0)
    g = t.backward(loss)[E.idx]
    assert g.shape == E0.shape and float(g[0].abs().sum()) == 0.0      # row 0 was not gathered
    for (r, c) in ((1, 0), (3, 5), (4, 7)):
        d = torch.zeros_like(E0)
        d[r, c] = 1e-3
        fp = float(loss_of(E0 + d)[0].value(loss_of(E0 + d)[2]))
        fm = float(loss_of(E0 - d)[0].value(loss_of(E0 - d)[2]))
        assert abs((fp - fm) / 2e-3 - float(g[r, c])) < 5e-3
    u, h = torch.randn(6, 3), torch.randn(6, 3)
    t2 = NdTape()
    y = t2.value(t2.input(u).causal_conv(t2.input(h)))
    ref = torch.zeros(6, 3)
    for tt in range(6):
        for c in range(3):
            acc = torch.tensor(0.0)
            for tau in range(tt + 1):
                acc = acc + h[tau, c] * u[tt - tau, c]
            ref[tt, c] = acc
    assert torch.equal(y, ref)
    with pytest.raises(NdTapeError):
        NdTape().input(u).add(t2.input(h))
    with pytest.raises(NdTapeError):
        t2.input(torch.randn(3, 4)).cross_entropy([0, 1, 9])
    s = t2.input(torch.ones(2, 3)).sum()
    assert t2.value(s).tolist() == [6.0] and s.shape() == [1]
    parts = t2.input(torch.ones(1, 3)).cat0([t2.input(torch.zeros(2, 3))])
    assert parts.shape() == [3, 3]


def test_attestation_log_certified_bounds_and_guard():
    from scirust_b200.certify import (IbpLinear, IbpMlp, Interval, StatisticalGuard, certified_robust, crown_bounds)
    from scirust_b200.io.attest import AttestationLog, P, VModel, attest_and_record, verify_inference
    from scirust_b200.io.execution_attestation import (ExecutionAttestation, build_decode_route_attestation,
                                                       build_training_route_attestation, sha256_hex)
    m = VModel(list(range(1, 25)), 4, 6)
    x = list(range(18))
    y = m.infer(x, 3)
    assert verify_inference(m, x, 3, y)
    log = AttestationLog()
    assert attest_and_record(log, m, x, 3, y) is not None and log.verify_chain()
    bad = list(y)
    bad[5] = (bad[5] + 1) % P
    assert attest_and_record(log, m, x, 3, bad) is None and len(log) == 1
    log.record(m.commit(), x, y)
    head = log.head
    log.events[0].output_hash = bytes(32)
    assert not log.verify_chain() and log.head == head

    torch.manual_seed(0)
    l1 = IbpLinear(torch.randn(4, 8) * 0.5, torch.randn(8) * 0.1)
    l2 = IbpLinear(torch.randn(8, 3) * 0.5, torch.randn(3) * 0.1)
    box = Interval.around([0.2, -0.5, 0.7, -0.1], 0.05)
    mlp = IbpMlp([l1, l2])
    ibp, cr = mlp.certify(box), crown_bounds(l1, l2, box)
    assert float(cr.width().mean()) <= float(ibp.width().mean()) + 1e-6
    for _ in range(200):
        pt = box.lo + (box.hi - box.lo) * torch.rand(4)
        out = mlp.forward(pt)
        assert bool((out >= cr.lo - 1e-5).all() and (out <= cr.hi + 1e-5).all())
        assert bool((out >= ibp.lo - 1e-5).all() and (out <= ibp.hi + 1e-5).all())
    tight = mlp.certify(Interval.around([0.2, -0.5, 0.7, -0.1], 1e-6))
    assert certified_robust(tight, int(mlp.forward([0.2, -0.5, 0.7, -0.1]).argmax()))

    g = torch.Generator().manual_seed(1)
    yv = torch.randint(0, 3, (3000,), generator=g)
    lg = torch.rand(3000, 3, generator=g) * 2 - 1
    lg[torch.arange(3000), yv] += 1.5
    pr = torch.softmax(lg, -1)
    guard = StatisticalGuard.calibrate(pr[:1500], yv[:1500], 0.1)
    cover = sum(guard.covers(p_, int(t_)) for p_, t_ in zip(pr[1500:], yv[1500:])) / 1500
    assert cover >= 0.87
    assert guard.decide([0.97, 0.02, 0.01])[0] == "accept" and guard.decide([0.34, 0.33, 0.33])[0] == "reject"

    a1 = build_training_route_attestation(sha256_hex(b"m"), sha256_hex(b"t"))
    a2 = build_decode_route_attestation(sha256_hex(b"m"), sha256_hex(b"t"), weights="int8")
    assert a1.verify() and a2.verify() and a1.attestation_sha256 != a2.attestation_sha256
    back = ExecutionAttestation.from_json(a2.to_json())
    assert back.verify() and back.profile.numeric_mode.startswith("int8")
    back.profile.model_sha256 = sha256_hex(b"other")
    assert not back.verify()


def test_api_header_lists_every_entry_point_and_matches_the_ctypes_tables():
    """csrc/api.h is generated from the extern "C" definitions: it must be current, and every ctypes signature
    registered by the ops modules must have the arity of its declaration."""
    import importlib
    import re
    from scirust_b200 import _build
    from scirust_b200.ops import _lib
    assert (_build.CSRC / "api.h").read_text() == _build.api_header_text(), \
        "api.h is stale: run python -m scirust_b200._build --api-header"
    decls = {}
    for _f, d in _build.cuda_entry_points():
        m = re.match(r".*?\b(sb_\w+)\((.*)\)$", d)
        args = [a for a in m.group(2).split(",") if a.strip() and a.strip() != "void"]
        decls[m.group(1)] = len(args)
    assert len(decls) >= 60
    for mod in ("basic", "gemm", "attention", "decode", "conv", "sampling", "canonical"):
        importlib.import_module(f"scirust_b200.ops.{mod}")
    for mod in ("symm", "fused_allreduce", "small_collectives", "tensor_parallel", "vocab_parallel"):
        importlib.import_module(f"scirust_b200.parallel.{mod}")
    checked = 0
    for name, sig in _lib._CUDA_SIGS.items():
        assert name in decls, f"{name} has a ctypes signature but no entry point"
        assert len(sig) == decls[name], f"{name}: ctypes table has {len(sig)} parameters, the definition {decls[name]}"
        checked += 1
    assert checked >= 40


def test_raw_runtime_validation_and_strict_compile_without_a_gpu():
    from scirust_b200.runtime import (RawAccess, RawBinding, RawBuffer, RawError, RawLaunchConfig, compile_cuda_c,
                                      validate_alias_groups, validate_launch_geometry)
    from scirust_b200.runtime.raw import validate_bindings
    ok = RawLaunchConfig((4, 1, 1), (256, 1, 1), 1024)
    validate_launch_geometry(ok)
    for bad, frag in ((RawLaunchConfig((0, 1, 1), (256, 1, 1)), "grid dimensions must be non-zero"),
                      (RawLaunchConfig((1, 1, 1), (0, 1, 1)), "block dimensions must be non-zero"),
                      (RawLaunchConfig((1, 70000, 1), (32, 1, 1)), "grid dimension 1"),
                      (RawLaunchConfig((1, 1, 1), (32, 32, 2)), "2048 threads"),
                      (RawLaunchConfig((1, 1, 1), (32, 1, 1), 300 * 1024), "shared-memory")):
        with pytest.raises(RawError, match=frag):
            validate_launch_geometry(bad)
    a, b = RawBuffer(1024), RawBuffer(1024)
    R, W = RawAccess.READ, RawAccess.WRITE
    validate_alias_groups([RawBinding(a, R), RawBinding(a, R), RawBinding(b, W)])             # two readers share
    validate_alias_groups([RawBinding(a, R, 0, 512), RawBinding(a, W, 512, 512)])             # disjoint halves
    with pytest.raises(RawError, match="alias"):
        validate_alias_groups([RawBinding(a, R), RawBinding(b, R), RawBinding(a, W, 100, 8)])
    with pytest.raises(RawError, match="alias"):
        validate_alias_groups([RawBinding(a, RawAccess.READ_WRITE), RawBinding(a, RawAccess.READ_WRITE)])
    with pytest.raises(RawError, match="exceeds buffer bounds"):
        validate_bindings([RawBinding(a, R, 1000, 100)])
    with pytest.raises(RawError, match="non-zero"):
        validate_bindings([RawBinding(a, R, 10, 0)])
    src = 'extern "C" __global__ void axpy(float* y, const float* x, float a, int n) {' \
          ' int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < n) y[i] = a * x[i] + y[i]; }'
    ptx = compile_cuda_c(src).decode(errors="replace")
    assert "axpy" in ptx and "sm_100a" in ptx
    assert "fma.rn.f32" not in ptx and "mul.rn.f32" in ptx and "add.rn.f32" in ptx        # --fmad=false: no contraction
    assert "fma.rn.f32" in compile_cuda_c(src, strict_ieee=False).decode(errors="replace")
    with pytest.raises(RawError, match="pinned"):
        compile_cuda_c(src, extra_options=["--use_fast_math"])
    with pytest.raises(RawError, match="compilation failed"):
        compile_cuda_c("this is not CUDA")


def test_squeezellm_spqr_omniquant_aqlm_quip_and_fake_quant():
    from scirust_b200 import quantization_methods as QM
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 32, generator=g) * 0.1
    w[3, 5], w[40, 7] = 2.5, -3.0                                    # heavy tails
    qmax = 7.0

    def rtn(x):
        s = x.abs().amax(0) / qmax
        return torch.clamp(torch.round(x / s), -qmax, qmax) * s
    e_rtn = (w - rtn(w)).pow(2).sum()

    # SqueezeLLM: lower sensitivity-weighted error than the uniform grid of the same size; deterministic
    sens = torch.ones(w.numel())
    cb = QM.SqueezeLlmCodebook.fit(w.reshape(-1), sens, 4, 25)
    rec = cb.dequantize(cb.quantize(w))
    s_all = w.abs().max() / qmax
    uni = torch.clamp(torch.round(w / s_all), -qmax - 1, qmax) * s_all
    assert (w - rec).pow(2).sum() < 0.5 * (w - uni).pow(2).sum()
    assert torch.equal(cb.levels, QM.SqueezeLlmCodebook.fit(w.reshape(-1), sens, 4, 25).levels)
    assert cb.levels.numel() == 16 and torch.equal(cb.levels, torch.sort(cb.levels).values)
    # SpQR: 1 % outliers remove most of the dense error, and are exactly the largest errors
    sp = QM.SpqrOutliers.extract(w, uni, 0.01)
    fixed = sp.apply(uni)
    assert sp.indices.numel() == round(w.numel() * 0.01)
    assert (w - fixed).pow(2).sum() < (w - uni).pow(2).sum()
    assert float((w - fixed).abs().max()) <= float((w - uni).abs().reshape(-1).sort().values[-sp.indices.numel() - 1]) + 1e-7
    assert QM.SpqrOutliers.extract(w, uni, 0.0).indices.numel() == 0
    # OmniQuant: never worse than RTN per channel, strictly better where a channel has an outlier
    oq = QM.omniquant_quantize(w, 4)
    e_oq = (w - oq.dequantize()).pow(2).sum(0)
    e_r = (w - rtn(w)).pow(2).sum(0)
    assert bool((e_oq <= e_r + 1e-9).all()) and e_oq[5] < e_r[5] and float(oq.gammas[5]) < 1.0 and e_oq.sum() < e_r.sum()
    assert oq.codes.dtype == torch.int8 and int(oq.codes.abs().max()) <= 7
    # AQLM: two additive codebooks beat one at the same group size; reported bit budget
    a1 = QM.quantize_aqlm(w, 8, 1, 16, 6)
    a2 = QM.quantize_aqlm(w, 8, 2, 16, 6)
    assert (w - a2.dequantize()).pow(2).sum() < (w - a1.dequantize()).pow(2).sum()
    assert a2.bits_per_weight() == 1.0 and a2.dequantize().shape == w.shape
    # QuIP#: the transform is orthonormal and self-inverse, E8 points are lattice points, error shrinks with bits
    v = torch.randn(37, generator=g)
    t = QM.random_hadamard_transform(v, 9)
    assert torch.allclose(QM.inverse_random_hadamard_transform(t, 9, 37), v, atol=1e-6)
    assert abs(float(t.pow(2).sum()) - float(v.pow(2).sum())) < 1e-4
    pts = QM.nearest_e8(torch.randn(200, 8, generator=g) * 2)
    twice = pts * 2
    assert torch.equal(twice, twice.round())                                     # integers or half-integers
    assert bool(((twice.long() % 2 == 0).all(1) | (twice.long() % 2 != 0).all(1)).all())   # never mixed
    assert bool((pts.sum(1).round().long() % 2 == 0).all())                      # even coordinate sum
    q2, q4 = QM.quantize_quip(w, 2, 3), QM.quantize_quip(w, 4, 3)
    assert (w - q4.dequantize()).pow(2).sum() < (w - q2.dequantize()).pow(2).sum()
    assert torch.equal(q4.dequantize(), QM.quantize_quip(w, 4, 3).dequantize())
    # fake quantisation: values on the grid, straight-through gradient with zero outside the clip range
    x = torch.tensor([0.11, -0.52, 3.0, -4.0], requires_grad=True)
    y = QM.fake_quantize(x, 4, scale=0.1)
    assert torch.allclose(y, torch.tensor([0.1, -0.5, 0.7, -0.7]))
    y.sum().backward()
    assert x.grad.tolist() == [1.0, 1.0, 0.0, 0.0]


def test_residual_latent_adaptive_and_tiered_kv_caches():
    from scirust_b200.nn.kv_cache import PlainKvCache
    from scirust_b200.nn.kv_cache_latent import (AdaptiveKvPlanner, ResidualLatentCacheError,
                                                 ResidualQuantizedLatentKvCache, SparseResidualConfig,
                                                 TieredResidualLatentBackend, estimate_channel_bytes, fit_basis)
    g = torch.Generator().manual_seed(0)
    dim, n = 32, 40
    low = torch.randn(n, 6, generator=g) @ torch.randn(6, dim, generator=g)       # rows near a rank-6 subspace
    K = low + 0.02 * torch.randn(n, dim, generator=g)
    V = torch.randn(n, 6, generator=g) @ torch.randn(6, dim, generator=g) + 0.02 * torch.randn(n, dim, generator=g)
    K[7, 3] += 4.0                                                               # an off-subspace spike
    kb, vb = fit_basis(K), fit_basis(V)
    plain = PlainKvCache(dim)
    full = ResidualQuantizedLatentKvCache(dim, n, dim, dim, "fp32", "fp32", key_basis=kb, value_basis=vb)
    lat = ResidualQuantizedLatentKvCache(dim, n, 8, 8, "int8", "int8", key_basis=kb, value_basis=vb)
    res = ResidualQuantizedLatentKvCache(dim, n, 8, 8, "int8", "int8", SparseResidualConfig(2, "int8"),
                                         SparseResidualConfig(2, "int8"), kb, vb)
    for t in range(n):
        for c in (plain, full, lat, res):
            c.append(K[t], V[t])
    q = torch.randn(dim, generator=g)
    want = plain.decode_step(q)
    assert torch.allclose(full.attention(q), want, atol=1e-4)                   # full rank, fp32: the exact attention
    e_lat, e_res = (lat.attention(q) - want).norm(), (res.attention(q) - want).norm()
    assert e_lat < 0.2 * want.norm() and e_res <= e_lat + 1e-6
    k7, _ = res.reconstruct_token(7)
    k7_lat, _ = lat.reconstruct_token(7)
    assert (k7 - K[7]).norm() < (k7_lat - K[7]).norm()          # the residual slots pick up what the subspace lost
    assert len(res.key_residual_indices_for(7)) == 2 and lat.key_residual_indices_for(7) is None
    assert res.bytes_per_token() == 2 * estimate_channel_bytes(8, "int8", SparseResidualConfig(2, "int8"))
    assert res.allocated_bytes() == n * res.bytes_per_token() and res.used_bytes() == res.allocated_bytes()
    with pytest.raises(ResidualLatentCacheError, match="full"):
        res.append(K[0], V[0])
    res.remove_oldest()
    assert len(res) == n - 1 and torch.allclose(res.reconstruct_token(6)[0], k7)
    with pytest.raises(ResidualLatentCacheError):
        ResidualQuantizedLatentKvCache(dim, 4, 8, 8).append(torch.full((dim,), float("nan")), V[0])

    # planner: a larger budget never gives a worse plan, every plan respects its budget, planning is deterministic
    pl = AdaptiveKvPlanner(dim, ranks=(4, 8, 16), slot_choices=(0, 2), formats=("int8", "int4"))
    for t in range(24):
        pl.observe(K[t], V[t])
    small, _, _ = pl.plan(20)
    big, _, _ = pl.plan(64)
    assert small.bytes_per_token <= 20 and big.bytes_per_token <= 64 and big.error <= small.error + 1e-9
    assert pl.plan(20)[0] == small
    with pytest.raises(ResidualLatentCacheError, match="budget"):
        pl.plan(3)
    cache = pl.build(64, 16)
    cache.append(K[0], V[0])
    assert cache.bytes_per_token() == big.bytes_per_token

    # tiers: rows age hot -> warm -> cold, the cold tier evicts, attention spans all tiers
    hot = dict(capacity=4, key_rank=dim, value_rank=dim, key_fmt="fp32", value_fmt="fp32")
    warm = dict(capacity=8, key_rank=12, value_rank=12, key_fmt="int8", value_fmt="int8",
                key_residual=SparseResidualConfig(2, "int8"), value_residual=SparseResidualConfig(2, "int8"))
    cold = dict(capacity=8, key_rank=8, value_rank=8, key_fmt="int4", value_fmt="int4")
    tb = TieredResidualLatentBackend(dim, hot, warm, cold, kb, vb)
    for t in range(26):
        tb.append(K[t], V[t])
    tel = tb.telemetry()
    assert (tel.hot_tokens, tel.warm_tokens, tel.cold_tokens, tel.evictions) == (4, 8, 8, 6) and len(tb) == 20
    ref = PlainKvCache(dim)
    for t in range(6, 26):
        ref.append(K[t], V[t])
    got, wantt = tb.attention(q), ref.decode_step(q)
    assert (got - wantt).norm() < 0.35 * wantt.norm()
    assert tel.planned_persistent_bytes <= tel.allocated_bytes


def test_native_cpu_flash_attention_w8a8_block_and_kv_cache():
    import math
    from scirust_b200 import cpu_kernels as CK
    g = torch.Generator().manual_seed(0)
    B, S, H, Hkv, dh = 2, 70, 4, 2, 16
    q, k, v = (torch.randn(B, S, h, dh, generator=g) for h in (H, Hkv, Hkv))
    kr, vr = k.repeat_interleave(H // Hkv, 2), v.repeat_interleave(H // Hkv, 2)
    for causal in (True, False):
        sc = torch.einsum("bqhd,bkhd->bhqk", q, kr) / math.sqrt(dh)
        if causal:
            sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        ref = torch.einsum("bhqk,bkhd->bqhd", sc.softmax(-1), vr)
        out1 = CK.flash_attention(q, k, v, causal, block=16, threads=1)
        out4 = CK.flash_attention(q, k, v, causal, block=16, threads=4)
        assert torch.allclose(out1, ref, atol=2e-5) and torch.equal(out1, out4)       # thread-count independent
    # W8A8: equals the reference arithmetic written out in torch (int32 accumulation, one rescale)
    x, w = torch.randn(9, 40, generator=g), torch.randn(40, 24, generator=g) * 0.2
    wq, ws = CK.quantize_weight(w)
    sx = x.abs().amax(1) / 127.0
    xv = x / sx[:, None]
    xq = torch.where(xv >= 0, torch.floor(xv + 0.5), torch.ceil(xv - 0.5)).clamp(-128, 127)
    want = (xq.to(torch.int64) @ wq.to(torch.int64)).float() * (sx[:, None] * ws[None, :])
    got = CK.w8a8_linear(x, wq, ws)
    assert torch.equal(got, want)
    assert (got - x @ w).abs().max() < 0.05 * (x @ w).abs().max()
    # int8 decoder block close to its fp32 statement
    S2, d, ff, Hh, Hk = 24, 32, 48, 4, 2
    ws_ = {n: torch.randn(a, b, generator=g) * (1.0 / math.sqrt(a)) for n, (a, b) in
           dict(wq=(d, d), wk=(d, d // 2), wv=(d, d // 2), wo=(d, d), wg=(d, ff), wu=(d, ff), wd=(ff, d)).items()}
    g1, g2 = torch.ones(d), torch.ones(d)
    blk = CK.Int8DecoderBlock(Hh, Hk, 10000.0, 1e-5, g1, g2, **ws_)
    xs = torch.randn(S2, d, generator=g)
    y = blk.forward(xs)

    def rms(t):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5)

    def rope(t, nh):
        dh2 = d // Hh
        t = t.view(S2, nh, dh2 // 2, 2)
        ang = torch.arange(S2).float()[:, None] * (10000.0 ** (-2 * torch.arange(dh2 // 2).float() / dh2))[None]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        return torch.stack([t[..., 0] * c - t[..., 1] * s, t[..., 0] * s + t[..., 1] * c], -1).reshape(S2, nh, dh2)
    h = rms(xs)
    qf, kf, vf = rope(h @ ws_["wq"], Hh), rope(h @ ws_["wk"], Hk), (h @ ws_["wv"]).view(S2, Hk, d // Hh)
    ctx = CK.flash_attention(qf[None], kf[None], vf[None], True)[0].reshape(S2, d)
    x2 = xs + ctx @ ws_["wo"]
    h2 = rms(x2)
    ref = x2 + (torch.nn.functional.silu(h2 @ ws_["wg"]) * (h2 @ ws_["wu"])) @ ws_["wd"]
    assert (y - ref).norm() < 0.06 * ref.norm()
    assert torch.equal(y, blk.forward(xs, threads=3))
    # KV cache: fp32 rows give the plain attention, int8 rows stay close at a quarter of the bytes
    dim = 32
    cf, cq = CK.NativeKvCache(dim, 50), CK.NativeKvCache(dim, 50, quantized=True)
    K, V = torch.randn(50, dim, generator=g), torch.randn(50, dim, generator=g)
    for t in range(50):
        cf.append(K[t], V[t])
        cq.append(K[t], V[t])
    qq = torch.randn(dim, generator=g)
    want = torch.softmax((K @ qq) / math.sqrt(dim), 0) @ V
    assert torch.allclose(cf.attend(qq, block=8), want, atol=1e-5)
    assert (cq.attend(qq) - want).norm() < 0.05 * want.norm()
    assert cq.nbytes() < 0.3 * cf.nbytes() and len(cf) == 50
    with pytest.raises(MemoryError):
        cf.append(K[0], V[0])


def test_debug_allocator_poisons_payload_and_catches_a_write_past_the_end():
    from scirust_b200.ops import _lib
    t = _lib.fenced_empty((5, 3), torch.float32, "cpu", tag="probe")
    assert torch.isnan(t).all() and t.is_contiguous() and t.data_ptr() % 16 == 0
    b = _lib.fenced_empty((7,), torch.bfloat16, "cpu")
    assert torch.isnan(b.float()).all()
    _lib.check_canaries()
    t.fill_(1.0)                                           # a well-behaved writer leaves the fences alone
    _lib.check_canaries()
    # what a kernel that runs one element past its output does, made on the host: the byte after the payload
    past = torch.empty(0, dtype=torch.uint8).set_(t.untyped_storage())   # the backing buffer: fence | payload | fence
    past[256 + 5 * 3 * 4] = 0
    with pytest.raises(_lib.NativeError, match="past the end.*probe"):
        _lib.check_canaries()
    del t, b, past
    _lib._fenced.clear()


def test_certified_transform_pairs_round_trip_within_their_certificates():
    import math
    import random
    from scirust_b200.numerics import certified as CN
    rng = random.Random(0)

    def ulp(x):
        return math.ulp(abs(x)) if x != 0 else math.ulp(0.0)
    cases = [(CN.Log(), 1e-6, 1e6), (CN.Log1p(), -0.9, 1e6), (CN.SignedLog(), -1e6, 1e6), (CN.Power(0.25), 1e-8, 1e8),
             (CN.MuLaw(255.0), -1.0, 1.0), (CN.Logit(), 1e-6, 0.999), (CN.Anscombe(), 0.5, 1e6)]
    for pair, lo, hi in cases:
        iv = CN.Interval(lo, hi)
        bound = pair.roundtrip_bound(iv).ulps
        for _ in range(400):
            x = rng.uniform(lo, hi) if lo < 0 else math.exp(rng.uniform(math.log(lo), math.log(hi)))
            if x == 0.0:
                continue
            back = pair.decode(pair.encode(x))
            assert abs(back - x) <= bound * ulp(x), (type(pair).__name__, x, back, bound)
            assert pair.kappa_rt(x) <= pair.kappa_rt_sup(iv) * (1 + 1e-12)
    assert CN.Log().encode(-1.0) is None and CN.Anscombe().invalid_at(1e-17) and not CN.Anscombe().invalid_at(1.0)
    assert CN.Power(0.5).roundtrip_bound(CN.Interval(1e-12, 1.0)).ulps > CN.Power(0.5).roundtrip_bound(CN.Interval(0.5, 1.0)).ulps


def test_certificate_driven_summation_picks_the_cheapest_sound_method():
    import math
    import random
    from scirust_b200.numerics import certified as CN
    rng = random.Random(1)
    easy = [rng.uniform(0.5, 1.5) for _ in range(1000)]
    sel = CN.select_sum(easy, 1e-9)
    assert sel.method == "naive" and abs(sel.value - math.fsum(easy)) <= sel.cert_rel_bound * abs(math.fsum(easy))
    big = [rng.uniform(0.5, 1.5) for _ in range(200000)]
    assert CN.select_sum(big, 1e-13).method in ("pairwise", "neumaier")
    hard = [1e16, 1.0, -1e16, 1e-3] * 50                  # catastrophic cancellation: condition ~ 1e18
    sel = CN.select_sum(hard, 1e-9)
    assert sel.method == "expansion" and sel.value == math.fsum(hard) and sel.condition > 1e15
    assert CN.sum_klein(hard) == math.fsum(hard)           # second-order compensation survives what first-order cannot
    assert CN.sum_expansion(hard) == math.fsum(hard) and CN.sum_condition([1.0, -1.0]) == math.inf
    xs = [rng.gauss(0, 1) for _ in range(5000)]
    for f in (CN.sum_neumaier, CN.sum_klein, CN.sum_pairwise, CN.sum_expansion):
        assert abs(f(xs) - math.fsum(xs)) <= 1e-12


def test_a_priori_rational_proofs_hold_and_the_kernels_meet_them():
    import math
    from fractions import Fraction
    from scirust_b200.numerics import formal as FP
    assert Fraction(math.log(2)) < FP.ln2_upper() < Fraction(math.log(2)) + Fraction(1, 2 ** 50)
    assert Fraction(math.pi) < FP.pi_upper() < Fraction(math.pi) + Fraction(1, 2 ** 40)
    for proof in (FP.prove_exp(), FP.prove_cos(), FP.prove_sin()):
        assert proof.holds(), proof.name
        assert proof.relative_bound > 0 and isinstance(proof.relative_bound, Fraction)
    # a degree-5 polynomial fails the exp proof: the threshold is not vacuous
    FP.EXP_DEGREE, keep = 5, FP.EXP_DEGREE
    try:
        assert not FP.prove_exp().holds()
    finally:
        FP.EXP_DEGREE = keep
    # the float64 kernels stay inside the proven relative bound on their ranges (measured against the host libm)
    lim = float(FP.THRESHOLD)
    for i in range(-200, 201):
        r = i / 200 * (math.log(2) / 2)
        assert abs(FP.exp_kernel(r) - math.exp(r)) <= lim * math.exp(r)
        q = i / 200 * (math.pi / 4)
        assert abs(FP.cos_kernel(q) - math.cos(q)) <= lim * math.cos(q)
        assert abs(FP.sin_kernel(q) - math.sin(q)) <= lim * abs(math.sin(q)) + 1e-300
    for x in (-50.0, -3.3, -1e-9, 0.0, 0.7, 12.5, 88.0):
        assert abs(FP.exp_portable(x) - math.exp(x)) <= 4e-16 * math.exp(x)
    assert FP.exp_portable(1000.0) == math.inf and FP.exp_portable(-1000.0) == 0.0


def test_elastic_bpe_kernels_match_the_rank_priority_oracle_and_autotune_keeps_semantics():
    import random
    from scirust_b200 import tokenizer_elastic as ET
    A, B, C, AB, BC, AA = 10, 11, 12, 21, 20, 30
    o = ET.CanonicalBpeOracle([(B, C, BC), (A, B, AB)])
    assert o.encode_ids([A, B, C]) == [A, BC]                  # rank beats left-to-right order
    assert ET.CanonicalBpeOracle([(A, A, AA)]).encode_ids([A, A, A]) == [AA, A]      # left-most occurrence on ties
    with pytest.raises(ET.DuplicateMergeRule):
        ET.CanonicalBpeOracle([(1, 2, 3), (1, 2, 4)])
    th = ET.ElasticThresholds(16, 64, 256, 1024, 4096)
    assert [th.classify(n) for n in (0, 16, 17, 65, 257, 1025, 4097)] == ["S", "S", "M", "L", "XL", "XXL", "XXXL"]
    with pytest.raises(ValueError):
        ET.ElasticThresholds(16, 16, 256, 1024, 4096)
    # a random merge table over bytes: every kernel reproduces the oracle on pieces of every class
    rng = random.Random(3)
    merges, next_id, seen = [], 256, set()
    pool = list(range(97, 105))
    while len(merges) < 300:
        l, r = rng.choice(pool), rng.choice(pool)
        if (l, r) in seen:
            continue
        seen.add((l, r))
        merges.append((l, r, next_id))
        pool.append(next_id)
        next_id += 1
    oracle = ET.CanonicalBpeOracle(merges)
    cases = {cls: [[rng.randrange(97, 105) for _ in range(n)] for _ in range(6)]
             for cls, n in zip(ET.CLASSES, (9, 40, 150, 600, 1500, 4200))}
    for cls, pieces in cases.items():
        for p in pieces[:2 if cls in ("XXL", "XXXL") else 6]:
            want = oracle.encode_ids(p)
            for name in ("tiny_scan", "indexed", "heap"):
                assert oracle.kernel(name)(p) == want, (cls, name)
    assert oracle.encode_heap([]) == [] and oracle.encode_indexed([97]) == [97]
    # the auto-tuner: picks per class, never a kernel that disagrees with the oracle
    small = {c: cases[c][:3] for c in ("S", "M", "L")}
    rep = ET.autotune(oracle, small, th, repeats=3)
    assert rep.profile.kernels[3:] == ("reference",) * 3 and all(k in ET.KERNELS for k in rep.profile.kernels)
    broken = ET.CanonicalBpeOracle(merges)
    broken.encode_heap = lambda ids: list(ids)                 # a fast kernel that is wrong
    rep2 = ET.autotune(broken, small, th, repeats=2)
    assert all("heap" in rep2.rejected[c] for c in small) and "heap" not in rep2.profile.kernels
    # two different profiles, identical ids
    t1 = ET.ElasticTokenizer(merges, ET.ElasticProfile.reference_only(th))
    t2 = ET.ElasticTokenizer(merges, rep.profile)
    data = bytes(rng.randrange(97, 105) for _ in range(500))
    assert t1.encode_bytes(data) == t2.encode_bytes(data) == ET.ElasticTokenizer(merges).encode_bytes(data)

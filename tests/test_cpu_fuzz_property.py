"""Fuzz, property and cross-process determinism tests (the reference's fuzz targets and determinism gate:
fuzz/fuzz_targets/*.rs, docs/TEST_PROTOCOL.md:103-119): parsers answer damaged input with ValueError, never with a
crash or a stray exception; tape gradients agree with finite differences on random graphs; determinism-tagged
computations give the same signature in two separate processes."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FUZZ = settings(max_examples=150, deadline=None, suppress_health_check=list(HealthCheck))


def _mutations(blob: bytes):
    """A strategy of damaged variants of a valid file: truncations, byte flips, splices of random bytes."""
    n = len(blob)
    trunc = st.integers(0, n).map(lambda k: blob[:k])
    flip = st.lists(st.tuples(st.integers(0, n - 1), st.integers(0, 255)), min_size=1, max_size=8).map(
        lambda edits: bytes(_apply(bytearray(blob), edits)))
    splice = st.tuples(st.integers(0, n), st.binary(max_size=32)).map(lambda t: blob[:t[0]] + t[1] + blob[t[0]:])
    return st.one_of(trunc, flip, splice, st.binary(max_size=64))


def _apply(buf, edits):
    for i, v in edits:
        buf[i] = v
    return buf


def _only_value_error(fn, data):
    try:
        fn(data)
    except ValueError:
        pass                      # the contract: a typed refusal (KeyError-style lookups are wrapped by the parsers)


def _tiny_qmodel_bytes(A):
    """A valid QSR1 artefact: two quantised linear layers."""
    rng = np.random.default_rng(0)
    layers = [A.QLinear(4, 3, 0.05, True, rng.random(3, dtype=np.float32), rng.integers(-127, 127, 12).astype(np.int8),
                        rng.integers(-50, 50, 3).astype(np.int32)),
              A.QLinear(3, 2, 0.1, False, rng.random(2, dtype=np.float32), rng.integers(-127, 127, 6).astype(np.int8),
                        rng.integers(-50, 50, 2).astype(np.int32))]
    return A.QModel(layers).to_bytes()


def test_safetensors_parser_refuses_damaged_files_cleanly():
    from scirust_b200.io import safetensors as ST
    blob = ST.serialize({"w": torch.arange(12, dtype=torch.float32).reshape(3, 4), "b": torch.ones(3)},
                        metadata={"format": "pt"})
    assert set(ST.deserialize(blob)) == {"w", "b"}

    @FUZZ
    @given(_mutations(blob))
    def run(data):
        _only_value_error(ST.deserialize, data)
    run()


def test_srt1_qsr1_manifest_and_proof_parsers_refuse_damaged_input_cleanly():
    from scirust_b200.io import artifacts as A
    from scirust_b200.io import proof as P
    sd = {"layer.weight": torch.randn(4, 3), "layer.bias": torch.zeros(4)}
    srt = A.srt1_to_bytes(sd)
    assert set(A.srt1_from_bytes(srt)) == set(sd)
    manifest = A.write_manifest([A.LayerSpec("linear", (3, 4)), A.LayerSpec("relu"), A.LayerSpec("layernorm", (4, 1e-5))])
    assert len(A.parse_manifest(manifest)) == 3
    qblob = _tiny_qmodel_bytes(A)
    assert len(A.QModel.from_bytes(qblob).layers) == 2

    @FUZZ
    @given(_mutations(srt))
    def run_srt(data):
        _only_value_error(A.srt1_from_bytes, data)
    run_srt()
    if manifest:
        text = manifest.encode()

        @FUZZ
        @given(_mutations(text))
        def run_manifest(data):
            _only_value_error(lambda d: A.parse_manifest(d.decode("utf-8", errors="replace")), data)
        run_manifest()

    if qblob:
        @FUZZ
        @given(_mutations(qblob))
        def run_qsr(data):
            _only_value_error(A.QModel.from_bytes, data)
        run_qsr()

    @FUZZ
    @given(st.text(max_size=200))
    def run_proof(text):
        _only_value_error(P.parse_canonical, text)
    run_proof()


def test_onnx_json_and_tokenizer_json_refuse_damaged_input_cleanly():
    from scirust_b200.io import onnx_json as O
    from scirust_b200.tokenizer import BpeTokenizer, BpeTrainer
    from scirust_b200.nn import modules as M
    from scirust_b200.nn.rng import PcgEngine
    rng = PcgEngine(5)
    model = M.Sequential(M.Linear(4, 3, rng=rng), M.ReLU(), M.Linear(3, 2, rng=rng))
    text = O.export_sequential(model, "m", (-1, 4))
    g = O.import_onnx_json(text)
    assert O.run_graph(g, torch.ones(1, 4)).shape == (1, 2)
    tok = BpeTrainer(300, min_frequency=1).train(["hello hello world", "hello there"])
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        tok.save_json(os.path.join(d, "t.json"))
        tj = open(os.path.join(d, "t.json"), encoding="utf-8").read()

    @FUZZ
    @given(_mutations(text.encode()))
    def run_onnx(data):
        _only_value_error(lambda b: O.import_onnx_json(b.decode("utf-8", errors="replace")), data)
    run_onnx()

    @FUZZ
    @given(_mutations(tj.encode()))
    def run_tok(data):
        _only_value_error(lambda b: BpeTokenizer.from_json_str(b.decode("utf-8", errors="replace")), data)
    run_tok()


@settings(max_examples=40, deadline=None, suppress_health_check=list(HealthCheck))
@given(st.integers(0, 2 ** 31 - 1), st.lists(st.sampled_from(["add", "mul", "tanh", "sigmoid", "relu", "matmul", "exp"]),
                                             min_size=1, max_size=6))
def test_tape_gradients_match_finite_differences_on_random_graphs(seed, ops):
    """Property test over random op chains on the 2-D tape (fp64 finite differences as the oracle)."""
    from scirust_b200.autodiff.tape import Tape
    g = torch.Generator().manual_seed(seed)
    x0 = torch.randn(3, 3, generator=g, dtype=torch.float64) * 0.5
    w0 = torch.randn(3, 3, generator=g, dtype=torch.float64) * 0.5

    def build(xv, wv):
        tape = Tape()
        x, w = tape.input(xv.float()), tape.input(wv.float())
        h = x
        for op in ops:
            if op == "add":
                h = h + w
            elif op == "mul":
                h = h * w
            elif op == "matmul":
                h = h.matmul(w)
            elif op == "exp":
                h = h.scale(0.2).exp()
            else:
                h = getattr(h, op)()
        return tape, x, w, (h * h).sum()
    tape, x, w, loss = build(x0.clone(), w0.clone())
    tape.backward(loss)
    gx = tape.grad(x.idx).t.double()
    if not torch.isfinite(loss.t).all() or float(loss.t.detach().abs()) > 1e4:
        return                                                # a chain that overflows fp32 says nothing about gradients
    eps = 1e-3
    for (i, j) in [(0, 0), (1, 2), (2, 1)]:
        xp, xm = x0.clone(), x0.clone()
        xp[i, j] += eps
        xm[i, j] -= eps
        fp = _fp64_chain(xp, w0, ops)
        fm = _fp64_chain(xm, w0, ops)
        fd = (fp - fm) / (2 * eps)
        got = float(gx[i, j])
        if "relu" in ops and abs(fd - got) > 1e-2 * max(1.0, abs(fd)):
            continue                                          # a kink inside the +-eps stencil
        assert abs(fd - got) <= 2e-3 * max(1.0, abs(fd), abs(got)), (ops, i, j, fd, got)


def _fp64_chain(x, w, ops):
    """The same chain in float64 torch: the finite-difference oracle is not limited by the tape's fp32 storage."""
    h = x
    for op in ops:
        if op == "add":
            h = h + w
        elif op == "mul":
            h = h * w
        elif op == "matmul":
            h = h @ w
        elif op == "exp":
            h = (h * 0.2).exp()
        else:
            h = getattr(torch, op)(h)
    return float((h * h).sum())


_SIGNATURE_PROGRAM = r"""
import hashlib, sys, torch, numpy as np
sys.path.insert(0, %r)
from scirust_b200.models.mlp_cpu import train_gaussian_mlp
from scirust_b200.parallel.host_collectives import tree_all_reduce
from scirust_b200.numerics.reproducible import reproducible_sum
h = hashlib.sha256()
model, hist = train_gaussian_mlp(epochs=5, seed=7)
for k, v in sorted(model.state_dict_ref().items()):
    h.update(k.encode()); h.update(v.numpy().tobytes())
g = torch.Generator().manual_seed(3)
parts = [torch.randn(1000, generator=g).numpy() for _ in range(5)]
out = tree_all_reduce(parts, jitter_seed=int(sys.argv[1]) if len(sys.argv) > 1 else 0)
h.update(np.asarray(out[0]).tobytes())
h.update(np.float64(reproducible_sum(torch.randn(5000, generator=g).numpy())).tobytes())
print(h.hexdigest())
"""


def test_cross_process_determinism_gate():
    """The determinism-tagged computations (bit-pinned MLP, fixed-tree all-reduce over thread ranks, order-independent
    sum) print the same signature from two separate interpreter processes, with different thread counts."""
    prog = _SIGNATURE_PROGRAM % ROOT
    sigs = []
    for threads in ("1", "4"):
        env = dict(os.environ, OMP_NUM_THREADS=threads, MKL_NUM_THREADS=threads, PYTHONHASHSEED=threads)
        r = subprocess.run([sys.executable, "-c", prog, threads], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        sigs.append(r.stdout.strip().splitlines()[-1])
    assert sigs[0] == sigs[1] and len(sigs[0]) == 64

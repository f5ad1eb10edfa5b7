"""The reference's PyTorch-parity vectors (tests/parity/fixtures/*.json: inputs, expected outputs and expected input
gradients for an upstream gradient ``gout``) replayed through THIS framework's tape, N-D tape, einsum, sparse and
low-precision code. Skipped when the reference tree is not mounted (SCIRUST_REFERENCE_DIR or ../reference)."""
import json
import math
import os

import pytest
import torch

from scirust_b200 import einsum as ES
from scirust_b200 import sparse as SP
from scirust_b200.autodiff.nd import NdTape
from scirust_b200.autodiff.tape import Tape
from scirust_b200.numerics import lowprec

REF = os.environ.get("SCIRUST_REFERENCE_DIR") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
FIX = os.path.join(REF, "tests", "parity", "fixtures")
need_fixtures = pytest.mark.skipif(not os.path.isdir(FIX), reason="reference parity fixtures not mounted")

TOL = 2e-5


def _cases(rel):
    with open(os.path.join(FIX, rel)) as f:
        return json.load(f)["cases"]


def _t(values, shape=None):
    t = torch.tensor(values, dtype=torch.float32)
    return t.reshape(shape) if shape is not None else t


def _2d(t):
    return t.reshape(1, -1) if t.dim() <= 1 else t.reshape(t.shape[0], -1) if t.dim() > 2 else t


def _close(got, want, tol=TOL):
    dt = torch.float64 if tol < 1e-7 else torch.float32
    got, want = torch.as_tensor(got, dtype=dt).reshape(-1), torch.as_tensor(want, dtype=dt).reshape(-1)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert float((got - want).abs().max()) <= tol * (1 + float(want.abs().max())), (got, want)


def _run(build, inputs, gout):
    """inputs: name -> 2-D tensor. build(tape, vars) -> Var. Returns (y, {name: grad}) with loss = sum(y * gout)."""
    tape = Tape()
    v = {k: tape.input(t) for k, t in inputs.items()}
    y = build(tape, v)
    yv = tape.value(y.idx).t
    if gout is not None:
        tape.backward(y.mul(tape.constant(_t(gout).reshape(yv.shape))).sum())
    return yv, {k: tape.grad(x.idx).t for k, x in v.items()} if gout is not None else {}


UNARY = ["acos", "asin", "atan", "cos", "cosh", "exp", "gelu", "log", "log10", "neg", "reciprocal", "relu", "rsqrt", "sigmoid", "silu",
         "sin", "sinh", "sqrt", "tan", "tanh"]


@need_fixtures
@pytest.mark.parametrize("op", UNARY)
def test_elementwise_unary(op):
    for c in _cases(f"elementwise/{op}.json"):
        name = {"gelu": "gelu_tanh"}.get(op, op)                              # the vectors use the tanh form of GELU
        f = (lambda t, v: v["x"].sqrt().reciprocal()) if op == "rsqrt" else (lambda t, v: getattr(v["x"], name)())
        y, g = _run(f, {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"], 5e-5)


@need_fixtures
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "atan2"])
def test_elementwise_binary_and_broadcast(op):
    for c in _cases(f"elementwise/{op}.json"):
        y, g = _run(lambda t, v: getattr(v["x"], op)(v["b"]), {"x": _t(c["x"], c["shape"]), "b": _t(c["b"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])
        _close(g["b"], c["gb"])
    for c in _cases(f"elementwise_broadcast/{op}.json"):
        r, k = c["out_shape"]
        y, g = _run(lambda t, v: getattr(v["x"].broadcast_to(r, k), op)(v["b"].broadcast_to(r, k)),
                    {"x": _t(c["x"], c["shape"]), "b": _t(c["b"], c["b_shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])                                               # gradients are summed back over the broadcast axes
        _close(g["b"], c["gb"])


@need_fixtures
def test_pow_and_reductions():
    for c in _cases("elementwise/pow.json"):
        y, g = _run(lambda t, v: v["x"].pow(c["scalar"]), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"], 5e-5)
    table = {"sum": lambda x, a: x.sum_axis(a), "mean": lambda x, a: x.mean_axis(a), "var": lambda x, a: x.var_axis(a),
             "max": lambda x, a: x.max_axis(a), "norm": lambda x, a: x.mul(x).sum_axis(a).sqrt()}
    for op, fn in table.items():
        for c in _cases(f"reductions/{op}.json"):
            y, g = _run(lambda t, v: fn(v["x"], c["axis"]), {"x": _t(c["x"], c["shape"])}, c["gout"])
            _close(y, c["y"])
            _close(g["x"], c["gx"])


@need_fixtures
def test_normalisation_family():
    for op in ("softmax", "log_softmax"):
        for c in _cases(f"normalization/{op}.json"):
            y, g = _run(lambda t, v: getattr(v["x"], op)(), {"x": _t(c["x"], c["shape"])}, c["gout"])
            _close(y, c["y"])
            _close(g["x"], c["gx"])
    for c in _cases("normalization/layer_norm.json"):
        y, g = _run(lambda t, v: v["x"].layer_norm(v["w"], v["b"], c["eps"]),
                    {"x": _t(c["x"], c["shape"]), "w": _t(c["w"], [1, -1]), "b": _t(c["b"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        for k, want in (("x", "gx"), ("w", "gw"), ("b", "gb")):
            _close(g[k], c[want], 5e-5)
    for c in _cases("normalization/rms_norm.json"):
        y, g = _run(lambda t, v: v["x"].rms_norm(v["w"], c["eps"]), {"x": _t(c["x"], c["shape"]), "w": _t(c["w"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"], 5e-5)
        _close(g["w"], c["gw"], 5e-5)
    for c in _cases("normalization/batch_norm.json"):                          # inference mode: running statistics
        inv = 1.0 / torch.sqrt(_t(c["rv"]) + c["eps"])
        y, g = _run(lambda t, v: v["x"].sub_broadcast(t.constant(_t(c["rm"], [1, -1]))).mul_broadcast(t.constant(inv.reshape(1, -1)))
                    .mul_broadcast(v["w"]).add_bias(v["b"]), {"x": _t(c["x"], c["shape"]), "w": _t(c["w"], [1, -1]), "b": _t(c["b"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        for k, want in (("x", "gx"), ("w", "gw"), ("b", "gb")):
            _close(g[k], c[want], 5e-5)
    for c in _cases("normalization/dropout.json"):                             # the committed mask stands in for the generator
        keep = _t(c["mask"], c["shape"]) / (1.0 - c["p"])
        y, g = _run(lambda t, v: v["x"].mul(t.constant(keep)), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])
    for c in _cases("linear/normalize.json"):
        y, g = _run(lambda t, v: v["x"].l2_normalize(), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"], 5e-5)


@need_fixtures
def test_linear_family_and_losses():
    for c in _cases("linear/matmul.json"):
        k = c["shape"][1]
        y, g = _run(lambda t, v: v["a"].matmul(v["b"]), {"a": _t(c["a"], c["shape"]), "b": _t(c["b"], [k, -1])}, c["gout"])
        _close(y, c["y"])
        _close(g["a"], c["gx"])
        _close(g["b"], c["gb"])
    for c in _cases("linear/linear.json"):                                     # torch's weight is [out, in]: A . B^T
        out = c["out_shape"][1]
        y, g = _run(lambda t, v: v["x"].matmul_bt(v["w"]).add_bias(v["b"]),
                    {"x": _t(c["x"], c["shape"]), "w": _t(c["w"], [out, -1]), "b": _t(c["b"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        for k_, want in (("x", "gx"), ("w", "gw"), ("b", "gb")):
            _close(g[k_], c[want])
    for c in _cases("linear/bmm.json"):
        b_, m, k = c["shape"]
        tape = NdTape()
        a, b = tape.input(_t(c["a"], c["shape"])), tape.input(_t(c["b"], [b_, k, -1]))
        y = a.bmm(b)
        _close(tape.value(y), c["y"])
        grads = tape.backward(y.mul(tape.input(_t(c["gout"], c["out_shape"]), requires_grad=False)).sum())
        _close(grads[a.idx], c["gx"])
        _close(grads[b.idx], c["gb"])
    for c in _cases("linear/cosine_similarity.json"):
        y, g = _run(lambda t, v: v["a"].l2_normalize().mul(v["b"].l2_normalize()).sum_axis(1),
                    {"a": _t(c["a"], c["shape"]), "b": _t(c["b"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["a"], c["gx"], 5e-5)
        _close(g["b"], c["gb"], 5e-5)
    for c in _cases("loss/mse_loss.json"):
        y, g = _run(lambda t, v: v["x"].sub(t.constant(_t(c["target"], c["shape"]))).pow(2.0).mean(), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])
    for c in _cases("loss/cross_entropy.json"):
        rows, cols = c["shape"]
        onehot = torch.nn.functional.one_hot(torch.tensor(c["indices"]), cols).float()
        y, g = _run(lambda t, v: v["x"].log_softmax().mul(t.constant(onehot)).sum().scale(-1.0 / rows), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])


@need_fixtures
def test_convolution_pooling_attention_embedding():
    for c in _cases("convolution/conv2d.json"):
        n, ic, h, w = c["shape"]
        oc = c["out_shape"][1]
        assert c["kh"] == c["kw"]
        y, g = _run(lambda t, v: v["x"].conv2d(v["w"], v["b"], ic, h, w, c["kh"], 1, False),
                    {"x": _t(c["x"], [n, -1]), "w": _t(c["w"], [oc, -1]), "b": _t(c["b"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        for k_, want in (("x", "gx"), ("w", "gw"), ("b", "gb")):
            _close(g[k_], c[want], 5e-5)
    for op in ("max_pool2d", "avg_pool2d"):
        for c in _cases(f"convolution/{op}.json"):
            n, ch, h, w = c["shape"]
            y, g = _run(lambda t, v: getattr(v["x"], op)(ch, h, w, c["kernel"], c["kernel"]), {"x": _t(c["x"], [n, -1])}, c["gout"])
            _close(y, c["y"])
            _close(g["x"], c["gx"])
    for c in _cases("attention/scaled_dot_product_attention.json"):
        _, s, d = c["shape"]
        y, g = _run(lambda t, v: v["q"].flash_attention(v["k"], v["v"]), {"q": _t(c["a"], [s, d]), "k": _t(c["b"], [s, d]), "v": _t(c["c"], [s, d])}, c["gout"])
        _close(y, c["y"], 5e-5)
        for k_, want in (("q", "gx"), ("k", "gk"), ("v", "gv")):
            _close(g[k_], c[want], 1e-4)
    for c in _cases("indexing/embedding.json"):
        d = c["out_shape"][-1]
        y, g = _run(lambda t, v: v["w"].embedding(c["indices"]), {"w": _t(c["w"], [-1, d])}, c["gout"])
        _close(y, c["y"])
        _close(g["w"], c["gw"])                                               # repeated indices accumulate


@need_fixtures
def test_shape_operations():
    def check(c, build, inputs=None):
        y, g = _run(build, inputs or {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        return g
    for c in _cases("shape/transpose.json") + _cases("shape/permute.json"):
        assert sorted(c["dims"]) == [0, 1]
        swapped = list(c["out_shape"]) == list(c["shape"])[::-1] and c["out_shape"] != c["shape"] or c["dims"] == [1, 0]
        _close(check(c, lambda t, v: v["x"].transpose() if swapped else v["x"])["x"], c["gx"])
    for c in _cases("shape/reshape.json"):
        rows = c["new_shape"][0] if len(c["new_shape"]) == 2 else 1           # the tape is 2-D: other ranks are compared flat
        _close(check(c, lambda t, v: v["x"].reshape(rows, -1))["x"], c["gx"])
    for c in _cases("shape/flatten.json"):
        _close(check(c, lambda t, v: v["x"].reshape(1, -1))["x"], c["gx"])
    for c in _cases("shape/slice.json"):
        _close(check(c, lambda t, v: v["x"].slice_rows(c["start"], c["end"]) if c["axis"] == 0 else v["x"].slice_cols(c["start"], c["end"]))["x"], c["gx"])
    for c in _cases("shape/broadcast_to.json"):
        _close(check(c, lambda t, v: v["x"].broadcast_to(*c["bcast_to"]))["x"], c["gx"])
    for c in _cases("shape/cat.json"):
        g = check(c, lambda t, v: type(v["a"]).concat_rows([v["a"], v["b"]]) if c["dims"] == [0] else type(v["a"]).concat_cols([v["a"], v["b"]]),
                  {"a": _t(c["a"], c["shape"]), "b": _t(c["b"], c["shape"])})
        _close(g["a"], c["gx"])
        _close(g["b"], c["gb"])


@need_fixtures
def test_rope_fake_quantisation_einsum_bf16_and_sparse():
    for c in _cases("positional/rope.json"):
        tape = NdTape()
        x = tape.input(_t(c["x"], c["shape"]))                                # the vectors are (position, head, dim)
        y = x.permute([1, 0, 2]).rope(c["base"]).permute([1, 0, 2])            # the tape rotates over (..., position, dim)
        _close(tape.value(y), c["y"])
        grads = tape.backward(y.mul(tape.input(_t(c["gout"], c["shape"]), requires_grad=False)).sum())
        _close(grads[x.idx], c["gx"])
    for c in _cases("quantization/fake_quantize_per_tensor.json"):
        lo, hi = (c["qmin"] - c["zp"]) * c["scale"], (c["qmax"] - c["zp"]) * c["scale"]
        bits = int(math.log2(c["qmax"] - c["qmin"] + 1))
        y, g = _run(lambda t, v: v["x"].fake_quantize_ste_range(lo, hi, bits), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])                                               # straight-through inside the range, zero outside
    for c in _cases("einsum/einsum.json"):
        ops = [_t(c[k], s) for k, s in zip(("x", "a", "b"), c["shapes"])]
        _close(ES.einsum(c["spec"], *ops), c["y"])
    for c in _cases("conversion/to_bf16.json"):
        _close(lowprec.to_bf16(_t(c["x"]).numpy()), c["y"], 0.0)
    for c in _cases("sparse/spmv.json"):
        a = SP.CsrTensor(c["values"], c["colidx"], c["rowptr"], c["n"], c["m"])   # the vectors are f64, the CSR type is f32
        _close(SP.spmm_dense(a, torch.tensor(c["x"]).reshape(c["m"], 1)), c["yv"], 1e-6)
        _close(SP.spmm_dense(a, torch.tensor(c["b"]).reshape(c["m"], -1)), c["ym"], 1e-6)


@need_fixtures
def test_special_functions_gather_unfold_conv1d_cholesky_and_sparse_solve():
    for op in ("lgamma", "digamma"):
        for c in _cases(f"special/{op}.json"):
            y, g = _run(lambda t, v: getattr(v["x"], op)(), {"x": _t(c["x"], c["shape"])}, c["gout"])
            _close(y, c["y"], 5e-5)
            _close(g["x"], c["gx"], 1e-4)
    for c in _cases("shape/gather.json"):
        y, g = _run(lambda t, v: v["x"].gather(c["axis"], c["indices"]), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])
    for c in _cases("shape/unfold.json"):
        y, g = _run(lambda t, v: v["x"].unfold(c["axis"], c["size"], c["step"]), {"x": _t(c["x"], c["shape"])}, c["gout"])
        _close(y, c["y"])
        _close(g["x"], c["gx"])                                               # overlapping windows add their gradients
    for c in _cases("convolution/conv1d.json"):
        n, ic, length = c["shape"]
        oc = c["out_shape"][1]
        y, g = _run(lambda t, v: v["x"].conv1d(v["w"], v["b"], ic, length, c["kernel"]),
                    {"x": _t(c["x"], [n, -1]), "w": _t(c["w"], [oc, -1]), "b": _t(c["b"], [1, -1])}, c["gout"])
        _close(y, c["y"])
        for k_, want in (("x", "gx"), ("w", "gw"), ("b", "gb")):
            _close(g[k_], c[want], 5e-5)
    for c in _cases("linalg/cholesky.json"):
        y, _ = _run(lambda t, v: v["a"].cholesky(), {"a": _t(c["a"], c["shape"])}, None)
        _close(y, c["y"], 5e-6)
    for c in _cases("sparse/solve.json"):
        n = c["n"]
        a = SP.CsrTensor.from_dense(torch.tensor(c["a"], dtype=torch.float64).reshape(n, n).float())
        _close(SP.solve(a, torch.tensor(c["b1"], dtype=torch.float64)), c["y1"], 1e-6)          # the CSR values are fp32
        _close(SP.solve(a, torch.tensor(c["b2"], dtype=torch.float64).reshape(n, -1)), c["y2"], 1e-6)


def test_error_paths_are_structured():
    """Malformed requests raise the framework's own error types with the offending sizes, not a backend exception."""
    from scirust_b200.autodiff.tape import TapeError
    t = Tape()
    x1, w1, b1 = t.input(torch.randn(1, 6)), t.input(torch.randn(2, 10)), t.input(torch.zeros(1, 2))
    with pytest.raises(TapeError, match="kernel 5 is larger"):
        x1.conv1d(w1, b1, 2, 3, 5)
    with pytest.raises(TapeError, match="kernel 3 is larger"):
        t.input(torch.randn(1, 4)).conv2d(t.input(torch.randn(1, 9)), None, 1, 2, 2, 3, 1, False)
    with pytest.raises(TapeError, match="not positive-definite"):
        t.input(torch.tensor([[-1.0]])).cholesky()
    with pytest.raises(TapeError, match="must be square"):
        t.input(torch.randn(2, 3)).cholesky()
    V = type(x1)
    assert V.concat_rows([t.input(torch.zeros(2, 3)), t.input(torch.zeros(1, 3))]).t.shape == (3, 3)     # unequal along the joined axis is fine
    with pytest.raises(TapeError, match="column counts differ"):
        V.concat_rows([t.input(torch.zeros(2, 3)), t.input(torch.zeros(1, 4))])
    with pytest.raises(ValueError, match="rows\\+1"):
        SP.CsrTensor([], [], [], 0, 0)
    with pytest.raises(ValueError, match="must have 3 rows"):
        SP.solve(SP.CsrTensor.from_dense(torch.eye(3)), torch.zeros(4))
    with pytest.raises(ValueError, match="dense operand"):
        SP.spmm_dense(SP.CsrTensor.from_dense(torch.eye(3)), torch.zeros(2, 1))
    with pytest.raises(ValueError, match="values.len"):
        SP.CsrTensor([1.0, 2.0], [0], [0, 2], 1, 2)
    assert ES.einsum("ij,ij->", torch.ones(2, 2), torch.ones(2, 2)).dim() == 0                               # a scalar result has rank zero
    assert t.input(torch.randn(1, 25)).avg_pool2d(1, 5, 5, 2, 2).t.shape == (1, 4)                           # the odd border is dropped

"""DiFR (verification despite nondeterministic summation order) and the length-checked enclave ABI."""
import numpy as np
import pytest
import torch

from scirust_b200.io import difr as D
from scirust_b200.io import enclave as E


def _layers(dims, seed):
    g = torch.Generator().manual_seed(seed)
    return [D.DifrLayer(torch.rand(a, b, generator=g) * 2 - 1, (torch.rand(b, generator=g) * 2 - 1) * 0.3) for a, b in zip(dims[:-1], dims[1:])]


def _honest_shuffled(layers, x, seed):
    """fp32 forward whose every dot product is summed in a random order, as another machine might."""
    g = torch.Generator().manual_seed(seed)
    h = x.clone()
    for li, l in enumerate(layers):
        out = torch.empty(l.out_f)
        for o in range(l.out_f):
            acc = torch.zeros((), dtype=torch.float32)
            for i in torch.randperm(l.in_f, generator=g).tolist():
                acc = acc + l.w[i, o] * h[i]
            out[o] = acc + l.b[o]
        h = out.clamp_min(0) if li + 1 < len(layers) else out
    return h


def test_difr_accepts_any_summation_order_and_rejects_tampering():
    layers = _layers([24, 32, 16, 5], 1)
    x = torch.rand(24, generator=torch.Generator().manual_seed(2)) * 2 - 1
    for seed in range(5):
        v = D.difr_verify(layers, x, _honest_shuffled(layers, x, seed))
        assert v.accepted and float((v.deviation / v.envelope).max()) < 0.5          # comfortably inside
    honest = _honest_shuffled(layers, x, 9)
    v = D.difr_verify(layers, x, honest)
    assert float(v.envelope.max()) < 1e-3 * float(v.reference.abs().max() + 1)       # the envelope is tiny
    tampered = honest.clone()
    tampered[2] += 10 * v.envelope[2]
    bad = D.difr_verify(layers, x, tampered)
    assert not bad.accepted and int((bad.deviation > bad.envelope).sum()) == 1
    assert not D.difr_verify(layers, x, torch.full((5,), float("nan"))).accepted
    # a batch of claims in one pass: only the tampered row is refused
    X = torch.rand(6, 24, generator=torch.Generator().manual_seed(3)) * 2 - 1
    Y = torch.stack([_honest_shuffled(layers, X[i], i) for i in range(6)])
    Y[4, 0] += 1e-2
    vb = D.difr_verify(layers, X, Y)
    assert not vb.accepted and vb.accepted_rows.tolist() == [True, True, True, True, False, True]
    one = D.difr_verify(layers, X[1], Y[1])
    assert torch.allclose(one.reference, vb.reference[1]) and torch.allclose(one.envelope, vb.envelope[1])
    # the plain library product is one more honest order
    h = X
    for li, l in enumerate(layers):
        h = h @ l.w + l.b
        h = h.clamp_min(0) if li + 1 < len(layers) else h
    assert D.difr_verify(layers, X, h).accepted
    with pytest.raises(ValueError):
        D.difr_verify(layers, torch.zeros(7), torch.zeros(5))


def test_enclave_abi_checks_every_length_before_touching_memory():
    w = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    x = np.array([[1, 0, 1]], dtype=np.float32)
    b = np.array([0.5, -0.5], dtype=np.float32)
    rt = E.EnclaveRuntime()
    assert rt.infer(w, x, b).tolist() == [[4.5, 9.5]] and rt.infer(w, x).tolist() == [[4.0, 10.0]]
    X = np.random.default_rng(0).standard_normal((7, 3)).astype(np.float32)
    assert np.allclose(rt.infer(w, X, b), X @ w.T + b, atol=1e-6) and E.abi_version() == 1
    lay = E.EnclaveLayout.new
    out = np.full(2, 7.0, dtype=np.float32)
    z5, z3 = np.zeros(5, np.float32), np.zeros(3, np.float32)
    call = lambda *a: E.raw_infer_v1(*a)
    assert call(1, z5, 5, z3, 3, out, 2, None, 0, lay(1, 3, 2, False)) == E.ERR_LENGTH          # weights one short
    assert call(1, w, 6, z3, 3, out, 1, None, 0, lay(1, 3, 2, False)) == E.ERR_LENGTH           # output too small
    assert call(1, w, 6, z3, 3, out, 2, None, 0, lay(1, 3, 2, True)) == E.ERR_LENGTH            # bias promised, none counted
    assert call(2, w, 6, z3, 3, out, 2, None, 0, lay(1, 3, 2, False)) == E.ERR_VERSION
    bad_flag = lay(1, 3, 2, False)
    bad_flag.has_bias = 3
    assert call(1, w, 6, z3, 3, out, 2, None, 0, bad_flag) == E.ERR_FLAG
    assert call(1, w, 6, z3, 3, out, 2, b, 0, lay(1, 3, 2, False)) == E.ERR_FLAG                # a bias pointer without the flag
    assert call(1, None, 6, z3, 3, out, 2, None, 0, lay(1, 3, 2, False)) == E.ERR_NULL
    huge = lay(2 ** 40, 2 ** 40, 1, False)
    assert call(1, w, 6, z3, 3, out, 2, None, 0, huge) == E.ERR_OVERFLOW
    buf = np.zeros(8, dtype=np.float32)
    assert call(1, buf[:6], 6, z3, 3, buf[4:6], 2, None, 0, lay(1, 3, 2, False)) == E.ERR_ALIAS  # output inside the weights
    assert out.tolist() == [7.0, 7.0]                                                            # nothing was written by any refusal
    assert E.legacy_infer(w, x, out, None, lay(1, 3, 2, False)) == E.ERR_LEGACY and out.tolist() == [7.0, 7.0]
    assert call(1, w, 6, x, 3, out, 2, None, 0, lay(1, 3, 2, False)) == E.OK and out.tolist() == [4.0, 10.0]
    empty = np.zeros(0, np.float32)
    assert call(1, empty, 0, empty, 0, empty, 0, None, 0, lay(0, 3, 0, False)) == E.OK           # nothing to do is not an error
    with pytest.raises(E.EnclaveError, match="length"):
        rt.infer(w, x, b, lay(1, 3, 3, True))
    with pytest.raises(ValueError):
        rt.infer(np.zeros(6, np.float32), x)

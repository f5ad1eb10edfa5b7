"""Quantum circuits (batched dense simulator, observables, three gradient methods, hybrid layer, MPS) and the tape ops
that complete the reference surface (tensor-train contraction, quantum expectations, portable ln / softmax, ...)."""
import math

import pytest
import torch

from scirust_b200 import quantum as Q
from scirust_b200.autodiff import Tape


def test_gates_states_and_observables():
    bell = Q.run_circuit(Q.Circuit(2).h(0).cnot(0, 1))[0]
    assert torch.allclose(bell.abs() ** 2, torch.tensor([0.5, 0, 0, 0.5]), atol=1e-6)
    n = 2
    assert float(Q.Observable([(0, "Z"), (1, "Z")]).expectation(bell[None], n)) == pytest.approx(1.0, abs=1e-6)
    assert float(Q.Observable([(0, "X"), (1, "X")]).expectation(bell[None], n)) == pytest.approx(1.0, abs=1e-6)
    assert float(Q.Observable([(0, "Y"), (1, "Y")]).expectation(bell[None], n)) == pytest.approx(-1.0, abs=1e-6)
    assert float(Q.Observable.z(0).expectation(bell[None], n)) == pytest.approx(0.0, abs=1e-6)
    # every gate keeps the norm; S^2 = Z, T^2 = S, Sdg / Tdg undo them, SWAP moves an excitation, CZ is symmetric
    c = Q.Circuit(3)
    for g in ("h", "x", "y", "z", "s", "sdg", "t", "tdg", "i"):
        c.push(g, 1)
    c.rx(0, 0.3).ry(1, -1.1).rz(2, 2.0).push("phase", 0, parameter=0.4).cnot(0, 2).cz(1, 2).push("swap", 0, 1)
    assert float((Q.run_circuit(c)[0].abs() ** 2).sum()) == pytest.approx(1.0, abs=1e-5)
    a = Q.run_circuit(Q.Circuit(1).h(0).push("s", 0).push("s", 0))[0]
    b = Q.run_circuit(Q.Circuit(1).h(0).push("z", 0))[0]
    assert torch.allclose(a, b, atol=1e-6)
    assert torch.allclose(Q.run_circuit(Q.Circuit(1).h(0).push("t", 0).push("tdg", 0))[0], Q.run_circuit(Q.Circuit(1).h(0))[0], atol=1e-6)
    sw = Q.run_circuit(Q.Circuit(2).x(0).push("swap", 0, 1))[0]
    assert sw.abs().argmax().item() == 1                                       # |10> -> |01> (qubit 0 is the high bit)
    assert torch.allclose(Q.run_circuit(Q.Circuit(2).h(0).h(1).cz(0, 1))[0], Q.run_circuit(Q.Circuit(2).h(0).h(1).cz(1, 0))[0])
    # Ry(theta)|0>: <Z> = cos(theta), <X> = sin(theta); a batch of angles advances together
    th = torch.linspace(-2, 2, 9)
    p = Q.ParameterId(0)
    st = Q.run_circuit(Q.Circuit(1).ry(0, p), {p: th}, batch=9)
    assert torch.allclose(Q.Observable.z(0).expectation(st, 1), torch.cos(th), atol=1e-6)
    assert torch.allclose(Q.Observable.x(0).expectation(st, 1), torch.sin(th), atol=1e-6)
    for bad in (lambda: Q.Circuit(0), lambda: Q.Circuit(2).push("h", 2), lambda: Q.Circuit(2).push("cnot", 1, 1),
                lambda: Q.Circuit(2).push("rx", 0), lambda: Q.Circuit(2).push("h", 0, parameter=0.1), lambda: Q.Circuit(2).push("foo", 0),
                lambda: Q.Circuit(1).rx(0, float("nan")), lambda: Q.run_circuit(Q.Circuit(1).ry(0, p)),
                lambda: Q.run_circuit(Q.Circuit(1).ry(0, p), {p: torch.zeros(3)}, batch=2),
                lambda: Q.Observable([]), lambda: Q.Observable([(0, "Z"), (0, "X")]), lambda: Q.Observable([(0, "W")]),
                lambda: Q.Observable.z(3).expectation(bell[None], 2)):
        with pytest.raises(Q.QuantumError):
            bad()


def test_three_gradient_methods_agree():
    a, b = Q.ParameterId(0), Q.ParameterId(1)
    c = Q.Circuit(2).ry(0, a).cnot(0, 1).rx(1, b).ry(0, a).rz(1, a)          # `a` occurs three times
    assert c.parameter_ids() == [a, b]
    bind = {a: 0.7, b: -0.4}
    for obs in (Q.Observable([(0, "Z"), (1, "X")]), Q.Observable.z(1), Q.Observable.y(0)):
        adj = Q.adjoint_gradients(c, obs, bind)
        for p in (a, b):
            shift = Q.parameter_shift_gradient(c, obs, bind, p)
            fd = Q.finite_difference_gradient(c, obs, bind, p)
            assert adj[p] == pytest.approx(shift, abs=1e-5) and shift == pytest.approx(fd, abs=2e-3)
    # closed form: d/dtheta <Z> after Ry(theta) = -sin(theta)
    c1, p = Q.Circuit(1).ry(0, a), a
    assert Q.parameter_shift_gradient(c1, Q.Observable.z(0), {a: 0.9}, p) == pytest.approx(-math.sin(0.9), abs=1e-6)


def test_quantum_layer_trains_through_the_tape():
    x_id, w0, w1 = Q.ParameterId(0), Q.ParameterId(1), Q.ParameterId(2)
    circ = Q.Circuit(2).ry(0, x_id).ry(1, w0).cnot(0, 1).ry(1, w1)
    layer = Q.QuantumLayer(circ, [Q.Observable.z(1), Q.Observable([(0, "Z"), (1, "Z")])], [x_id], [w0, w1])
    feats = torch.linspace(-1.5, 1.5, 16).reshape(-1, 1)
    target = layer.forward(feats, torch.tensor([[0.9, -1.3]]))[:, 0]            # reachable by construction
    params = torch.tensor([[0.1, -0.2]])
    losses = []
    for _ in range(150):
        t = Tape()
        f, p = t.constant(feats), t.input(params)
        out = f.quantum_expectations(p, layer)
        assert out.t.shape == (16, 2)
        loss = ((out.t[:, 0] - target) ** 2).mean()
        loss.backward()
        params = params - 0.3 * p.t.grad
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.05 * losses[0]
    # gradient of the layer against finite differences, and batched == one row at a time
    p0 = torch.tensor([[0.3, -0.7]], requires_grad=True)
    layer.forward(feats, p0)[:, 1].sum().backward()
    eps, fd = 1e-3, []
    for i in range(2):
        d = torch.zeros(1, 2)
        d[0, i] = eps
        fd.append(float((layer.forward(feats, p0.detach() + d)[:, 1].sum() - layer.forward(feats, p0.detach() - d)[:, 1].sum()) / (2 * eps)))
    assert torch.allclose(p0.grad[0], torch.tensor(fd), atol=2e-3)
    rows = torch.cat([layer.forward(feats[i:i + 1], p0.detach()) for i in range(16)])
    assert torch.allclose(rows, layer.forward(feats, p0.detach()), atol=1e-6)
    t = Tape()
    single = Q.QuantumLayer(circ, Q.Observable.z(1), [x_id], [w0, w1])
    assert t.constant(feats[:1]).quantum_expectation(t.input(params), single).t.shape == (1, 1)
    for bad in (lambda: t.constant(feats).quantum_expectation(t.input(params), single),
                lambda: t.constant(feats[:1]).quantum_expectation(t.input(params), layer),
                lambda: layer.forward(feats, torch.zeros(1, 3)), lambda: layer.forward(torch.zeros(0, 1), params),
                lambda: layer.forward(torch.zeros(4, 2), params), lambda: Q.QuantumLayer(circ, [], [x_id], [w0, w1]),
                lambda: Q.QuantumLayer(circ, Q.Observable.z(0), [x_id], [w0]), lambda: Q.QuantumLayer(circ, Q.Observable.z(0), [x_id, w0], [w0, w1])):
        with pytest.raises(Q.QuantumError):
            bad()


def test_matrix_product_state_matches_the_dense_simulator():
    m = Q.Mps.zero(4)
    m.apply_1qubit_gate(0, Q.gates.H)
    for q in range(3):
        m.apply_2qubit_gate(q, Q.gates.CNOT, 8)
    ghz = m.to_statevector()
    assert torch.allclose(ghz[[0, 15]], torch.full((2,), 2 ** -0.5), atol=1e-6) and float(ghz[1:15].abs().max()) < 1e-6
    assert m.max_bond() == 2 and m.norm_sqr() == pytest.approx(1.0, abs=1e-6) and m.amplitude([1, 1, 1, 1]) == pytest.approx(2 ** -0.5, abs=1e-6)
    assert m.storage() < 2 ** 4 * 2
    # a real circuit of Ry and CZ against the dense simulator
    torch.manual_seed(0)
    angles = (torch.rand(8) * 3).tolist()
    mps, dense = Q.Mps.zero(4), Q.Circuit(4)
    for layer in range(2):
        for q in range(4):
            mps.apply_1qubit_gate(q, Q.gates.ry(angles[layer * 4 + q]))
            dense.ry(q, angles[layer * 4 + q])
        for q in range(3):
            mps.apply_2qubit_gate(q, Q.gates.CZ, 16)
            dense.cz(q, q + 1)
    want = Q.run_circuit(dense)[0]
    assert float(want.imag.abs().max()) < 1e-6 and torch.allclose(mps.to_statevector(), want.real, atol=1e-5)
    # truncating the bond loses norm; a product state never needs more than bond 1
    cut = Q.Mps.zero(4)
    for q in range(4):
        cut.apply_1qubit_gate(q, Q.gates.ry(angles[q]))
    assert cut.max_bond() == 1
    for q in range(3):
        cut.apply_2qubit_gate(q, Q.gates.CZ, 1)
    assert cut.max_bond() == 1 and cut.norm_sqr() < 1.0
    with pytest.raises(Q.QuantumError):
        cut.apply_2qubit_gate(3, Q.gates.CZ, 2)


def test_tensor_train_contraction_on_the_tape():
    torch.manual_seed(0)
    in_d, out_d, ranks = [2, 3, 2], [2, 2, 3], [1, 3, 2, 1]
    cores = [torch.randn(ranks[k] * in_d[k] * out_d[k], ranks[k + 1]) for k in range(3)]
    g = [c.reshape(ranks[k], in_d[k], out_d[k], ranks[k + 1]) for k, c in enumerate(cores)]
    W = torch.einsum("aiob,bjpc,ckqd->ijkopq", *g).reshape(12, 12)
    t = Tape()
    x, cs, b = t.input(torch.randn(5, 12)), [t.input(c) for c in cores], t.input(torch.randn(1, 12))
    y = x.tt_contract(cs, b, in_d, out_d, ranks)
    assert torch.allclose(y.t, x.t @ W + b.t, atol=1e-5)
    y.t.pow(2).sum().backward()
    xr = x.t.detach().clone().requires_grad_(True)
    cr = [c.detach().clone().requires_grad_(True) for c in cores]
    gr = [c.reshape(ranks[k], in_d[k], out_d[k], ranks[k + 1]) for k, c in enumerate(cr)]
    ((xr @ torch.einsum("aiob,bjpc,ckqd->ijkopq", *gr).reshape(12, 12) + b.t.detach()) ** 2).sum().backward()
    assert torch.allclose(x.t.grad, xr.grad, atol=1e-4) and all(torch.allclose(a.t.grad, r.grad, atol=1e-4) for a, r in zip(cs, cr))
    assert x.tt_contract(cs, None, in_d, out_d, ranks).t.shape == (5, 12)
    from scirust_b200.autodiff.tape import TapeError
    for bad in (lambda: x.tt_contract(cs[:2], b, in_d, out_d, ranks), lambda: x.tt_contract(cs, b, in_d, out_d, [2, 3, 2, 1]),
                lambda: x.tt_contract(cs, b, [2, 3, 3], out_d, ranks), lambda: x.tt_contract([cs[0], cs[0], cs[2]], b, in_d, out_d, ranks)):
        with pytest.raises(TapeError):
            bad()


def test_remaining_tape_ops():
    from scirust_b200.autodiff.tape import TapeError
    from scirust_b200.numerics import portable
    t = Tape()
    a, b, c = t.input(torch.tensor([[1.0, -2.0, 0.5]])), t.input(torch.tensor([[0.5, 0.25, 4.0]])), t.input(torch.tensor([[2.0, 2.0, 2.0]]))
    assert torch.allclose(a.add_hadamard(b, c).t, a.t + b.t * c.t) and torch.allclose(a.sub_hadamard(b, c).t, a.t - b.t * c.t)
    assert torch.allclose(a.add_scaled(b, -3.0).t, a.t - 3 * b.t)
    assert torch.allclose(a.sinh().t, torch.sinh(a.t)) and torch.allclose(a.cosh().t, torch.cosh(a.t)) and torch.allclose(b.log10().t, torch.log10(b.t))
    assert a.broadcast_to(4, 3).t.shape == (4, 3) and t.zeros(2, 3).t.sum() == 0 and t.ones(2, 2).t.sum() == 4
    with pytest.raises(TapeError):
        a.broadcast_to(4, 5)
    d = a.mul(b).detach()
    assert not d.t.requires_grad and torch.equal(d.t, a.t * b.t)
    ln = b.ln_portable()
    assert ln.t.tolist()[0] == [float(portable.ln_f32(v)) for v in (0.5, 0.25, 4.0)]
    sm = a.softmax_portable()
    assert torch.allclose(sm.t, torch.softmax(a.t, 1), atol=1e-6) and float(sm.t.sum()) == pytest.approx(1.0, abs=1e-6)
    (ln.t.sum() + (sm.t * torch.tensor([[1.0, 2.0, 3.0]])).sum()).backward()
    ref_a = a.t.detach().clone().requires_grad_(True)
    (torch.softmax(ref_a, 1) * torch.tensor([[1.0, 2.0, 3.0]])).sum().backward()
    assert torch.allclose(b.t.grad, 1 / b.t.detach(), atol=1e-6) and torch.allclose(a.t.grad, ref_a.grad, atol=1e-6)
    t.clip_grad_value([a.idx, b.idx], 0.5)
    assert float(b.t.grad.abs().max()) <= 0.5
    x = t.input(torch.tensor([[-2.0, -0.3, 0.1, 0.52, 3.0]]))
    q = x.fake_quantize_ste_range(-1.0, 1.0, bits=2)                         # 4 levels: -1, -1/3, 1/3, 1
    assert torch.allclose(q.t, torch.tensor([[-1.0, -1 / 3, 1 / 3, 1 / 3, 1.0]]), atol=1e-6)
    q.t.sum().backward()
    assert x.t.grad.tolist() == [[0.0, 1.0, 1.0, 1.0, 0.0]]                   # straight through inside the range only
    with pytest.raises(TapeError):
        x.fake_quantize_ste_range(1.0, 1.0)

"""Variational circuit builder, readouts and training session (CPU)."""
import math

import pytest
import torch

from scirust_b200 import quantum as Q
from scirust_b200 import vqnet as V


def test_builder_allocates_parameters_and_topologies():
    b = V.VariationalCircuitBuilder(4)
    h = b.angle_encoding("y", [0, 1, 2, 3])
    assert len(h) == 4 and len(b.inputs) == 4
    b.hardware_efficient_ansatz(2)
    assert len(b.trainable) == 2 * 2 * 4
    assert b.entangling_pairs("none") == []
    assert b.entangling_pairs("linear") == [(0, 1), (1, 2), (2, 3)]
    assert b.entangling_pairs("ring")[-1] == (3, 0)
    assert len(b.entangling_pairs("full")) == 6
    two = V.VariationalCircuitBuilder(2)
    assert two.entangling_pairs("ring") == [(0, 1)]          # no duplicate edge on two qubits
    with pytest.raises(Q.QuantumError):
        b.angle_encoding("x", [0, 0])
    with pytest.raises(Q.QuantumError):
        b.variational_ansatz(0, ["y"])
    with pytest.raises(Q.QuantumError):
        b.build()                                             # nothing measured


def test_reupload_reuses_inputs_and_changes_the_function():
    def make(reupload):
        b = V.VariationalCircuitBuilder(2)
        h = b.angle_encoding("y", [0, 1])
        b.variational_ansatz(1, ["y", "z"], "linear", "cnot")
        if reupload:
            b.reupload_angle_encoding("y", h)
        b.measure_all_z()
        return b.build(seed=3)
    a, r = make(False), make(True)
    assert a.input_parameter_count() == r.input_parameter_count() == 2
    x = torch.tensor([[0.3, -0.7]])
    assert not torch.allclose(a(x), r(x))


def test_basis_probabilities_match_the_state_vector():
    b = V.VariationalCircuitBuilder(3)
    b.angle_encoding("x", [0, 1, 2])
    b.variational_ansatz(2, ["y", "z"], "ring", "cz")
    b.measure_computational_basis_moments()
    vc = b.build(seed=1)
    ro = V.ComputationalBasisReadout.from_circuit(vc)
    assert (ro.moment_count(), ro.probability_count()) == (7, 8)
    x = torch.randn(4, 3)
    p = ro.apply(vc(x))
    assert torch.allclose(p.sum(1), torch.ones(4), atol=1e-5) and float(p.min()) > -1e-6
    bind = {pid: x[:, i] for i, pid in enumerate(vc.layer.input_parameters)}
    bind.update({pid: vc.theta[0, i] for i, pid in enumerate(vc.layer.trainable_parameters)})
    direct = Q.run_circuit(vc.circuit, bind, 4).abs() ** 2
    z0 = vc(x)[:, 0]                                           # <Z_0> = P(q0=0) - P(q0=1), bit 0 of the state index
    q0 = p[:, [s for s in range(8) if not s & 1]].sum(1) - p[:, [s for s in range(8) if s & 1]].sum(1)
    assert torch.allclose(z0, q0, atol=1e-5)
    assert torch.allclose(p.sort(dim=1).values, direct.sort(dim=1).values, atol=1e-5)
    with pytest.raises(Q.QuantumError):
        V.ComputationalBasisReadout(3, [Q.Observable.z(0)])


def test_hamiltonian_readout_is_a_linear_map_of_expectations():
    b = V.VariationalCircuitBuilder(2)
    b.angle_encoding("y", [0, 1])
    b.hardware_efficient_ansatz(1)
    zz = Q.Observable([Q.PauliTerm(0, "Z"), Q.PauliTerm(1, "Z")])
    b.measure_z([0, 1]).measure(zz)
    vc = b.build(seed=5)
    h1 = V.Hamiltonian([V.HamiltonianTerm(0.5, Q.Observable.z(0)), V.HamiltonianTerm(-1.5, zz)], offset=0.25)
    h2 = V.Hamiltonian([V.HamiltonianTerm(2.0, Q.Observable.z(1))])
    ro = V.HamiltonianReadout.from_observables(vc.observables, [h1, h2])
    x = torch.randn(3, 2)
    e = vc(x)
    out = vc.forward_hamiltonians(x, ro)
    assert torch.allclose(out[:, 0], 0.5 * e[:, 0] - 1.5 * e[:, 2] + 0.25, atol=1e-6)
    assert torch.allclose(out[:, 1], 2.0 * e[:, 1], atol=1e-6)
    with pytest.raises(Q.QuantumError):
        V.HamiltonianReadout(vc.observables, [V.Hamiltonian([V.HamiltonianTerm(1.0, Q.Observable.x(0))])])
    with pytest.raises(Q.QuantumError):
        V.HamiltonianTerm(math.inf, zz)


def test_training_session_minimises_an_energy_and_rejects_non_finite_loss():
    b = V.VariationalCircuitBuilder(2)
    b.angle_encoding("y", [0, 1])
    b.variational_ansatz(2, ["y", "z"], "linear", "cnot")
    zz = Q.Observable([Q.PauliTerm(0, "Z"), Q.PauliTerm(1, "Z")])
    b.measure_z([0, 1]).measure(zz)
    vc = b.build(seed=2)
    ro = V.HamiltonianReadout(vc.observables, [V.Hamiltonian([V.HamiltonianTerm(1.0, Q.Observable.z(0)),
                                                                 V.HamiltonianTerm(1.0, Q.Observable.z(1)),
                                                                 V.HamiltonianTerm(0.5, zz)])])
    x = torch.zeros(1, 2)
    sess = V.TrainingSession(torch.optim.Adam(vc.parameters(), lr=0.1))
    loss_fn = lambda e, _t: ro.apply(e).mean()
    first = sess.train_step(vc, loss_fn, x, None)
    rep = None
    for ep in range(60):
        rep = sess.train_epoch(vc, loss_fn, [(x, None)], epoch=ep)
    assert rep.last.loss < first.loss - 0.5 and rep.last.loss < -1.3       # ground energy is -1.5 at |11>
    assert rep.batches == 1 and sess.steps == 61 and first.gradient_norm > 0
    before = vc.theta.detach().clone()
    with pytest.raises(Q.QuantumError):
        sess.train_step(vc, lambda e, _t: e.sum() * float("nan"), x, None)
    assert torch.equal(before, vc.theta.detach())


def _hybrid(seed=0):
    b = V.VariationalCircuitBuilder(1)
    b.angle_encoding("y", [0])
    b.variational_ansatz(1, ["y", "z"], "none")
    b.measure_z([0])
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(2, 1), b.build(seed=seed), torch.nn.Linear(1, 1))


def test_quantum_module_composes_with_classical_layers_state_round_trips_and_trains_from_a_loader():
    model = _hybrid()
    x = torch.randn(6, 2, generator=torch.Generator().manual_seed(1))
    out = model(x)
    assert out.shape == (6, 1)
    out.sum().backward()
    assert all(p.grad is not None and bool(torch.isfinite(p.grad).all()) for p in model.parameters())   # gradients cross the circuit
    state = model.state_dict()
    assert "1.theta" in state and state["1.theta"].shape == (1, 2)                                       # the circuit's angles are ordinary state
    other = _hybrid(seed=9)
    assert not torch.allclose(other(x), model(x))
    other.load_state_dict(state)
    assert torch.equal(other(x), model(x))
    bad = dict(state)
    bad["1.theta"] = torch.zeros(1, 3)
    with pytest.raises(RuntimeError):
        other.load_state_dict(bad)
    with pytest.raises(Q.QuantumError):
        model[1](torch.zeros(4, 3))                                                                      # wrong feature count: the circuit's own error
    target = torch.sin(x[:, :1] + 0.5 * x[:, 1:])
    data = torch.utils.data.DataLoader(torch.utils.data.TensorDataset(x, target), batch_size=3, shuffle=False)
    opt = torch.optim.Adam(model.parameters(), lr=0.05)
    sess = V.TrainingSession(opt)
    first = sess.train_epoch(model, torch.nn.functional.mse_loss, data, epoch=0)
    for ep in range(1, 40):
        last = sess.train_epoch(model, torch.nn.functional.mse_loss, data, epoch=ep)
    assert first.batches == 2 and last.mean_loss < 0.5 * first.mean_loss and sess.steps == 80
    import copy
    opt_state = copy.deepcopy(opt.state_dict())                                                          # as a checkpoint on disk would hold it
    resumed, ropt = _hybrid(seed=3), None
    resumed.load_state_dict(model.state_dict())
    ropt = torch.optim.Adam(resumed.parameters(), lr=0.05)
    ropt.load_state_dict(opt_state)
    a = V.TrainingSession(opt).train_epoch(model, torch.nn.functional.mse_loss, data)
    b2 = V.TrainingSession(ropt).train_epoch(resumed, torch.nn.functional.mse_loss, data)
    assert a.mean_loss == b2.mean_loss and torch.equal(model[1].theta, resumed[1].theta)                  # exact resume

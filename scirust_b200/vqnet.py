"""Building blocks for variational hybrid quantum / classical models on top of ``scirust_b200.quantum``.

``VariationalCircuitBuilder`` owns parameter allocation, so encodings and ansatz layers compose without the caller
juggling ids: ``angle_encoding`` (one input angle per qubit on a chosen axis), ``reupload_angle_encoding`` (the same
inputs encoded again later in the circuit), ``hardware_efficient_ansatz`` (per layer: Ry on every qubit, Rz on every
qubit, a CNOT chain), ``variational_ansatz`` (chosen rotation axes, entangling gate CNOT / CZ, topology none / linear /
ring / full: ring closes the chain only from three qubits up, full takes every unordered pair once in lexicographic
order), then ``measure`` / ``measure_z`` / ``measure_all_z`` / ``measure_computational_basis_moments``.
``VariationalCircuit`` is a ``torch.nn.Module`` (its trainable angles are a parameter, seeded uniform in [-pi, pi)), so it
trains with any optimizer and moves to a GPU with ``.to``; a batch of feature rows is simulated at once.
Readouts: ``HamiltonianReadout`` (weighted sums of measured Pauli observables plus offsets, a fixed linear map) and
``ComputationalBasisReadout`` (the Walsh-Hadamard projection from the complete set of Z-product moments to the 2^n
basis-state probabilities). ``TrainingSession`` runs steps / epochs and reports losses and gradient norms.
Reference counterpart: scirust-core/src/vqnet.rs and scirust-core/src/vqnet/{ansatz,encoding,readout,probability,
nn_module,trainer,module_state,optimizer_state,loader_training}.rs.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass

import torch

from . import quantum as Q
from .nn.rng import PcgEngine

AXES = {"x": "rx", "y": "ry", "z": "rz"}
MAX_PROBABILITY_QUBITS = 10


class VariationalCircuit(torch.nn.Module):
    def __init__(self, layer: Q.QuantumLayer, seed: int = 0):
        super().__init__()
        self.layer = layer
        n = len(layer.trainable_parameters)
        init = (PcgEngine(seed).fill_uniform_signed((1, n), math.pi) if n else torch.zeros(1, 0))
        self.theta = torch.nn.Parameter(init)

    @property
    def circuit(self):
        return self.layer.circuit

    @property
    def observables(self):
        return self.layer.observables

    def input_parameter_count(self) -> int:
        return len(self.layer.input_parameters)

    def trainable_parameter_count(self) -> int:
        return len(self.layer.trainable_parameters)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        """``[batch, inputs]`` (or one row) -> ``[batch, observables]``."""
        x = features if features.dim() == 2 else features.reshape(1, -1)
        return self.layer.forward(x.to(self.theta.device), self.theta)

    forward_batch = forward

    def forward_hamiltonians(self, features, readout: "HamiltonianReadout") -> torch.Tensor:
        return readout.apply(self.forward(features))


class VariationalCircuitBuilder:
    def __init__(self, num_qubits: int):
        self.circuit = Q.Circuit(num_qubits)
        self.observables: list = []
        self.inputs: list = []
        self.trainable: list = []
        self._next = 0

    def num_qubits(self) -> int:
        return self.circuit.num_qubits

    def _alloc(self, bucket) -> Q.ParameterId:
        p = Q.ParameterId(self._next)
        self._next += 1
        bucket.append(p)
        return p

    def _distinct(self, qubits):
        if len(set(qubits)) != len(qubits):
            raise Q.QuantumError("qubits must be distinct")
        if any(not 0 <= q < self.num_qubits() for q in qubits):
            raise Q.QuantumError("qubit index out of range")

    def angle_encoding(self, axis: str, qubits) -> "AngleEncodingHandle":
        self._distinct(qubits)
        params = []
        for q in qubits:
            p = self._alloc(self.inputs)
            self.circuit.push(AXES[axis], q, parameter=p)
            params.append(p)
        return AngleEncodingHandle(tuple(qubits), tuple(params))

    def reupload_angle_encoding(self, axis: str, handle: "AngleEncodingHandle") -> "VariationalCircuitBuilder":
        """Encode the SAME input features again (data re-uploading): no new input parameters."""
        for q, p in zip(handle.qubits, handle.parameters):
            self.circuit.push(AXES[axis], q, parameter=p)
        return self

    def hardware_efficient_ansatz(self, layers: int) -> "VariationalCircuitBuilder":
        if layers == 0:
            raise Q.QuantumError("hardware-efficient ansatz needs at least one layer")
        n = self.num_qubits()
        for _ in range(layers):
            for kind in ("ry", "rz"):
                for q in range(n):
                    self.circuit.push(kind, q, parameter=self._alloc(self.trainable))
            for c in range(n - 1):
                self.circuit.push("cnot", c, c + 1)
        return self

    def entangling_pairs(self, topology: str) -> list:
        n = self.num_qubits()
        if topology == "none":
            return []
        chain = [(q, q + 1) for q in range(n - 1)]
        if topology == "linear":
            return chain
        if topology == "ring":
            return chain + ([(n - 1, 0)] if n >= 3 else [])
        if topology == "full":
            return list(itertools.combinations(range(n), 2))
        raise Q.QuantumError(f"unknown entanglement topology {topology!r}")

    def variational_ansatz(self, layers: int, rotations, topology: str = "linear", entangler: str = "cnot") -> "VariationalCircuitBuilder":
        if layers == 0:
            raise Q.QuantumError("variational ansatz needs at least one layer")
        if not rotations:
            raise Q.QuantumError("variational ansatz needs at least one rotation axis")
        if entangler not in ("cnot", "cz"):
            raise Q.QuantumError("entangling gate is cnot or cz")
        pairs = self.entangling_pairs(topology)
        for _ in range(layers):
            for axis in rotations:
                for q in range(self.num_qubits()):
                    self.circuit.push(AXES[axis], q, parameter=self._alloc(self.trainable))
            for a, b in pairs:
                self.circuit.push(entangler, a, b)
        return self

    def measure(self, observable: Q.Observable) -> "VariationalCircuitBuilder":
        if any(t.qubit >= self.num_qubits() for t in observable.terms):
            raise Q.QuantumError("observable acts on a qubit the circuit does not have")
        self.observables.append(observable)
        return self

    def measure_z(self, qubits) -> "VariationalCircuitBuilder":
        self._distinct(qubits)
        self.observables += [Q.Observable.z(q) for q in qubits]
        return self

    def measure_all_z(self) -> "VariationalCircuitBuilder":
        return self.measure_z(list(range(self.num_qubits())))

    def measure_computational_basis_moments(self) -> "VariationalCircuitBuilder":
        """Every non-empty product of Z operators, in ascending binary-mask order (bit q = Z on qubit q)."""
        n = self.num_qubits()
        if n > MAX_PROBABILITY_QUBITS:
            raise Q.QuantumError(f"the probability readout is limited to {MAX_PROBABILITY_QUBITS} qubits")
        self.observables += z_moment_basis(n)
        return self

    def build(self, seed: int = 0) -> VariationalCircuit:
        if not self.observables:
            raise Q.QuantumError("a variational circuit needs at least one observable")
        return VariationalCircuit(Q.QuantumLayer(self.circuit, self.observables, self.inputs, self.trainable), seed)


@dataclass(frozen=True)
class AngleEncodingHandle:
    qubits: tuple
    parameters: tuple

    def __len__(self):
        return len(self.qubits)


def z_moment_basis(n: int) -> list:
    return [Q.Observable([Q.PauliTerm(q, "Z") for q in range(n) if (mask >> q) & 1]) for mask in range(1, 1 << n)]


# ------------------------------------------------------------------ readouts
@dataclass(frozen=True)
class HamiltonianTerm:
    coefficient: float
    observable: Q.Observable

    def __post_init__(self):
        if not math.isfinite(self.coefficient):
            raise Q.QuantumError("Hamiltonian coefficients must be finite")


class Hamiltonian:
    def __init__(self, terms, offset: float = 0.0):
        terms = list(terms)
        if not terms:
            raise Q.QuantumError("a Hamiltonian needs at least one term")
        if not math.isfinite(offset):
            raise Q.QuantumError("the Hamiltonian offset must be finite")
        self.terms, self.offset = terms, float(offset)


def _obs_key(o: Q.Observable):
    return tuple(sorted((t.qubit, t.pauli) for t in o.terms))


class HamiltonianReadout:
    """``energies = expectations @ M + offsets`` where ``M [observables, hamiltonians]`` holds the coefficients; every
    Hamiltonian term must be one of the measured observables."""

    def __init__(self, observables, hamiltonians):
        self.observables = list(observables)
        index = {_obs_key(o): i for i, o in enumerate(self.observables)}
        if len(index) != len(self.observables):
            raise Q.QuantumError("measured observables must be distinct")
        hs = list(hamiltonians)
        if not hs:
            raise Q.QuantumError("a readout needs at least one Hamiltonian")
        self.matrix = torch.zeros(len(self.observables), len(hs))
        self.offsets = torch.zeros(len(hs))
        for j, h in enumerate(hs):
            self.offsets[j] = h.offset
            for t in h.terms:
                k = _obs_key(t.observable)
                if k not in index:
                    raise Q.QuantumError("a Hamiltonian term is not among the measured observables")
                self.matrix[index[k], j] += t.coefficient

    @staticmethod
    def from_observables(observables, hamiltonians) -> "HamiltonianReadout":
        return HamiltonianReadout(observables, hamiltonians)

    def observable_count(self) -> int:
        return self.matrix.shape[0]

    def hamiltonian_count(self) -> int:
        return self.matrix.shape[1]

    def apply(self, expectations: torch.Tensor) -> torch.Tensor:
        if expectations.shape[-1] != self.matrix.shape[0]:
            raise Q.QuantumError(f"expected {self.matrix.shape[0]} expectations per row, got {expectations.shape[-1]}")
        return expectations @ self.matrix.to(expectations.device) + self.offsets.to(expectations.device)


class ComputationalBasisReadout:
    """Probabilities of the 2^n basis states (state index bit q = qubit q measured as 1) from the complete set of
    Z-product moments: ``p_s = 2^-n * (1 + sum_mask (-1)^{popcount(s & mask)} <Z_mask>)``: a fixed linear map."""

    def __init__(self, num_qubits: int, observables):
        if not 1 <= num_qubits <= MAX_PROBABILITY_QUBITS:
            raise Q.QuantumError(f"the probability readout supports 1..{MAX_PROBABILITY_QUBITS} qubits")
        want = [_obs_key(o) for o in z_moment_basis(num_qubits)]
        if [_obs_key(o) for o in observables] != want:
            raise Q.QuantumError("the observables must be every non-empty Z product in ascending mask order")
        n = num_qubits
        s = torch.arange(1 << n)[:, None]
        m = torch.arange(1, 1 << n)[None, :]
        par = torch.zeros_like(s & m)
        v = s & m
        while bool(v.any()):
            par ^= v & 1
            v = v >> 1
        self.walsh = ((1.0 - 2.0 * par.float()) / (1 << n)).t().contiguous()          # [moments, states]
        self.bias = 1.0 / (1 << n)
        self.num_qubits = n

    @staticmethod
    def from_circuit(circuit: VariationalCircuit) -> "ComputationalBasisReadout":
        return ComputationalBasisReadout(circuit.circuit.num_qubits, circuit.observables)

    def moment_count(self) -> int:
        return self.walsh.shape[0]

    def probability_count(self) -> int:
        return self.walsh.shape[1]

    def apply(self, moments: torch.Tensor) -> torch.Tensor:
        if moments.shape[-1] != self.walsh.shape[0]:
            raise Q.QuantumError(f"expected {self.walsh.shape[0]} moments per row, got {moments.shape[-1]}")
        return moments @ self.walsh.to(moments.device) + self.bias


# ------------------------------------------------------------------ training
@dataclass
class TrainStepReport:
    step: int
    loss: float
    gradient_norm: float


@dataclass
class EpochReport:
    epoch: int
    batches: int
    mean_loss: float
    last: TrainStepReport | None


class TrainingSession:
    """Steps and epochs of ``loss_fn(model(features), targets)`` with any torch optimizer; non-finite losses or gradients
    stop the step BEFORE the optimizer moves the parameters."""

    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.steps = 0

    def train_step(self, model, loss_fn, features, targets) -> TrainStepReport:
        self.optimizer.zero_grad()
        loss = loss_fn(model(features), targets)
        if not bool(torch.isfinite(loss)):
            raise Q.QuantumError("training loss is not finite")
        loss.backward()
        sq = 0.0
        for group in self.optimizer.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    sq += float(p.grad.double().pow(2).sum())
        if not math.isfinite(sq):
            raise Q.QuantumError("gradient is not finite")
        self.optimizer.step()
        self.steps += 1
        return TrainStepReport(self.steps, float(loss.detach()), math.sqrt(sq))

    def train_epoch(self, model, loss_fn, batches, epoch: int = 0) -> EpochReport:
        total, n, last = 0.0, 0, None
        for features, targets in batches:
            last = self.train_step(model, loss_fn, features, targets)
            total += last.loss
            n += 1
        return EpochReport(epoch, n, total / n if n else math.nan, last)

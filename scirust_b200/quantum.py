"""Quantum circuit simulation for hybrid models: a typed circuit IR, a dense state-vector simulator that runs a whole
BATCH of parameter bindings at once, Pauli-string observables, exact gradients three ways, the hybrid layer and its tape
op, and a matrix-product-state simulator with bond truncation.

* ``Circuit``: qubit count plus an ordered list of operations (I, H, X, Y, Z, S, Sdg, T, Tdg, Rx / Ry / Rz / PhaseShift with
  a fixed angle or a ``ParameterId``, CNOT, CZ, SWAP); targets are checked when an operation is pushed.
* Simulator: the state is a complex64 tensor ``[batch, 2, ..., 2]`` (qubit 0 = most significant index); a gate is one
  tensor contraction over its axis, with a per-sample 2x2 matrix when its angle is a batched parameter. On a GPU all
  samples of a batch advance together: the natural shape of the work for a wide machine.
* ``Observable``: a product of X / Y / Z on distinct qubits; expectation ``<psi| P |psi>`` (real).
* Gradients: autograd through the simulator (the exact adjoint of every contraction: the default of ``QuantumLayer``),
  ``parameter_shift_gradient`` (two evaluations per occurrence of a parameter at +-pi/2: exact for these gates) and
  ``finite_difference_gradient`` (the sanity check).
* ``QuantumLayer``: ``classical_features [batch, n_inputs]`` and ``parameters [1, n_trainable]`` -> ``[batch, n_observables]``;
  ``Var.quantum_expectations`` records it on a tape.
* ``Mps``: left-to-right matrix product state with real amplitudes; one-qubit gates are local, two-qubit gates on
  neighbours contract, apply and split again by SVD keeping at most ``max_chi`` singular values.

Reference counterparts: scirust-core/src/quantum/{ir,dense,complex_gates,observable,gradient,hybrid,backend}.rs,
scirust-core/src/quantum.rs:50-290 (MPS) and the tape op scirust-core/src/autodiff/reverse.rs:3644-3800.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


class QuantumError(ValueError):
    pass


@dataclass(frozen=True)
class ParameterId:
    value: int


FIXED_GATES = ("i", "h", "x", "y", "z", "s", "sdg", "t", "tdg")
ROTATIONS = ("rx", "ry", "rz", "phase")
TWO_QUBIT = ("cnot", "cz", "swap")


@dataclass(frozen=True)
class Operation:
    kind: str
    qubits: tuple
    parameter: object = None          # float | ParameterId for rotations


def _c(re, im=0.0):
    return complex(re, im)


_S2 = 1.0 / math.sqrt(2.0)
_FIXED = {
    "i": [[1, 0], [0, 1]], "h": [[_S2, _S2], [_S2, -_S2]], "x": [[0, 1], [1, 0]], "y": [[0, -1j], [1j, 0]],
    "z": [[1, 0], [0, -1]], "s": [[1, 0], [0, 1j]], "sdg": [[1, 0], [0, -1j]],
    "t": [[1, 0], [0, complex(_S2, _S2)]], "tdg": [[1, 0], [0, complex(_S2, -_S2)]],
}


class Circuit:
    def __init__(self, num_qubits: int):
        if not 1 <= num_qubits <= 24:
            raise QuantumError("a dense circuit needs between 1 and 24 qubits")
        self.num_qubits = num_qubits
        self.operations: list = []

    def push(self, kind: str, *qubits: int, parameter=None) -> "Circuit":
        kind = kind.lower()
        if kind not in FIXED_GATES + ROTATIONS + TWO_QUBIT:
            raise QuantumError(f"unknown gate {kind!r}")
        need = 2 if kind in TWO_QUBIT else 1
        if len(qubits) != need:
            raise QuantumError(f"{kind} acts on {need} qubit(s)")
        if any(not 0 <= q < self.num_qubits for q in qubits):
            raise QuantumError(f"qubit index out of range for {self.num_qubits} qubits")
        if need == 2 and qubits[0] == qubits[1]:
            raise QuantumError("a two-qubit gate needs two different qubits")
        if kind in ROTATIONS:
            if parameter is None:
                raise QuantumError(f"{kind} needs an angle or a parameter")
            if not isinstance(parameter, ParameterId) and not math.isfinite(float(parameter)):
                raise QuantumError("a fixed angle must be finite")
        elif parameter is not None:
            raise QuantumError(f"{kind} takes no parameter")
        self.operations.append(Operation(kind, tuple(qubits), parameter))
        return self

    # fluent helpers
    def h(self, q): return self.push("h", q)
    def x(self, q): return self.push("x", q)
    def rx(self, q, p): return self.push("rx", q, parameter=p)
    def ry(self, q, p): return self.push("ry", q, parameter=p)
    def rz(self, q, p): return self.push("rz", q, parameter=p)
    def cnot(self, c, t): return self.push("cnot", c, t)
    def cz(self, c, t): return self.push("cz", c, t)

    def parameter_ids(self) -> list:
        seen, out = set(), []
        for op in self.operations:
            if isinstance(op.parameter, ParameterId) and op.parameter not in seen:
                seen.add(op.parameter)
                out.append(op.parameter)
        return out


def _rotation(kind: str, theta: torch.Tensor) -> torch.Tensor:
    """``theta [B]`` (real) -> ``[B, 2, 2]`` complex64."""
    h = theta * 0.5
    c, s = torch.cos(h).to(torch.complex64), torch.sin(h).to(torch.complex64)
    z = torch.zeros_like(c)
    if kind == "rx":
        m = [[c, -1j * s], [-1j * s, c]]
    elif kind == "ry":
        m = [[c, -s], [s, c]]
    elif kind == "rz":
        e = torch.exp(-1j * h.to(torch.complex64))
        m = [[e, z], [z, e.conj()]]
    else:                                   # phase shift: diag(1, e^{i theta})
        m = [[torch.ones_like(c), z], [z, torch.exp(1j * theta.to(torch.complex64))]]
    return torch.stack([torch.stack(r, -1) for r in m], -2)


def _apply_1q(state: torch.Tensor, mat: torch.Tensor, q: int) -> torch.Tensor:
    """state [B, 2...]; mat [2, 2] or [B, 2, 2]; acts on axis q + 1."""
    st = state.movedim(q + 1, -1)
    out = torch.einsum("ij,...j->...i", mat, st) if mat.dim() == 2 else torch.einsum("bij,b...j->b...i", mat, st)
    return out.movedim(-1, q + 1)


def _apply_2q(state: torch.Tensor, kind: str, a: int, b: int) -> torch.Tensor:
    st = state.movedim((a + 1, b + 1), (-2, -1))
    if kind == "cnot":
        st = torch.stack([st[..., 0, :], st[..., 1, :].flip(-1)], -2)
    elif kind == "cz":
        sign = torch.ones(2, 2, dtype=st.dtype, device=st.device)
        sign[1, 1] = -1
        st = st * sign
    else:
        st = st.transpose(-2, -1)
    return st.movedim((-2, -1), (a + 1, b + 1))


def run_circuit(circuit: Circuit, bindings=None, batch: int = 1, device="cpu") -> torch.Tensor:
    """Final states ``[batch, 2^n]``. ``bindings`` maps every ``ParameterId`` of the circuit to a float or to a real
    tensor of ``batch`` angles (differentiable)."""
    bindings = bindings or {}
    n = circuit.num_qubits
    missing = [p for p in circuit.parameter_ids() if p not in bindings]
    if missing:
        raise QuantumError(f"unbound parameter {missing[0].value}")
    state = torch.zeros((batch,) + (2,) * n, dtype=torch.complex64, device=device)
    state[(slice(None),) + (0,) * n] = 1.0
    for op in circuit.operations:
        if op.kind in TWO_QUBIT:
            state = _apply_2q(state, op.kind, *op.qubits)
        elif op.kind in FIXED_GATES:
            state = _apply_1q(state, torch.tensor(_FIXED[op.kind], dtype=torch.complex64, device=device), op.qubits[0])
        else:
            v = bindings[op.parameter] if isinstance(op.parameter, ParameterId) else op.parameter
            theta = torch.as_tensor(v, dtype=torch.float32, device=device).reshape(-1)
            if theta.numel() not in (1, batch):
                raise QuantumError(f"a batched angle needs {batch} values, got {theta.numel()}")
            if not bool(torch.isfinite(theta).all()):
                raise QuantumError("angles must be finite")
            state = _apply_1q(state, _rotation(op.kind, theta.expand(batch)), op.qubits[0])
    return state.reshape(batch, -1)


@dataclass(frozen=True)
class PauliTerm:
    qubit: int
    pauli: str               # "X" | "Y" | "Z"


class Observable:
    def __init__(self, terms):
        terms = [t if isinstance(t, PauliTerm) else PauliTerm(*t) for t in terms]
        if not terms:
            raise QuantumError("a Pauli observable needs at least one factor")
        if len({t.qubit for t in terms}) != len(terms):
            raise QuantumError("a qubit appears twice in one observable")
        if any(t.pauli not in "XYZ" or len(t.pauli) != 1 for t in terms):
            raise QuantumError("Pauli factors are X, Y or Z")
        self.terms = terms

    @staticmethod
    def x(q): return Observable([PauliTerm(q, "X")])
    @staticmethod
    def y(q): return Observable([PauliTerm(q, "Y")])
    @staticmethod
    def z(q): return Observable([PauliTerm(q, "Z")])

    def expectation(self, states: torch.Tensor, num_qubits: int) -> torch.Tensor:
        """Real expectation of every state of the batch: ``[batch]``."""
        if any(t.qubit >= num_qubits for t in self.terms):
            raise QuantumError("observable acts on a qubit the circuit does not have")
        B = states.shape[0]
        psi = states.reshape((B,) + (2,) * num_qubits)
        phi = psi
        for t in self.terms:
            m = torch.tensor(_FIXED[t.pauli.lower()], dtype=torch.complex64, device=states.device)
            phi = _apply_1q(phi, m, t.qubit)
        return (psi.conj() * phi).reshape(B, -1).sum(1).real


def expectation_value(circuit: Circuit, observable: Observable, bindings=None) -> float:
    return float(observable.expectation(run_circuit(circuit, bindings), circuit.num_qubits)[0])


def finite_difference_gradient(circuit, observable, bindings, parameter: ParameterId, step: float = 1e-3) -> float:
    hi, lo = dict(bindings), dict(bindings)
    hi[parameter] = float(bindings[parameter]) + step
    lo[parameter] = float(bindings[parameter]) - step
    return (expectation_value(circuit, observable, hi) - expectation_value(circuit, observable, lo)) / (2 * step)


def parameter_shift_gradient(circuit, observable, bindings, parameter: ParameterId) -> float:
    """Exact for Rx / Ry / Rz / PhaseShift: each OCCURRENCE of the parameter is shifted by +-pi/2 on its own."""
    total = 0.0
    for k, op in enumerate(circuit.operations):
        if op.parameter != parameter:
            continue
        vals = []
        for sign in (1.0, -1.0):
            c = Circuit(circuit.num_qubits)
            c.operations = list(circuit.operations)
            c.operations[k] = Operation(op.kind, op.qubits, float(bindings[parameter]) + sign * math.pi / 2)
            vals.append(expectation_value(c, observable, bindings))
        total += 0.5 * (vals[0] - vals[1])
    return total


def adjoint_gradients(circuit, observable, bindings) -> dict:
    """All parameter gradients from ONE forward and one reverse sweep (autograd through the contractions)."""
    ids = circuit.parameter_ids()
    leaves = {p: torch.tensor(float(bindings[p]), requires_grad=True) for p in ids}
    e = observable.expectation(run_circuit(circuit, leaves), circuit.num_qubits)[0]
    grads = torch.autograd.grad(e, [leaves[p] for p in ids], allow_unused=True)
    return {p: (0.0 if g is None else float(g)) for p, g in zip(ids, grads)}


class QuantumLayer:
    """``input_parameters`` are fed per sample from the classical features, ``trainable_parameters`` are shared weights."""

    def __init__(self, circuit: Circuit, observables, input_parameters, trainable_parameters):
        obs = list(observables) if isinstance(observables, (list, tuple)) else [observables]
        if not obs:
            raise QuantumError("a quantum layer needs at least one observable")
        self.circuit, self.observables = circuit, obs
        self.input_parameters, self.trainable_parameters = list(input_parameters), list(trainable_parameters)
        both = self.input_parameters + self.trainable_parameters
        if len(set(both)) != len(both):
            raise QuantumError("a parameter is listed twice")
        if set(circuit.parameter_ids()) - set(both):
            raise QuantumError("the circuit has a parameter that is neither an input nor trainable")

    def forward(self, features: torch.Tensor, parameters: torch.Tensor) -> torch.Tensor:
        if features.dim() != 2 or features.shape[0] == 0 or features.shape[1] != len(self.input_parameters):
            raise QuantumError(f"classical_features must be [batch >= 1, {len(self.input_parameters)}], got {tuple(features.shape)}")
        if tuple(parameters.shape) != (1, len(self.trainable_parameters)):
            raise QuantumError(f"quantum_parameters must be [1, {len(self.trainable_parameters)}], got {tuple(parameters.shape)}")
        B = features.shape[0]
        bind = {p: features[:, i] for i, p in enumerate(self.input_parameters)}
        bind.update({p: parameters[0, i] for i, p in enumerate(self.trainable_parameters)})
        states = run_circuit(self.circuit, bind, B, features.device)
        return torch.stack([o.expectation(states, self.circuit.num_qubits) for o in self.observables], 1)

    __call__ = forward


# ------------------------------------------------------------------ matrix product states
class Mps:
    """Real-amplitude MPS: site tensors ``A_k [dl, 2, dr]``; |0...0> initially (all bonds 1)."""

    def __init__(self, tensors):
        self.tensors = list(tensors)

    @staticmethod
    def zero(n_qubits: int) -> "Mps":
        t = torch.zeros(1, 2, 1)
        t[0, 0, 0] = 1.0
        return Mps([t.clone() for _ in range(n_qubits)])

    def num_qubits(self) -> int:
        return len(self.tensors)

    def max_bond(self) -> int:
        return max(max(t.shape[0], t.shape[2]) for t in self.tensors)

    def storage(self) -> int:
        return sum(t.numel() for t in self.tensors)

    def apply_1qubit_gate(self, q: int, gate) -> None:
        g = torch.as_tensor(gate, dtype=torch.float32).reshape(2, 2)
        self.tensors[q] = torch.einsum("pq,lqr->lpr", g, self.tensors[q])

    def apply_2qubit_gate(self, q: int, gate, max_chi: int) -> None:
        """Gate on qubits (q, q + 1), row-major ``(q1 q2) x (p1 p2)``; the bond is cut to ``max_chi``."""
        if not 0 <= q < len(self.tensors) - 1:
            raise QuantumError("two-qubit MPS gates act on neighbours q, q + 1")
        g = torch.as_tensor(gate, dtype=torch.float32).reshape(2, 2, 2, 2)
        a, b = self.tensors[q], self.tensors[q + 1]
        theta = torch.einsum("lpm,mqr->lpqr", a, b)
        theta = torch.einsum("abpq,lpqr->labr", g, theta)
        dl, dr = a.shape[0], b.shape[2]
        u, s, vh = torch.linalg.svd(theta.reshape(dl * 2, 2 * dr), full_matrices=False)
        keep = max(1, min(max_chi, int((s > 1e-12 * s[0]).sum()) if s[0] > 0 else 1))
        self.tensors[q] = u[:, :keep].reshape(dl, 2, keep)
        self.tensors[q + 1] = (s[:keep, None] * vh[:keep]).reshape(keep, 2, dr)

    def amplitude(self, bits) -> float:
        v = torch.ones(1)
        for t, b in zip(self.tensors, bits):
            v = v @ t[:, int(b), :]
        return float(v[0])

    def to_statevector(self) -> torch.Tensor:
        v = torch.ones(1, 1)
        for t in self.tensors:
            v = torch.einsum("xl,lpr->xpr", v, t).reshape(-1, t.shape[2])
        return v[:, 0]

    def norm_sqr(self) -> float:
        env = torch.ones(1, 1)
        for t in self.tensors:
            env = torch.einsum("ab,apc,bpd->cd", env, t, t)
        return float(env[0, 0])


class gates:
    """Real one- and two-qubit matrices (row-major) for the MPS simulator."""
    H = [_S2, _S2, _S2, -_S2]
    X = [0.0, 1.0, 1.0, 0.0]
    Z = [1.0, 0.0, 0.0, -1.0]
    I = [1.0, 0.0, 0.0, 1.0]
    CNOT = [1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 0, 1, 0, 0, 1, 0]
    CZ = [1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0, 0, 0, 0, -1]

    @staticmethod
    def ry(theta: float):
        c, s = math.cos(theta / 2), math.sin(theta / 2)
        return [c, -s, s, c]

"""Command-line front ends for the symbolic / numeric core and the MPS circuit simulator: ``diff simplify eval solve prove
gradient to-rust to-cuda regress trig patterns integrate root minimize optimize linsolve lstsq det cholesky qr cg polyroots
ode inverse solve-system fem-heat sat symreg quantum``. Matrices are written ``"a,b;c,d"`` (rows separated by ``;``),
vectors ``"a,b,c"``; exit status 0 = done (``prove``: proved), 1 = negative answer, 2 = usage or input error.
Reference counterpart: scirust-cli/src/{symbolic,numeric,reasoning}.rs and ``run_quantum`` of scirust-cli/src/learning.rs.
"""
from __future__ import annotations

import math
import sys

import torch


def _matrix(s: str) -> torch.Tensor:
    rows = [[float(v) for v in r.split(",")] for r in s.split(";") if r.strip()]
    if not rows or any(len(r) != len(rows[0]) for r in rows):
        raise ValueError("matrix rows must have the same length")
    return torch.tensor(rows, dtype=torch.float64)


def _vector(s: str) -> torch.Tensor:
    return torch.tensor([float(v) for v in s.split(",")], dtype=torch.float64)


def _bindings(items) -> dict:
    out = {}
    for it in items:
        k, _, v = it.partition("=")
        if not k or not v:
            raise ValueError(f"bindings look like x=1.5, got {it!r}")
        out[k] = float(v)
    return out


def _fmt(v: float) -> str:
    return f"{v:.12g}"


def _show_matrix(name: str, m: torch.Tensor) -> None:
    print(f"{name} =")
    for row in m.tolist():
        print("  [" + ", ".join(f"{v: .8g}" for v in row) + "]")


def _guard(fn):
    def run(a):
        from .symbolic import SymbolicError
        try:
            return fn(a) or 0
        except (SymbolicError, ValueError, ZeroDivisionError, RuntimeError) as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
    return run


def cmd_diff(a):
    from . import symbolic as S
    print(S.to_string(S.diff(a.expr, a.var)))


def cmd_simplify(a):
    from . import symbolic as S
    print(S.simplify_str(a.expr))


def cmd_eval(a):
    from . import symbolic as S
    print(_fmt(float(S.evaluate(a.expr, _bindings(a.bindings)))))


def cmd_solve(a):
    from . import symbolic as S
    roots = S.solve(a.expr, a.var)
    if not roots:
        print("no real solution found")
        return 1
    print(f"{a.var} = " + ", ".join(_fmt(r) for r in roots))


def cmd_prove(a):
    from . import symbolic as S
    ok, how = S.prove_equal(a.lhs, a.rhs)
    print(("proved: " if ok else "not equal: " if "differ" in how else "") + how)
    return 0 if ok else 1


def cmd_gradient(a):
    from . import symbolic as S
    point = _bindings(a.bindings)
    for k, v in S.gradient(a.expr, point).items():
        print(f"d/d{k} = {_fmt(v)}")


def cmd_to_rust(a):
    from . import symbolic as S
    print(S.to_rust(a.expr))


def cmd_to_cuda(a):
    from . import symbolic as S
    print(S.to_cuda(a.expr))


def cmd_regress(a):
    from . import symbolic as S
    co, r2 = S.polyfit(_vector(a.xs), _vector(a.ys), a.degree)
    print("y = " + " + ".join(f"{c:.8g}" + ("" if i == 0 else "*x" if i == 1 else f"*x^{i}") for i, c in enumerate(co)))
    print(f"R^2 = {r2:.8f}")


def cmd_patterns(a):
    from . import symbolic as S
    found = S.discover_patterns(_vector(a.series).tolist())
    print("patterns: " + ", ".join(found) if found else "no dominant pattern detected")


def cmd_integrate(a):
    from . import symbolic as S
    print(_fmt(S.integrate(a.expr, a.a, a.b, a.var, a.method)))


def cmd_root(a):
    from . import symbolic as S
    print(_fmt(S.find_root(a.expr, a.a, a.b, a.var, a.method)))


def cmd_minimize(a):
    from . import symbolic as S
    x, fx = S.minimize_1d(a.expr, a.a, a.b, a.var)
    print(f"{a.var} = {_fmt(x)}  f = {_fmt(fx)}")


def cmd_optimize(a):
    from . import symbolic as S
    vars_ = a.vars.split(",") if a.vars else None
    pt, fx, it = S.optimize(a.expr, [float(v) for v in a.start.split(",")], vars_)
    print(", ".join(f"{k} = {_fmt(v)}" for k, v in pt.items()) + f"  f = {_fmt(fx)}  ({it} iterations)")


def cmd_linsolve(a):
    x = torch.linalg.solve(_matrix(a.matrix), _vector(a.rhs))
    print("x = [" + ", ".join(_fmt(v) for v in x.tolist()) + "]")


def cmd_lstsq(a):
    m, b = _matrix(a.matrix), _vector(a.rhs)
    if m.shape[0] < m.shape[1]:
        raise ValueError("need at least as many rows as columns")
    x = torch.linalg.lstsq(m, b[:, None]).solution[:, 0]
    print("x = [" + ", ".join(_fmt(v) for v in x.tolist()) + "]")
    print(f"residual norm = {_fmt(float((m @ x - b).norm()))}")


def cmd_det(a):
    print(_fmt(float(torch.linalg.det(_matrix(a.matrix)))))


def cmd_cholesky(a):
    m = _matrix(a.matrix)
    if not torch.allclose(m, m.t()):
        raise ValueError("the matrix is not symmetric")
    l, info = torch.linalg.cholesky_ex(m)
    if int(info):
        raise ValueError("the matrix is not positive-definite")
    _show_matrix("L", l)


def cmd_qr(a):
    q, r = torch.linalg.qr(_matrix(a.matrix))
    _show_matrix("Q", q)
    _show_matrix("R", r)


def cmd_cg(a):
    from . import symbolic as S
    x, it = S.conjugate_gradient(_matrix(a.matrix), _vector(a.rhs))
    print("x = [" + ", ".join(_fmt(v) for v in x.tolist()) + f"]  ({it} iterations)")


def cmd_polyroots(a):
    from . import symbolic as S
    for z in S.polyroots(_vector(a.coeffs).tolist()):
        print(_fmt(z.real) if abs(z.imag) < 1e-12 else f"{_fmt(z.real)} {'+' if z.imag >= 0 else '-'} {_fmt(abs(z.imag))}i")


def cmd_ode(a):
    from . import symbolic as S
    y, steps = S.ode(a.expr, a.y0, a.t0, a.t1, a.h, a.method)
    print(f"y({_fmt(a.t1)}) = {_fmt(y)}  ({steps} steps, {a.method})")


def cmd_inverse(a):
    m = _matrix(a.matrix)
    if m.shape[0] != m.shape[1] or abs(float(torch.linalg.det(m))) < 1e-14:
        raise ValueError("the matrix must be square and non-singular")
    _show_matrix("A^-1", torch.linalg.inv(m))


def cmd_solve_system(a):
    from . import symbolic as S
    pt = S.solve_system([e for e in a.system.split(";") if e.strip()], a.vars.split(","), [float(v) for v in a.start.split(",")])
    print(", ".join(f"{k} = {_fmt(v)}" for k, v in pt.items()))


def cmd_fem_heat(a):
    from . import symbolic as S
    xs, u = S.fem_heat_1d(a.nodes, a.length, a.source)
    for x, v in zip(xs.tolist(), u.tolist()):
        print(f"x = {x:.6f}  u = {v:.8f}")
    print(f"max u = {_fmt(float(u.max()))}  (analytic {_fmt(a.source * a.length ** 2 / 8)})")


def cmd_sat(a):
    from . import symbolic as S
    clauses = [[int(v) for v in c.split(",")] for c in a.clauses.split(";") if c.strip()]
    model = S.sat_solve(clauses)
    if model is None:
        print("UNSAT")
        return 1
    print("SAT: " + " ".join(f"{k}={'T' if v else 'F'}" for k, v in sorted(model.items())))


def cmd_symreg(a):
    from . import symbolic as S
    expr, mse = S.symreg(_vector(a.xs), _vector(a.ys), a.seed)
    print(f"y = {expr}   (mse {mse:.3e})")


def cmd_quantum(a):
    from . import quantum as Q
    from .nn.rng import PcgEngine
    qubits, chi = min(max(a.qubits, 2), 28), max(a.chi, 1)
    ghz = Q.Mps.zero(4)
    ghz.apply_1qubit_gate(0, Q.gates.H)
    for q in range(3):
        ghz.apply_2qubit_gate(q, Q.gates.CNOT, 8)
    sv = ghz.to_statevector()
    rng = PcgEngine(a.seed)
    mps = Q.Mps.zero(qubits)
    for _ in range(6):
        for q in range(qubits):
            mps.apply_1qubit_gate(q, Q.gates.ry(rng.float_signed() * 3.0))
        for start in (0, 1):
            for q in range(start, qubits - 1, 2):
                mps.apply_2qubit_gate(q, Q.gates.CNOT, chi)
    dense, store = 1 << qubits, mps.storage()
    print(f"MPS circuit simulator, deterministic (seed {a.seed})")
    print(f"  GHZ(4): |0000> = {abs(float(sv[0])):.4f}, |1111> = {abs(float(sv[15])):.4f}  (target {math.sqrt(0.5):.4f})")
    print(f"  random circuit: {qubits} qubits, 6 layers, bond cap chi = {chi}")
    print(f"    bond dimension reached: {mps.max_bond()}")
    print(f"    MPS storage: {store} amplitudes vs dense 2^{qubits} = {dense}  ({dense / store:.3e}x smaller)")
    if qubits <= 14:
        print(f"    norm of the truncated state: {float(mps.to_statevector().abs().pow(2).sum().sqrt()):.6f}")


def register(sub):
    def add(name, fn, *args, **opts):
        p = sub.add_parser(name)
        for arg in args:
            p.add_argument(arg)
        for k, (kw) in opts.items():
            p.add_argument(*kw.pop("flags", [f"--{k.replace('_', '-')}"]), **kw)
        p.set_defaults(fn=_guard(fn))
        return p

    add("diff", cmd_diff, "expr").add_argument("var", nargs="?", default="x")
    add("simplify", cmd_simplify, "expr")
    add("trig", cmd_simplify, "expr")
    add("eval", cmd_eval, "expr").add_argument("bindings", nargs="*")
    add("solve", cmd_solve, "expr").add_argument("var", nargs="?", default="x")
    add("prove", cmd_prove, "lhs", "rhs")
    add("gradient", cmd_gradient, "expr").add_argument("bindings", nargs="+")
    add("to-rust", cmd_to_rust, "expr")
    add("to-cuda", cmd_to_cuda, "expr")
    add("regress", cmd_regress, "xs", "ys").add_argument("degree", nargs="?", type=int, default=1)
    add("patterns", cmd_patterns, "series")
    for name, fn, methods, default in (("integrate", cmd_integrate, ("romberg", "simpson", "gauss"), "romberg"),
                                       ("root", cmd_root, ("brent", "bisection", "secant", "newton"), "brent"),
                                       ("minimize", cmd_minimize, None, None)):
        p = add(name, fn, "expr")
        p.add_argument("a", type=float)
        p.add_argument("b", type=float)
        p.add_argument("var", nargs="?", default="x")
        if methods:
            p.add_argument("--method", choices=methods, default=default)
    p = add("optimize", cmd_optimize, "expr")
    p.add_argument("--start", required=True)
    p.add_argument("--vars", default="")
    add("linsolve", cmd_linsolve, "matrix", "rhs")
    add("lstsq", cmd_lstsq, "matrix", "rhs")
    add("det", cmd_det, "matrix")
    add("cholesky", cmd_cholesky, "matrix")
    add("qr", cmd_qr, "matrix")
    add("cg", cmd_cg, "matrix", "rhs")
    add("polyroots", cmd_polyroots, "coeffs")
    p = add("ode", cmd_ode, "expr")
    for n in ("y0", "t0", "t1"):
        p.add_argument(n, type=float)
    p.add_argument("h", nargs="?", type=float, default=None)
    p.add_argument("--method", choices=("rk4", "dopri5"), default="rk4")
    add("inverse", cmd_inverse, "matrix")
    p = add("solve-system", cmd_solve_system, "system")
    p.add_argument("--vars", required=True)
    p.add_argument("--start", required=True)
    p = add("fem-heat", cmd_fem_heat)
    p.add_argument("nodes", type=int)
    p.add_argument("length", type=float)
    p.add_argument("source", type=float)
    add("sat", cmd_sat, "clauses")
    add("symreg", cmd_symreg, "xs", "ys").add_argument("--seed", type=int, default=0)
    p = add("quantum", cmd_quantum)
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--qubits", type=int, default=12)
    p.add_argument("--chi", type=int, default=16)

"""Small computer-algebra core: parse -> tree -> evaluate (vectorised on tensors) / differentiate / simplify / prove /
solve / emit source, plus the numeric routines that take an expression string (quadrature, root finding, minimisation,
ODEs, non-linear systems with the exact symbolic Jacobian), a DPLL SAT solver and a template symbolic regressor.

Grammar: numbers, names, ``+ - * / ^``, unary minus, parentheses, functions ``sin cos tan asin acos atan sinh cosh tanh exp
ln log sqrt abs``, constants ``pi`` and ``e``; ``^`` is right-associative and binds tighter than unary minus.
``simplify`` brings an expression to a canonical sum of monomials over "atoms" (variables and function calls with
canonical arguments) with exact rational coefficients, rewriting ``cos(u)^2 -> 1 - sin(u)^2``; two expressions are proved
equal when the canonical form of their difference is empty (and, as a fallback for forms the rewriter does not
normalise, refuted when they differ at random points). ``to_cuda`` prints a device expression in fp32, so that a checked
formula can be pasted into a kernel.
Reference counterpart: scirust-symbolic/src/lib.rs (parser, ``diff``, ``simplify``, ``discover_patterns``, finite-difference
helpers) and the commands of scirust-cli/src/{symbolic,numeric,reasoning}.rs.
"""
from __future__ import annotations

import math
from fractions import Fraction

import torch

FUNCS = ("sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh", "tanh", "exp", "ln", "log", "sqrt", "abs")
CONSTS = {"pi": math.pi, "e": math.e}


class SymbolicError(ValueError):
    pass


# ------------------------------------------------------------------ parser
def _tokens(s: str):
    out, i = [], 0
    while i < len(s):
        c = s[i]
        if c.isspace():
            i += 1
        elif c.isdigit() or (c == "." and i + 1 < len(s) and s[i + 1].isdigit()):
            j = i
            while j < len(s) and (s[j].isdigit() or s[j] == "."):
                j += 1
            if j < len(s) and s[j] in "eE" and j + 1 < len(s) and (s[j + 1].isdigit() or (s[j + 1] in "+-" and j + 2 < len(s) and s[j + 2].isdigit())):
                j += 2
                while j < len(s) and s[j].isdigit():
                    j += 1
            out.append(("num", s[i:j]))
            i = j
        elif c.isalpha() or c == "_":
            j = i
            while j < len(s) and (s[j].isalnum() or s[j] == "_"):
                j += 1
            out.append(("id", s[i:j]))
            i = j
        elif c in "+-*/^(),":
            out.append((c, c))
            i += 1
        else:
            raise SymbolicError(f"unexpected character {c!r} at {i}")
    return out


def parse(s: str):
    toks, pos = _tokens(s), [0]

    def peek():
        return toks[pos[0]][0] if pos[0] < len(toks) else None

    def take(kind=None):
        if pos[0] >= len(toks) or (kind and toks[pos[0]][0] != kind):
            raise SymbolicError(f"expected {kind or 'a token'} at token {pos[0]}")
        pos[0] += 1
        return toks[pos[0] - 1]

    def expr():
        node = term()
        while peek() in ("+", "-"):
            op = take()[0]
            node = ("add" if op == "+" else "sub", node, term())
        return node

    def term():
        node = unary()
        while peek() in ("*", "/"):
            op = take()[0]
            node = ("mul" if op == "*" else "div", node, unary())
        return node

    def unary():
        if peek() == "-":
            take()
            return ("neg", unary())
        if peek() == "+":
            take()
            return unary()
        return power()

    def power():
        base = atom()
        if peek() == "^":
            take()
            return ("pow", base, unary())                                   # right-associative, allows x^-2
        return base

    def atom():
        k = peek()
        if k == "num":
            t = take()[1]
            return ("num", Fraction(t) if "e" not in t.lower() else Fraction(float(t)))
        if k == "id":
            name = take()[1]
            if peek() == "(":
                if name not in FUNCS:
                    raise SymbolicError(f"unknown function {name!r}")
                take("(")
                arg = expr()
                take(")")
                return ("fn", "ln" if name == "log" else name, arg)
            return ("const", name) if name in CONSTS else ("var", name)
        if k == "(":
            take("(")
            node = expr()
            take(")")
            return node
        raise SymbolicError("unexpected end of expression" if k is None else f"unexpected token {k!r}")

    tree = expr()
    if pos[0] != len(toks):
        raise SymbolicError(f"trailing input at token {pos[0]}")
    return tree


def _as_tree(e):
    return parse(e) if isinstance(e, str) else e


# ------------------------------------------------------------------ evaluation
_TORCH = {"sin": torch.sin, "cos": torch.cos, "tan": torch.tan, "asin": torch.asin, "acos": torch.acos, "atan": torch.atan,
          "sinh": torch.sinh, "cosh": torch.cosh, "tanh": torch.tanh, "exp": torch.exp, "ln": torch.log, "sqrt": torch.sqrt,
          "abs": torch.abs}


def evaluate(e, env=None, dtype=torch.float64):
    """Value of the expression with variables bound to numbers or tensors (broadcast together); returns a tensor."""
    env = env or {}

    def ev(n):
        k = n[0]
        if k == "num":
            return torch.tensor(float(n[1]), dtype=dtype)
        if k == "const":
            return torch.tensor(CONSTS[n[1]], dtype=dtype)
        if k == "var":
            if n[1] not in env:
                raise SymbolicError(f"unbound variable {n[1]!r}")
            return torch.as_tensor(env[n[1]], dtype=dtype)
        if k == "neg":
            return -ev(n[1])
        if k == "fn":
            return _TORCH[n[1]](ev(n[2]))
        a, b = ev(n[1]), ev(n[2])
        return {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "pow": torch.pow}[k](a, b)
    return ev(_as_tree(e))


def variables(e) -> list:
    out = set()

    def walk(n):
        if n[0] == "var":
            out.add(n[1])
        for c in n[1:]:
            if isinstance(c, tuple):
                walk(c)
    walk(_as_tree(e))
    return sorted(out)


# ------------------------------------------------------------------ differentiation
def _num(v):
    return ("num", Fraction(v))


def diff(e, var: str = "x"):
    def d(n):
        k = n[0]
        if k in ("num", "const"):
            return _num(0)
        if k == "var":
            return _num(1 if n[1] == var else 0)
        if k == "neg":
            return ("neg", d(n[1]))
        if k in ("add", "sub"):
            return (k, d(n[1]), d(n[2]))
        if k == "mul":
            return ("add", ("mul", d(n[1]), n[2]), ("mul", n[1], d(n[2])))
        if k == "div":
            return ("div", ("sub", ("mul", d(n[1]), n[2]), ("mul", n[1], d(n[2]))), ("pow", n[2], _num(2)))
        if k == "pow":
            base, ex = n[1], n[2]
            if not variables(ex):
                return ("mul", ("mul", ex, ("pow", base, ("sub", ex, _num(1)))), d(base))
            return ("mul", n, ("add", ("mul", d(ex), ("fn", "ln", base)), ("div", ("mul", ex, d(base)), base)))
        if k == "fn":
            u, du = n[2], d(n[2])
            f = n[1]
            inner = {
                "sin": ("fn", "cos", u), "cos": ("neg", ("fn", "sin", u)), "tan": ("div", _num(1), ("pow", ("fn", "cos", u), _num(2))),
                "asin": ("div", _num(1), ("fn", "sqrt", ("sub", _num(1), ("pow", u, _num(2))))),
                "acos": ("neg", ("div", _num(1), ("fn", "sqrt", ("sub", _num(1), ("pow", u, _num(2)))))),
                "atan": ("div", _num(1), ("add", _num(1), ("pow", u, _num(2)))),
                "sinh": ("fn", "cosh", u), "cosh": ("fn", "sinh", u), "tanh": ("sub", _num(1), ("pow", ("fn", "tanh", u), _num(2))),
                "exp": ("fn", "exp", u), "ln": ("div", _num(1), u), "sqrt": ("div", _num(1), ("mul", _num(2), ("fn", "sqrt", u))),
                "abs": ("div", u, ("fn", "abs", u))}[f]
            return ("mul", inner, du)
        raise SymbolicError(f"cannot differentiate node {k!r}")
    return simplify(d(_as_tree(e)))


def gradient(e, point: dict) -> dict:
    t = _as_tree(e)
    return {v: float(evaluate(diff(t, v), point)) for v in sorted(point)}


# ------------------------------------------------------------------ canonical form
# A polynomial is {monomial: Fraction}; a monomial is a sorted tuple of (atom_key, exponent) with non-zero exponents;
# an atom_key is a printable canonical string (a variable name, a constant name or "fn(canonical argument)").
def _pmul(a, b):
    out = {}
    for ma, ca in a.items():
        for mb, cb in b.items():
            d = dict(ma)
            for k, ex in mb:
                d[k] = d.get(k, 0) + ex
            m = tuple(sorted((k, ex) for k, ex in d.items() if ex != 0))
            out[m] = out.get(m, 0) + ca * cb
    return {m: c for m, c in out.items() if c != 0}


def _padd(a, b, sign=1):
    out = dict(a)
    for m, c in b.items():
        out[m] = out.get(m, 0) + sign * c
    return {m: c for m, c in out.items() if c != 0}


def _const_poly(c):
    return {(): Fraction(c)} if c != 0 else {}


def _trig_reduce(p):
    """cos(u)^n with n >= 2 -> (1 - sin(u)^2) cos(u)^(n-2), repeated: sin^2 + cos^2 collapses to 1."""
    changed = True
    while changed:
        changed = False
        for m, c in list(p.items()):
            for k, ex in m:
                if k.startswith("cos(") and ex >= 2:
                    rest = {tuple(x for x in m if x[0] != k): c}
                    s = "sin(" + k[4:]
                    repl = _pmul(rest, _pmul({((k, ex - 2),) if ex > 2 else (): Fraction(1)},
                                              {(): Fraction(1), ((s, 2),): Fraction(-1)}))
                    del p[m]
                    p = _padd(p, repl)
                    changed = True
                    break
            if changed:
                break
    return p


def _canon(n):
    k = n[0]
    if k == "num":
        return _const_poly(n[1])
    if k in ("var", "const"):
        return {((n[1], 1),): Fraction(1)}
    if k == "neg":
        return {m: -c for m, c in _canon(n[1]).items()}
    if k == "add":
        return _padd(_canon(n[1]), _canon(n[2]))
    if k == "sub":
        return _padd(_canon(n[1]), _canon(n[2]), -1)
    if k == "mul":
        return _pmul(_canon(n[1]), _canon(n[2]))
    if k == "div":
        den = _canon(n[2])
        if not den:
            raise SymbolicError("division by zero")
        if len(den) == 1:                                                      # a single monomial can be inverted
            (m, c), = den.items()
            return _pmul(_canon(n[1]), {tuple((a, -ex) for a, ex in m): 1 / c})
        return _pmul(_canon(n[1]), {(("(" + poly_to_string(den) + ")", -1),): Fraction(1)})
    if k == "pow":
        base, ex = _canon(n[1]), _canon(n[2])
        if not ex:
            return _const_poly(1)
        if list(ex) == [()] and ex[()].denominator == 1:                       # integer exponent
            e_int = int(ex[()])
            if len(base) == 1:
                (m, c), = base.items()
                return {tuple((a, x * e_int) for a, x in m): c ** e_int}
            if not base:
                if e_int <= 0:
                    raise SymbolicError("zero to a non-positive power")
                return {}
            if 0 < e_int <= 12:
                out = _const_poly(1)
                for _ in range(e_int):
                    out = _pmul(out, base)
                return out
            return {(("(" + poly_to_string(base) + ")", e_int),): Fraction(1)}
        if list(ex) == [()] and list(base) == [()] and base[()] > 0:            # number ^ fraction: exact roots only
            q = ex[()]
            root_n = _exact_root(base[()].numerator, q.denominator)
            root_d = _exact_root(base[()].denominator, q.denominator)
            if root_n is not None and root_d is not None:
                return _const_poly(Fraction(root_n, root_d) ** q.numerator)
        return {((f"({poly_to_string(base)})^({poly_to_string(ex)})", 1),): Fraction(1)}
    if k == "fn":
        arg = _canon(n[2])
        if n[1] == "ln" and arg == _const_poly(1):
            return {}
        if n[1] == "exp" and arg == {}:
            return _const_poly(1)
        if n[1] in ("sin", "tan", "sinh", "tanh", "asin", "atan") and arg == {}:
            return {}
        if n[1] in ("cos", "cosh") and arg == {}:
            return _const_poly(1)
        if n[1] == "sqrt" and list(arg.keys()) == [()]:
            v = arg[()]
            rn, rd = math.isqrt(v.numerator) if v > 0 else -1, math.isqrt(v.denominator)
            if v > 0 and rn * rn == v.numerator and rd * rd == v.denominator:
                return _const_poly(Fraction(rn, rd))
        inner = poly_to_string(arg)
        if n[1] == "tan":                                                       # one spelling for the quotient
            return {((f"cos({inner})", -1), (f"sin({inner})", 1)): Fraction(1)}
        return {((f"{n[1]}({inner})", 1),): Fraction(1)}
    raise SymbolicError(f"cannot canonicalise node {k!r}")


def _exact_root(v: int, k: int):
    r = round(v ** (1.0 / k))
    for c in (r - 1, r, r + 1):
        if c >= 0 and c ** k == v:
            return c
    return None


def _fr(c: Fraction) -> str:
    return str(c.numerator) if c.denominator == 1 else f"{c.numerator}/{c.denominator}"


def poly_to_string(p) -> str:
    if not p:
        return "0"
    def mono_key(m):
        return (-sum(ex for _, ex in m if ex > 0), m)
    parts = []
    for m in sorted(p, key=mono_key):
        c = p[m]
        num = [f"{a}^{ex}" if ex != 1 else a for a, ex in m if ex > 0]
        den = [f"{a}^{-ex}" if ex != -1 else a for a, ex in m if ex < 0]
        body = "*".join(num)
        mag = abs(c)
        if not body:
            body = _fr(mag)
        elif mag != 1:
            body = (_fr(mag) if mag.denominator == 1 else f"({_fr(mag)})") + "*" + body
        if den:
            body += "/" + (den[0] if len(den) == 1 else "(" + "*".join(den) + ")")
        parts.append(("-" if c < 0 else "+", body))
    s = ("-" if parts[0][0] == "-" else "") + parts[0][1]
    for sign, body in parts[1:]:
        s += f" {sign} {body}"
    return s


def canonical(e):
    return _trig_reduce(_canon(_as_tree(e)))


def simplify(e):
    """Canonical tree of the expression (parse of its canonical string)."""
    return parse(poly_to_string(canonical(e)))


def simplify_str(e) -> str:
    return poly_to_string(canonical(e))


def prove_equal(a, b, trials: int = 16, seed: int = 0):
    """-> (verdict, how): True by canonical form, else numeric refutation / agreement at random points in (0.1, 2)."""
    ta, tb = _as_tree(a), _as_tree(b)
    if canonical(("sub", ta, tb)) == {}:
        return True, "canonical forms agree"
    g = torch.Generator().manual_seed(seed)
    vs = sorted(set(variables(ta)) | set(variables(tb)))
    env = {v: torch.rand(trials, generator=g, dtype=torch.float64) * 1.9 + 0.1 for v in vs}
    da, db = evaluate(ta, env), evaluate(tb, env)
    ok = torch.isfinite(da) & torch.isfinite(db)
    if bool(ok.any()) and bool(((da - db).abs()[ok] > 1e-9 * (1 + da.abs()[ok])).any()):
        return False, "they differ at a sampled point"
    return False, "not proved (they agree numerically at the sampled points, but the canonical forms differ)"


# ------------------------------------------------------------------ printing
_PREC = {"add": 1, "sub": 1, "mul": 2, "div": 2, "neg": 3, "pow": 4}


def to_string(e) -> str:
    def s(n, parent=0, right=False):
        k = n[0]
        if k == "num":
            t = _fr(n[1])
            return f"({t})" if ("/" in t or n[1] < 0) and parent > 1 else t
        if k in ("var", "const"):
            return n[1]
        if k == "fn":
            return f"{n[1]}({s(n[2])})"
        if k == "neg":
            t = "-" + s(n[1], 3)
            return f"({t})" if parent >= 3 else t
        p = _PREC[k]
        op = {"add": " + ", "sub": " - ", "mul": "*", "div": "/", "pow": "^"}[k]
        t = s(n[1], p, False) + op + s(n[2], p + (0 if k in ("add", "mul") else 1) if k != "pow" else p, True)
        if k == "pow":
            t = s(n[1], p + 1) + "^" + s(n[2], p)
        return f"({t})" if p < parent or (p == parent and right and k in ("sub", "div")) else t
    return s(_as_tree(e))


def _emit(e, lit, powf, fn_map) -> str:
    def s(n):
        k = n[0]
        if k == "num":
            return lit(float(n[1]))
        if k == "const":
            return lit(CONSTS[n[1]])
        if k == "var":
            return n[1]
        if k == "neg":
            return f"(-{s(n[1])})"
        if k == "fn":
            return fn_map(n[1], s(n[2]))
        if k == "pow":
            if n[2][0] == "num" and n[2][1].denominator == 1 and 0 < n[2][1] <= 4:
                return "(" + " * ".join([s(n[1])] * int(n[2][1])) + ")"
            return powf(s(n[1]), s(n[2]))
        return f"({s(n[1])} {dict(add='+', sub='-', mul='*', div='/')[k]} {s(n[2])})"
    return s(_as_tree(e))


def to_rust(e) -> str:
    return _emit(e, lambda v: repr(float(v)) + "_f64", lambda a, b: f"{a}.powf({b})", lambda f, a: f"{a}.{f}()")


def to_cuda(e) -> str:
    """fp32 device expression: ``sinf`` / ``expf`` / ``powf`` ..., literals with the ``f`` suffix."""
    names = {"ln": "logf", "abs": "fabsf"}
    return _emit(e, lambda v: repr(float(v)) + "f", lambda a, b: f"powf({a}, {b})", lambda f, a: f"{names.get(f, f + 'f')}({a})")


# ------------------------------------------------------------------ equation solving
def polynomial_coefficients(e, var: str = "x"):
    """Ascending coefficients (floats) if the canonical form is a polynomial in ``var`` with numeric coefficients, else None."""
    out = {}
    for m, c in canonical(e).items():
        deg = 0
        for a, ex in m:
            if a == var and ex > 0:
                deg = ex
            elif a in CONSTS and ex > 0:
                c = c * Fraction(CONSTS[a]) ** ex
            else:
                return None
        out[deg] = out.get(deg, 0) + c
    if not out:
        return [0.0]
    return [float(out.get(i, 0)) for i in range(max(out) + 1)]


def polyroots(coeffs):
    """Roots of ``c0 + c1 x + ...`` as complex numbers (eigenvalues of the companion matrix), sorted."""
    c = [float(v) for v in coeffs]
    while len(c) > 1 and c[-1] == 0.0:
        c.pop()
    n = len(c) - 1
    if n < 1:
        return []
    comp = torch.zeros(n, n, dtype=torch.float64)
    comp[1:, :-1] = torch.eye(n - 1, dtype=torch.float64)
    comp[:, -1] = -torch.tensor(c[:-1], dtype=torch.float64) / c[-1]
    ev = torch.linalg.eigvals(comp)
    return sorted((complex(v) for v in ev), key=lambda z: (round(z.real, 12), round(z.imag, 12)))


def solve(e, var: str = "x", lo: float = -100.0, hi: float = 100.0):
    """Real solutions of ``e = 0``: exact route for polynomials (companion matrix), sign-change scan + Brent otherwise."""
    co = polynomial_coefficients(e, var)
    if co is not None:
        roots = [z.real for z in polyroots(co) if abs(z.imag) < 1e-9 * max(1.0, abs(z.real))]
        f = lambda v: float(evaluate(e, {var: v}))
        return sorted({round(_polish(f, r), 12) + 0.0 for r in roots})
    t = _as_tree(e)
    xs = torch.linspace(lo, hi, 4001, dtype=torch.float64)
    ys = evaluate(t, {var: xs})
    out = []
    for i in range(4000):
        a, b = float(ys[i]), float(ys[i + 1])
        if math.isfinite(a) and math.isfinite(b) and (a == 0.0 or a * b < 0):
            out.append(find_root(t, float(xs[i]), float(xs[i + 1]), var))
    return sorted({round(r, 10) + 0.0 for r in out})


def _polish(f, r):
    for _ in range(3):
        h = 1e-6 * max(1.0, abs(r))
        d = (f(r + h) - f(r - h)) / (2 * h)
        if d == 0 or not math.isfinite(d):
            break
        r -= f(r) / d
    return r


# ------------------------------------------------------------------ numeric routines on expressions
def _scalar_fn(e, var):
    t = _as_tree(e)
    return lambda v: float(evaluate(t, {var: v}))


def integrate(e, a: float, b: float, var: str = "x", method: str = "romberg", tol: float = 1e-10) -> float:
    t = _as_tree(e)
    f = lambda xs: evaluate(t, {var: xs})
    if method == "simpson":
        n = 1024
        xs = torch.linspace(a, b, n + 1, dtype=torch.float64)
        ys = f(xs) + torch.zeros_like(xs)
        return float((b - a) / (3 * n) * (ys[0] + ys[-1] + 4 * ys[1:-1:2].sum() + 2 * ys[2:-1:2].sum()))
    if method == "gauss":
        import numpy as np
        nodes, weights = np.polynomial.legendre.leggauss(64)
        xs = torch.from_numpy(0.5 * (b - a) * nodes + 0.5 * (b + a))
        return float(0.5 * (b - a) * ((f(xs) + torch.zeros_like(xs)) * torch.from_numpy(weights)).sum())
    if method != "romberg":
        raise SymbolicError(f"unknown quadrature {method!r}")
    rows = [[0.5 * (b - a) * float(f(torch.tensor(a, dtype=torch.float64)) + f(torch.tensor(b, dtype=torch.float64)))]]
    for k in range(1, 22):
        n = 1 << (k - 1)
        h = (b - a) / (2 * n)
        mids = a + h * (2 * torch.arange(n, dtype=torch.float64) + 1)
        row = [0.5 * rows[-1][0] + h * float((f(mids) + torch.zeros_like(mids)).sum())]
        for j in range(1, k + 1):
            row.append(row[j - 1] + (row[j - 1] - rows[-1][j - 1]) / (4 ** j - 1))
        rows.append(row)
        if k >= 4 and abs(row[-1] - rows[-2][-1]) <= tol * max(1.0, abs(row[-1])):
            break
    return rows[-1][-1]


def find_root(e, a: float, b: float, var: str = "x", method: str = "brent", tol: float = 1e-13, max_iter: int = 200) -> float:
    f = _scalar_fn(e, var)
    if method == "newton":
        df = _scalar_fn(diff(e, var), var)
        x = 0.5 * (a + b)
        for _ in range(max_iter):
            fx, d = f(x), df(x)
            if d == 0:
                raise SymbolicError("zero derivative")
            step = fx / d
            x -= step
            if abs(step) <= tol * max(1.0, abs(x)):
                return x
        raise SymbolicError("Newton's method did not converge")
    if method == "secant":
        x0, x1 = a, b
        for _ in range(max_iter):
            f0, f1 = f(x0), f(x1)
            if f1 == f0:
                break
            x0, x1 = x1, x1 - f1 * (x1 - x0) / (f1 - f0)
            if abs(x1 - x0) <= tol * max(1.0, abs(x1)):
                return x1
        return x1
    fa, fb = f(a), f(b)
    if fa == 0:
        return a
    if fb == 0:
        return b
    if fa * fb > 0:
        raise SymbolicError("the function has the same sign at both ends of the bracket")
    if method == "bisection":
        for _ in range(max_iter * 2):
            m = 0.5 * (a + b)
            fm = f(m)
            if fm == 0 or 0.5 * (b - a) <= tol * max(1.0, abs(m)):
                return m
            a, b, fa = (m, b, fm) if fa * fm > 0 else (a, m, fa)
        return 0.5 * (a + b)
    if method != "brent":
        raise SymbolicError(f"unknown root finder {method!r}")
    c, fc, d, mflag = a, fa, 0.0, True
    if abs(fa) < abs(fb):
        a, b, fa, fb = b, a, fb, fa
        c, fc = a, fa
    for _ in range(max_iter):
        if fa != fc and fb != fc:
            s = a * fb * fc / ((fa - fb) * (fa - fc)) + b * fa * fc / ((fb - fa) * (fb - fc)) + c * fa * fb / ((fc - fa) * (fc - fb))
        else:
            s = b - fb * (b - a) / (fb - fa)
        lo_, hi_ = sorted(((3 * a + b) / 4, b))
        if (not lo_ < s < hi_ or (mflag and abs(s - b) >= abs(b - c) / 2) or (not mflag and abs(s - b) >= abs(c - d) / 2)
                or (mflag and abs(b - c) < tol) or (not mflag and abs(c - d) < tol)):
            s, mflag = 0.5 * (a + b), True
        else:
            mflag = False
        fs = f(s)
        d, c, fc = c, b, fb
        if fa * fs < 0:
            b, fb = s, fs
        else:
            a, fa = s, fs
        if abs(fa) < abs(fb):
            a, b, fa, fb = b, a, fb, fa
        if fb == 0 or abs(b - a) <= tol * max(1.0, abs(b)):
            return b
    return b


def minimize_1d(e, a: float, b: float, var: str = "x", tol: float = 1e-10):
    """Golden-section search on [a, b] -> (argmin, minimum)."""
    f = _scalar_fn(e, var)
    g = (math.sqrt(5) - 1) / 2
    c, d = b - g * (b - a), a + g * (b - a)
    fc, fd = f(c), f(d)
    while abs(b - a) > tol * max(1.0, abs(a) + abs(b)):
        if fc < fd:
            b, d, fd = d, c, fc
            c = b - g * (b - a)
            fc = f(c)
        else:
            a, c, fc = c, d, fd
            d = a + g * (b - a)
            fd = f(d)
    x = 0.5 * (a + b)
    return x, f(x)


def optimize(e, start, vars_=None, max_iter: int = 500, tol: float = 1e-10):
    """BFGS with the exact symbolic gradient and a backtracking line search -> (point dict, value, iterations)."""
    t = _as_tree(e)
    vs = list(vars_ or variables(t))
    if len(vs) != len(start):
        raise SymbolicError("one start value per variable")
    grads = [diff(t, v) for v in vs]
    f = lambda x: float(evaluate(t, dict(zip(vs, x.tolist()))))
    gf = lambda x: torch.tensor([float(evaluate(g, dict(zip(vs, x.tolist())))) for g in grads], dtype=torch.float64)
    x = torch.tensor([float(s) for s in start], dtype=torch.float64)
    h = torch.eye(len(vs), dtype=torch.float64)
    fx, g = f(x), gf(x)
    it = 0
    for it in range(1, max_iter + 1):
        if float(g.norm()) <= tol:
            break
        p = -(h @ g)
        if float(p @ g) >= 0:
            h, p = torch.eye(len(vs), dtype=torch.float64), -g
        step = 1.0
        while step > 1e-14 and not f(x + step * p) <= fx + 1e-4 * step * float(p @ g):
            step *= 0.5
        s = step * p
        xn = x + s
        gn = gf(xn)
        y = gn - g
        sy = float(s @ y)
        if sy > 1e-14:
            rho = 1.0 / sy
            i_ = torch.eye(len(vs), dtype=torch.float64)
            h = (i_ - rho * torch.outer(s, y)) @ h @ (i_ - rho * torch.outer(y, s)) + rho * torch.outer(s, s)
        x, g, fx = xn, gn, f(xn)
        if float(s.norm()) <= 1e-15 * max(1.0, float(x.norm())):
            break
    return dict(zip(vs, x.tolist())), fx, it


def solve_system(exprs, vars_, start, max_iter: int = 100, tol: float = 1e-12):
    """Newton's method on ``f_i = 0`` with the symbolic Jacobian -> point dict."""
    ts = [_as_tree(e) for e in exprs]
    if len(ts) != len(vars_) or len(start) != len(vars_):
        raise SymbolicError("need as many equations and start values as variables")
    jac = [[diff(t, v) for v in vars_] for t in ts]
    x = torch.tensor([float(s) for s in start], dtype=torch.float64)
    for _ in range(max_iter):
        env = dict(zip(vars_, x.tolist()))
        f = torch.tensor([float(evaluate(t, env)) for t in ts], dtype=torch.float64)
        if float(f.abs().max()) <= tol:
            return env
        j = torch.tensor([[float(evaluate(d, env)) for d in row] for row in jac], dtype=torch.float64)
        x = x - torch.linalg.solve(j, f)
    raise SymbolicError("Newton's method did not converge")


def ode(e, y0: float, t0: float, t1: float, h: float | None = None, method: str = "rk4", tol: float = 1e-9):
    """``y' = e(t, y)`` from t0 to t1 -> (y(t1), steps). rk4: fixed step ``h`` (default (t1 - t0) / 100);
    dopri5: adaptive Dormand-Prince 5(4) with step control on the embedded error."""
    tr = _as_tree(e)
    f = lambda t, y: float(evaluate(tr, {"t": t, "y": y}))
    if method == "rk4":
        n = max(1, round(abs(t1 - t0) / (h or abs(t1 - t0) / 100)))
        hh, t, y = (t1 - t0) / n, t0, y0
        for _ in range(n):
            k1 = f(t, y)
            k2 = f(t + hh / 2, y + hh * k1 / 2)
            k3 = f(t + hh / 2, y + hh * k2 / 2)
            k4 = f(t + hh, y + hh * k3)
            y += hh * (k1 + 2 * k2 + 2 * k3 + k4) / 6
            t += hh
        return y, n
    if method != "dopri5":
        raise SymbolicError(f"unknown integrator {method!r}")
    c = [0, 1 / 5, 3 / 10, 4 / 5, 8 / 9, 1, 1]
    a = [[], [1 / 5], [3 / 40, 9 / 40], [44 / 45, -56 / 15, 32 / 9], [19372 / 6561, -25360 / 2187, 64448 / 6561, -212 / 729],
         [9017 / 3168, -355 / 33, 46732 / 5247, 49 / 176, -5103 / 18656], [35 / 384, 0, 500 / 1113, 125 / 192, -2187 / 6784, 11 / 84]]
    b5 = a[6] + [0]
    b4 = [5179 / 57600, 0, 7571 / 16695, 393 / 640, -92097 / 339200, 187 / 2100, 1 / 40]
    t, y, hh, steps = t0, y0, (h or (t1 - t0) / 100), 0
    while (t1 - t) * (1 if t1 >= t0 else -1) > 1e-14 * max(1.0, abs(t1)):
        hh = min(hh, t1 - t) if t1 >= t0 else max(hh, t1 - t)
        k = []
        for i in range(7):
            k.append(f(t + c[i] * hh, y + hh * sum(a[i][j] * k[j] for j in range(i))))
        y5 = y + hh * sum(b5[i] * k[i] for i in range(7))
        err = abs(hh * sum((b5[i] - b4[i]) * k[i] for i in range(7)))
        sc = tol * (1 + max(abs(y), abs(y5)))
        if err <= sc:
            t, y, steps = t + hh, y5, steps + 1
        hh *= min(5.0, max(0.2, 0.9 * (sc / err) ** 0.2)) if err > 0 else 5.0
        if steps > 1_000_000:
            raise SymbolicError("too many steps")
    return y, steps


def fem_heat_1d(nodes: int, length: float, source: float):
    """-u'' = source on (0, length), u = 0 at both ends, linear elements -> (node positions, temperatures)."""
    if nodes < 3:
        raise SymbolicError("need at least 3 nodes")
    n, h = nodes - 2, length / (nodes - 1)
    k = (2.0 * torch.eye(n, dtype=torch.float64) - torch.diag(torch.ones(n - 1, dtype=torch.float64), 1)
         - torch.diag(torch.ones(n - 1, dtype=torch.float64), -1)) / h
    u = torch.linalg.solve(k, torch.full((n,), source * h, dtype=torch.float64))
    return torch.linspace(0, length, nodes, dtype=torch.float64), torch.cat([torch.zeros(1, dtype=torch.float64), u, torch.zeros(1, dtype=torch.float64)])


def conjugate_gradient(a, b, tol: float = 1e-12, max_iter: int | None = None):
    a, b = torch.as_tensor(a, dtype=torch.float64), torch.as_tensor(b, dtype=torch.float64)
    x = torch.zeros_like(b)
    r = b.clone()
    p = r.clone()
    rs = float(r @ r)
    it = 0
    for it in range(1, (max_iter or 10 * b.numel()) + 1):
        ap = a @ p
        alpha = rs / float(p @ ap)
        x, r = x + alpha * p, r - alpha * ap
        rn = float(r @ r)
        if math.sqrt(rn) <= tol * max(1.0, float(b.norm())):
            break
        p, rs = r + (rn / rs) * p, rn
    return x, it


def polyfit(xs, ys, degree: int = 1):
    x, y = torch.as_tensor(xs, dtype=torch.float64), torch.as_tensor(ys, dtype=torch.float64)
    if x.numel() != y.numel() or x.numel() <= degree:
        raise SymbolicError("need more points than the degree, and as many x as y")
    v = torch.stack([x ** i for i in range(degree + 1)], 1)
    co = torch.linalg.lstsq(v, y[:, None]).solution[:, 0]
    pred = v @ co
    ss_tot = float(((y - y.mean()) ** 2).sum())
    r2 = 1.0 - float(((y - pred) ** 2).sum()) / ss_tot if ss_tot > 0 else 1.0
    return co.tolist(), r2


def discover_patterns(data) -> list:
    d = [float(v) for v in data]
    if len(d) < 3:
        return []
    out = []
    inc = sum(1 for a, b in zip(d, d[1:]) if b > a)
    dec = sum(1 for a, b in zip(d, d[1:]) if b < a)
    total = len(d) - 1
    if inc / total > 0.7:
        out.append("trend_upward")
    elif dec / total > 0.7:
        out.append("trend_downward")
    mean = sum(d) / len(d)
    var = sum((v - mean) ** 2 for v in d) / len(d)
    if math.sqrt(var) / max(abs(mean), 1e-8) < 0.05:
        out.append("stable")
    return out


# ------------------------------------------------------------------ SAT (DPLL with unit propagation and pure literals)
def sat_solve(clauses):
    """Clauses are lists of non-zero ints (negative = negated). -> {var: bool} or None when unsatisfiable."""
    clauses = [list(dict.fromkeys(c)) for c in clauses]
    if any(0 in c for c in clauses):
        raise SymbolicError("0 is not a literal")

    def assign(cs, lit):
        out = []
        for c in cs:
            if lit in c:
                continue
            if -lit in c:
                c = [l for l in c if l != -lit]
                if not c:
                    return None
            out.append(c)
        return out

    def dpll(cs, model):
        while True:
            unit = next((c[0] for c in cs if len(c) == 1), None)
            if unit is None:
                break
            model = {**model, abs(unit): unit > 0}
            cs = assign(cs, unit)
            if cs is None:
                return None
        if not cs:
            return model
        lits = {l for c in cs for l in c}
        pure = next((l for l in sorted(lits, key=abs) if -l not in lits), None)
        if pure is not None:
            return dpll(assign(cs, pure), {**model, abs(pure): pure > 0})
        l = cs[0][0]
        for choice in (l, -l):
            nxt = assign(cs, choice)
            if nxt is not None:
                res = dpll(nxt, {**model, abs(choice): choice > 0})
                if res is not None:
                    return res
        return None

    model = dpll(clauses, {})
    if model is None:
        return None
    for v in {abs(l) for c in clauses for l in c}:
        model.setdefault(v, False)
    return model


# ------------------------------------------------------------------ symbolic regression over closed-form templates
def symreg(xs, ys, seed: int = 0):
    """Fit a dictionary of closed forms (each linear in its parameters after a fixed transform) by least squares and
    return the best by mean squared error + a small complexity charge -> (expression string, mse)."""
    x, y = torch.as_tensor(xs, dtype=torch.float64), torch.as_tensor(ys, dtype=torch.float64)
    if x.numel() != y.numel() or x.numel() < 3:
        raise SymbolicError("need at least three (x, y) pairs")
    cands = []

    def lin(cols, fmt, cost, tx=None, ty=None, inv=None):
        try:
            a = torch.stack(cols, 1)
            t = y if ty is None else ty(y)
            if not bool(torch.isfinite(a).all() and torch.isfinite(t).all()):
                return
            co = torch.linalg.lstsq(a, t[:, None]).solution[:, 0]
            pred = a @ co
            pred = pred if inv is None else inv(pred)
            mse = float(((pred - y) ** 2).mean())
            if math.isfinite(mse):
                cands.append((mse * (1 + 0.02 * cost) + 1e-12 * cost, mse, fmt(*[float(c) for c in co])))
        except RuntimeError:
            return

    one = torch.ones_like(x)
    g = lambda v: f"{v:.6g}"
    lin([one], lambda a: g(a), 1)
    lin([x, one], lambda a, b: f"{g(a)}*x + {g(b)}", 2)
    lin([x * x, x, one], lambda a, b, c: f"{g(a)}*x^2 + {g(b)}*x + {g(c)}", 3)
    lin([x ** 3, x * x, x, one], lambda a, b, c, d: f"{g(a)}*x^3 + {g(b)}*x^2 + {g(c)}*x + {g(d)}", 4)
    lin([torch.sin(x), torch.cos(x), one], lambda a, b, c: f"{g(a)}*sin(x) + {g(b)}*cos(x) + {g(c)}", 4)
    lin([torch.sqrt(x.clamp_min(0)), one], lambda a, b: f"{g(a)}*sqrt(x) + {g(b)}", 3) if bool((x >= 0).all()) else None
    lin([1.0 / x, one], lambda a, b: f"{g(a)}/x + {g(b)}", 3) if bool((x != 0).all()) else None
    if bool((x > 0).all()):
        lin([torch.log(x), one], lambda a, b: f"{g(a)}*ln(x) + {g(b)}", 3)
    if bool((y > 0).all()):
        lin([x, one], lambda b, la: f"{g(math.exp(la))}*exp({g(b)}*x)", 3, ty=torch.log, inv=torch.exp)
        if bool((x > 0).all()):
            lin([torch.log(x), one], lambda b, la: f"{g(math.exp(la))}*x^{g(b)}", 3, ty=torch.log, inv=torch.exp)
    if not cands:
        raise SymbolicError("no template could be fitted")
    _, mse, expr = min(cands)
    return expr, mse

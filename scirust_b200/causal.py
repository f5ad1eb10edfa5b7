"""Causal graphs, structural models and discovery.

* ``CausalGraph``: a DAG over named variables: parents / ancestors / descendants, topological order, d-separation (by
  reachability in the moralised ancestral graph), the back-door criterion and a search for a minimal adjustment set.
* ``LinearScm``: linear structural equations with Gaussian noise: batched sampling, ``do`` interventions, the total
  effect read off ``(I - B)^-1``, and unit-level counterfactuals (abduction of the noise, action, prediction).
* conditional independence: partial correlation from the precision matrix of the selected columns, Fisher's z test.
* ``pc_algorithm``: skeleton by conditional-independence tests of growing order, v-structures from the separating sets,
  Meek's rules 1-3 -> a CPDAG (directed and undirected edge sets).
* ``notears_linear``: continuous structure learning: least squares + l1 under the acyclicity function
  ``h(W) = tr(exp(W * W)) - d`` by an augmented Lagrangian, optimised with autograd (``torch.linalg.matrix_exp``), so it
  runs on a GPU for wide problems.
* effects: regression adjustment and inverse-probability weighting for a binary treatment.
Reference counterpart: scirust-causal/src/{graph,d_separation,adjustment,scm,intervention,partial_correlation,
conditional_independence,skeleton_discovery,orientation,cpdag,acyclicity,effect_estimation}.rs.
"""
from __future__ import annotations

import itertools
import math

import torch

D = torch.float64


class CausalError(ValueError):
    pass


class CausalGraph:
    def __init__(self, nodes=(), edges=()):
        self.nodes: list = []
        self.pa: dict = {}
        for n in nodes:
            self.add_node(n)
        for a, b in edges:
            self.add_edge(a, b)

    def add_node(self, n) -> None:
        if n not in self.pa:
            self.nodes.append(n)
            self.pa[n] = set()

    def add_edge(self, a, b) -> None:
        self.add_node(a)
        self.add_node(b)
        if a == b or a in self.descendants(b):
            raise CausalError(f"edge {a} -> {b} would close a cycle")
        self.pa[b].add(a)

    def parents(self, n) -> set:
        return set(self.pa[n])

    def children(self, n) -> set:
        return {c for c in self.nodes if n in self.pa[c]}

    def _closure(self, start, step) -> set:
        seen, stack = set(), list(start)
        while stack:
            for m in step(stack.pop()):
                if m not in seen:
                    seen.add(m)
                    stack.append(m)
        return seen

    def ancestors(self, n) -> set:
        return self._closure([n], self.parents)

    def descendants(self, n) -> set:
        return self._closure([n], self.children)

    def edges(self) -> list:
        return [(p, c) for c in self.nodes for p in sorted(self.pa[c], key=self.nodes.index)]

    def topological_order(self) -> list:
        out, done = [], set()
        while len(out) < len(self.nodes):
            for n in self.nodes:
                if n not in done and self.pa[n] <= done:
                    out.append(n)
                    done.add(n)
        return out

    def d_separated(self, xs, ys, zs=()) -> bool:
        """X and Y are d-separated by Z iff they are disconnected in the moral graph of the ancestral set of X, Y, Z
        once Z is removed."""
        xs, ys, zs = set(xs), set(ys), set(zs)
        if xs & ys:
            return False
        keep = set().union(xs, ys, zs, *(self.ancestors(n) for n in xs | ys | zs))
        adj = {n: set() for n in keep}
        for c in keep:
            ps = [p for p in self.pa[c] if p in keep]
            for p in ps:
                adj[p].add(c)
                adj[c].add(p)
            for p, q in itertools.combinations(ps, 2):                        # marry the parents
                adj[p].add(q)
                adj[q].add(p)
        reach = self._closure([x for x in xs if x not in zs], lambda n: [m for m in adj[n] if m not in zs]) | (xs - zs)
        return not (reach & ys)

    def satisfies_backdoor(self, x, y, zs) -> bool:
        zs = set(zs)
        if zs & (self.descendants(x) | {x, y}):
            return False
        cut = CausalGraph(self.nodes, [(a, b) for a, b in self.edges() if a != x])     # remove edges out of x
        return cut.d_separated([x], [y], zs)

    def minimal_adjustment_set(self, x, y):
        """Smallest back-door set among the non-descendants of x (ties: node order), or None."""
        cand = [n for n in self.nodes if n not in (x, y) and n not in self.descendants(x)]
        for k in range(len(cand) + 1):
            for zs in itertools.combinations(cand, k):
                if self.satisfies_backdoor(x, y, zs):
                    return list(zs)
        return None


# ------------------------------------------------------------------ linear structural causal models
class LinearScm:
    """``x_j = sum_i weights[i -> j] x_i + bias_j + sigma_j eps_j`` over the graph's topological order."""

    def __init__(self, graph: CausalGraph, weights: dict, noise_std=None, bias=None):
        self.graph, self.order = graph, graph.topological_order()
        self.index = {n: i for i, n in enumerate(self.order)}
        d = len(self.order)
        self.b = torch.zeros(d, d, dtype=D)                                   # b[i, j]: effect of i on j
        for (a, c), w in weights.items():
            if a not in graph.pa[c]:
                raise CausalError(f"weight given for {a} -> {c}, which is not an edge")
            self.b[self.index[a], self.index[c]] = w
        self.sigma = torch.tensor([(noise_std or {}).get(n, 1.0) for n in self.order], dtype=D)
        self.bias = torch.tensor([(bias or {}).get(n, 0.0) for n in self.order], dtype=D)

    def _solve(self, noise, do=None):
        x = torch.zeros_like(noise)
        for j, n in enumerate(self.order):
            if do and n in do:
                x[:, j] = float(do[n])
            else:
                x[:, j] = x @ self.b[:, j] + self.bias[j] + noise[:, j]
        return x

    def sample(self, n: int, seed: int = 0, do: dict | None = None):
        """-> (data [n, d] in ``self.order`` column order, the noise that produced it)."""
        g = torch.Generator().manual_seed(seed)
        noise = torch.randn(n, len(self.order), generator=g, dtype=D) * self.sigma
        return self._solve(noise, do), noise

    def total_effect(self, x, y) -> float:
        d = len(self.order)
        return float(torch.linalg.inv(torch.eye(d, dtype=D) - self.b)[self.index[x], self.index[y]])

    def counterfactual(self, observed: dict, do: dict) -> dict:
        """Abduction: recover every noise term from a fully observed unit; action: fix ``do``; prediction: re-solve."""
        x = torch.tensor([[float(observed[n]) for n in self.order]], dtype=D)
        noise = x - x @ self.b - self.bias
        out = self._solve(noise, do)[0]
        return {n: float(out[i]) for i, n in enumerate(self.order)}


# ------------------------------------------------------------------ conditional independence
def partial_correlation(data: torch.Tensor, i: int, j: int, cond=()) -> float:
    cols = [i, j] + list(cond)
    c = torch.corrcoef(data[:, cols].t().to(D))
    p = torch.linalg.pinv(c)
    return float((-p[0, 1] / torch.sqrt(p[0, 0] * p[1, 1])).clamp(-1.0, 1.0))


def fisher_z_test(data: torch.Tensor, i: int, j: int, cond=(), alpha: float = 0.05):
    """-> (independent?, p-value). z = atanh(r) sqrt(n - |cond| - 3) is standard normal under independence."""
    from .numerics.special import normal_cdf
    r = partial_correlation(data, i, j, cond)
    dof = data.shape[0] - len(cond) - 3
    if dof < 1:
        raise CausalError("too few observations for this conditioning set")
    z = math.atanh(max(min(r, 1 - 1e-12), -1 + 1e-12)) * math.sqrt(dof)
    p = 2.0 * (1.0 - float(normal_cdf(abs(z))))
    return p > alpha, p


# ------------------------------------------------------------------ PC algorithm
def pc_algorithm(data: torch.Tensor, names=None, alpha: float = 0.01, max_cond: int | None = None):
    """-> (directed edges [(a, b)], undirected edges [frozenset], separating sets)."""
    n_var = data.shape[1]
    names = list(names) if names is not None else list(range(n_var))
    adj = {i: set(range(n_var)) - {i} for i in range(n_var)}
    sep: dict = {}
    k = 0
    while (max_cond is None or k <= max_cond) and any(len(adj[i]) - 1 >= k for i in adj):
        for i in range(n_var):
            for j in sorted(adj[i]):
                if j not in adj[i]:
                    continue
                for cond in itertools.combinations(sorted(adj[i] - {j}), k):
                    if fisher_z_test(data, i, j, cond, alpha)[0]:
                        adj[i].discard(j)
                        adj[j].discard(i)
                        sep[frozenset((i, j))] = set(cond)
                        break
        k += 1
    directed = set()
    for b in range(n_var):                                                    # unshielded colliders a -> b <- c
        for a, c in itertools.combinations(sorted(adj[b]), 2):
            if c not in adj[a] and b not in sep.get(frozenset((a, c)), set()):
                directed |= {(a, b), (c, b)}
    directed = {(a, b) for a, b in directed if (b, a) not in directed}         # conflicting colliders stay undirected
    und = lambda a, b: b in adj[a] and (a, b) not in directed and (b, a) not in directed
    changed = True
    while changed:                                                            # Meek's rules 1-3
        changed = False
        for a, b in [(a, b) for a in range(n_var) for b in adj[a] if und(a, b)]:
            r1 = any((c, a) in directed and b not in adj[c] for c in adj[a] if c != b)
            r2 = any((a, c) in directed and (c, b) in directed for c in adj[a] & adj[b])
            r3 = any(und(a, c) and und(a, e) and (c, b) in directed and (e, b) in directed and e not in adj[c]
                     for c, e in itertools.combinations(sorted(adj[a] & adj[b]), 2))
            if (r1 or r2 or r3) and und(a, b):
                directed.add((a, b))
                changed = True
    undirected = {frozenset((names[a], names[b])) for a in range(n_var) for b in adj[a] if a < b and und(a, b)}
    return sorted((names[a], names[b]) for a, b in directed), undirected, {frozenset(names[i] for i in k_): {names[i] for i in v} for k_, v in sep.items()}


# ------------------------------------------------------------------ NOTEARS
def acyclicity(w: torch.Tensor) -> torch.Tensor:
    """``tr(exp(W * W)) - d``: zero exactly on weighted DAGs, positive otherwise, differentiable."""
    return torch.trace(torch.linalg.matrix_exp(w * w)) - w.shape[0]


def notears_linear(data: torch.Tensor, lam: float = 0.05, max_outer: int = 12, inner_steps: int = 300, h_tol: float = 1e-8,
                   threshold: float = 0.3, lr: float = 2e-2):
    """-> weighted adjacency ``W [d, d]`` (``W[i, j]``: i -> j) with small entries cut to zero."""
    x = (data - data.mean(0)).to(D)
    n, d = x.shape
    w = torch.zeros(d, d, dtype=D, device=x.device, requires_grad=True)
    mask = 1.0 - torch.eye(d, dtype=D, device=x.device)
    rho, alpha, h_prev = 1.0, 0.0, math.inf
    for _ in range(max_outer):
        opt = torch.optim.Adam([w], lr=lr)
        for _ in range(inner_steps):
            opt.zero_grad()
            wm = w * mask
            h = acyclicity(wm)
            loss = 0.5 / n * ((x - x @ wm) ** 2).sum() + lam * wm.abs().sum() + 0.5 * rho * h * h + alpha * h
            loss.backward()
            opt.step()
        with torch.no_grad():
            h_val = float(acyclicity(w * mask))
        if h_val > 0.25 * h_prev:
            rho *= 10.0
        alpha += rho * h_val
        h_prev = h_val
        if h_val <= h_tol or rho > 1e16:
            break
    out = (w * mask).detach().clone()
    out[out.abs() < threshold] = 0.0
    return out


# ------------------------------------------------------------------ effect estimation
def regression_adjustment(data: torch.Tensor, treatment: int, outcome: int, adjust=()) -> float:
    """Coefficient of the treatment in a linear regression of the outcome on treatment + adjustment set."""
    cols = [treatment] + list(adjust)
    a = torch.cat([torch.ones(data.shape[0], 1, dtype=D), data[:, cols].to(D)], 1)
    return float(torch.linalg.lstsq(a, data[:, outcome:outcome + 1].to(D)).solution[1, 0])


def ipw_effect(data: torch.Tensor, treatment: int, outcome: int, covariates, clip: float = 0.01, steps: int = 200) -> float:
    """Average treatment effect of a binary treatment: logistic propensity (Newton steps), normalised inverse weights."""
    t, y = data[:, treatment].to(D), data[:, outcome].to(D)
    a = torch.cat([torch.ones(data.shape[0], 1, dtype=D), data[:, list(covariates)].to(D)], 1)
    beta = torch.zeros(a.shape[1], dtype=D)
    for _ in range(steps):
        p = torch.sigmoid(a @ beta)
        grad = a.t() @ (t - p)
        hess = (a * (p * (1 - p))[:, None]).t() @ a + 1e-9 * torch.eye(a.shape[1], dtype=D)
        step = torch.linalg.solve(hess, grad)
        beta = beta + step
        if float(step.abs().max()) < 1e-10:
            break
    p = torch.sigmoid(a @ beta).clamp(clip, 1 - clip)
    w1, w0 = t / p, (1 - t) / (1 - p)
    return float((w1 * y).sum() / w1.sum() - (w0 * y).sum() / w0.sum())

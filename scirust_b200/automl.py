"""Model search: hyper-parameter optimisation, cross-validation, a small AutoML driver and an
evolutionary architecture search (scirust-automl/src/lib.rs:80-3400, scirust-nas/src/lib.rs:30-400).

Everything is seeded (xorshift64, as in the reference's search code) and runs on torch tensors in
fp64 on the host, so that two runs with one seed return the same trials in the same order.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

_MASK = (1 << 64) - 1


class XorShift64:
    """xorshift64 (13, 7, 17); a zero seed is replaced by the golden-ratio constant (lib.rs:17-75)."""

    def __init__(self, seed: int):
        self.s = (seed & _MASK) or 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & _MASK
        x ^= x >> 7
        x ^= (x << 17) & _MASK
        self.s = x
        return x

    def uniform(self, lo: float = 0.0, hi: float = 1.0) -> float:
        return lo + (hi - lo) * ((self.next_u64() >> 11) / float(1 << 53))

    def below(self, n: int) -> int:
        return self.next_u64() % n

    def shuffled(self, n: int) -> List[int]:
        v = list(range(n))
        for i in range(n - 1, 0, -1):
            j = self.below(i + 1)
            v[i], v[j] = v[j], v[i]
        return v


# ------------------------------------------------------------------ search spaces
@dataclass
class Uniform:
    lo: float
    hi: float

    def sample(self, rng):
        return rng.uniform(self.lo, self.hi)

    def to_unit(self, v):
        return (v - self.lo) / (self.hi - self.lo)

    def from_unit(self, u):
        return self.lo + u * (self.hi - self.lo)


@dataclass
class LogUniform:
    lo: float
    hi: float

    def sample(self, rng):
        return math.exp(rng.uniform(math.log(self.lo), math.log(self.hi)))

    def to_unit(self, v):
        return (math.log(v) - math.log(self.lo)) / (math.log(self.hi) - math.log(self.lo))

    def from_unit(self, u):
        return math.exp(math.log(self.lo) + u * (math.log(self.hi) - math.log(self.lo)))


@dataclass
class IntRange:
    lo: int
    hi: int

    def sample(self, rng):
        return self.lo + rng.below(self.hi - self.lo + 1)

    def to_unit(self, v):
        return (v - self.lo) / max(self.hi - self.lo, 1)

    def from_unit(self, u):
        return int(min(self.hi, max(self.lo, round(self.lo + u * (self.hi - self.lo)))))


@dataclass
class Choice:
    options: Sequence

    def sample(self, rng):
        return self.options[rng.below(len(self.options))]

    def to_unit(self, v):
        return list(self.options).index(v) / max(len(self.options) - 1, 1)

    def from_unit(self, u):
        return self.options[int(min(len(self.options) - 1, max(0, round(u * (len(self.options) - 1)))))]


# ------------------------------------------------------------------ metrics and splits
def metric_value(name: str, y: torch.Tensor, pred: torch.Tensor) -> float:
    """Score oriented so that larger is better: "neg_mse", "neg_mae", "r2", "accuracy"."""
    y, pred = y.double(), pred.double()
    if name == "neg_mse":
        return -float(((y - pred) ** 2).mean())
    if name == "neg_mae":
        return -float((y - pred).abs().mean())
    if name == "r2":
        ss = float(((y - y.mean()) ** 2).sum())
        return 1.0 - float(((y - pred) ** 2).sum()) / ss if ss > 0 else 0.0
    if name == "accuracy":
        return float((pred.round() == y.round()).double().mean())
    raise ValueError(name)


def k_fold_splits(n: int, k: int, rng: XorShift64) -> List[Tuple[List[int], List[int]]]:
    """Shuffled k-fold (train, validation) index lists with folds of ceil(n / k) (lib.rs:1717-1750)."""
    idx = rng.shuffled(n)
    size = -(-n // k)
    out = []
    for f in range(k):
        lo, hi = f * size, min((f + 1) * size, n)
        if lo < hi:
            out.append((idx[:lo] + idx[hi:], idx[lo:hi]))
    return out


def time_series_splits(n: int, n_splits: int) -> List[Tuple[List[int], List[int]]]:
    """Forward chaining: fold i trains on the first (i + 1) blocks and validates on the next one."""
    size = n // (n_splits + 1)
    return [(list(range(0, (i + 1) * size)), list(range((i + 1) * size, min((i + 2) * size, n))))
            for i in range(n_splits) if size > 0]


@dataclass
class CvResult:
    fold_train: List[float]
    fold_val: List[float]

    @property
    def mean(self) -> float:
        return sum(self.fold_val) / len(self.fold_val)

    @property
    def std(self) -> float:
        m = self.mean
        return math.sqrt(sum((v - m) ** 2 for v in self.fold_val) / len(self.fold_val))


# ------------------------------------------------------------------ models of the driver
class StandardScaler:
    def fit(self, x):
        self.mu, self.sd = x.mean(0), x.std(0, unbiased=False).clamp_min(1e-12)
        return self

    def transform(self, x):
        return (x - self.mu) / self.sd


class Ridge:
    def __init__(self, alpha: float = 1e-3):
        self.alpha = alpha

    def fit(self, x, y):
        xa = torch.cat([x, torch.ones(len(x), 1, dtype=x.dtype)], 1)
        a = xa.t() @ xa + self.alpha * torch.eye(xa.shape[1], dtype=x.dtype)
        self.w = torch.linalg.solve(a, xa.t() @ y)
        return self

    def predict(self, x):
        return torch.cat([x, torch.ones(len(x), 1, dtype=x.dtype)], 1) @ self.w


class KNN:
    def __init__(self, k: int = 5):
        self.k = k

    def fit(self, x, y):
        self.x, self.y = x, y
        return self

    def predict(self, x):
        d = torch.cdist(x, self.x)
        idx = d.topk(min(self.k, len(self.x)), largest=False).indices
        return self.y[idx].mean(1)


class MLP:
    def __init__(self, hidden: int = 32, lr: float = 1e-2, epochs: int = 200, seed: int = 0):
        self.hidden, self.lr, self.epochs, self.seed = hidden, lr, epochs, seed

    def fit(self, x, y):
        g = torch.Generator().manual_seed(self.seed)
        d = x.shape[1]
        self.p = [torch.randn(d, self.hidden, generator=g, dtype=x.dtype) / math.sqrt(d),
                  torch.zeros(self.hidden, dtype=x.dtype),
                  torch.randn(self.hidden, 1, generator=g, dtype=x.dtype) / math.sqrt(self.hidden),
                  torch.zeros(1, dtype=x.dtype)]
        for t in self.p:
            t.requires_grad_(True)
        opt = torch.optim.Adam(self.p, lr=self.lr)
        for _ in range(self.epochs):
            opt.zero_grad()
            ((self._fwd(x) - y) ** 2).mean().backward()
            opt.step()
        return self

    def _fwd(self, x):
        return (torch.tanh(x @ self.p[0] + self.p[1]) @ self.p[2] + self.p[3]).squeeze(1)

    def predict(self, x):
        with torch.no_grad():
            return self._fwd(x)


MODEL_KINDS: Dict[str, Callable] = {"ridge": Ridge, "knn": KNN, "mlp": MLP}
MODEL_SPACES: Dict[str, Dict[str, object]] = {
    "ridge": {"alpha": LogUniform(1e-6, 10.0)},
    "knn": {"k": IntRange(1, 15)},
    "mlp": {"hidden": IntRange(4, 64), "lr": LogUniform(1e-3, 5e-2)},
}


def cross_validate(make_model: Callable[[], object], x: torch.Tensor, y: torch.Tensor, splits, metric: str = "neg_mse",
                   scale: bool = True) -> CvResult:
    """Fits on each training fold (scaler fitted on that fold only) and scores both folds."""
    x, y = x.double(), y.double()
    tr_s, va_s = [], []
    for tr, va in splits:
        xt, xv = x[tr], x[va]
        if scale:
            sc = StandardScaler().fit(xt)
            xt, xv = sc.transform(xt), sc.transform(xv)
        m = make_model().fit(xt, y[tr])
        tr_s.append(metric_value(metric, y[tr], m.predict(xt)))
        va_s.append(metric_value(metric, y[va], m.predict(xv)))
    return CvResult(tr_s, va_s)


# ------------------------------------------------------------------ Bayesian optimisation
class GaussianProcess:
    """Zero-mean GP with an RBF kernel exp(-|a-b|^2 / (2 l^2)) and observation noise (lib.rs:1844-1930)."""

    def __init__(self, x: torch.Tensor, y: torch.Tensor, length_scale: float = 0.5, noise: float = 1e-6):
        self.x, self.l = x.double(), length_scale
        self.y_mean = float(y.double().mean())
        k = self._k(self.x, self.x) + noise * torch.eye(len(x), dtype=torch.float64)
        self.chol = torch.linalg.cholesky(k)
        self.alpha = torch.cholesky_solve((y.double() - self.y_mean).unsqueeze(1), self.chol)

    def _k(self, a, b):
        return torch.exp(-torch.cdist(a, b) ** 2 / (2 * self.l ** 2))

    def predict(self, xq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        ks = self._k(xq.double(), self.x)
        mu = (ks @ self.alpha).squeeze(1) + self.y_mean
        v = torch.cholesky_solve(ks.t(), self.chol)
        var = (1.0 - (ks * v.t()).sum(1)).clamp_min(0.0)
        return mu, var


def expected_improvement(gp: GaussianProcess, xq: torch.Tensor, y_best: float, xi: float = 0.01) -> torch.Tensor:
    """E[max(f - y_best - xi, 0)] under the GP posterior; zero where the posterior has no spread."""
    mu, var = gp.predict(xq)
    sigma = var.sqrt()
    z = (mu - y_best - xi) / sigma.clamp_min(1e-12)
    cdf = 0.5 * (1 + torch.erf(z / math.sqrt(2)))
    pdf = torch.exp(-0.5 * z * z) / math.sqrt(2 * math.pi)
    return torch.where(sigma < 1e-12, torch.zeros_like(mu), (mu - y_best - xi) * cdf + sigma * pdf)


def bayesian_optimize(f: Callable[[List[float]], float], bounds: Sequence[Tuple[float, float]], max_iter: int = 30,
                      initial_samples: int = 5, seed: int = 0, candidates: int = 512):
    """Maximises ``f`` over a box: random start-up samples, then at each step the candidate with the largest
    expected improvement among ``candidates`` seeded random points (the reference climbs EI by finite
    differences from 20 starts, lib.rs:1973-2050; a dense candidate set finds the same maxima without a
    step-size to tune). Returns (best_x, best_y, history)."""
    rng = XorShift64(seed)
    lo = torch.tensor([b[0] for b in bounds], dtype=torch.float64)
    hi = torch.tensor([b[1] for b in bounds], dtype=torch.float64)
    xs: List[List[float]] = []
    ys: List[float] = []
    for _ in range(min(initial_samples, max_iter)):
        x = [rng.uniform(a, b) for a, b in bounds]
        xs.append(x)
        ys.append(float(f(x)))
    for _ in range(max_iter - len(xs)):
        xu = (torch.tensor(xs, dtype=torch.float64) - lo) / (hi - lo)
        gp = GaussianProcess(xu, torch.tensor(ys, dtype=torch.float64))
        cand = torch.tensor([[rng.uniform() for _ in bounds] for _ in range(candidates)], dtype=torch.float64)
        ei = expected_improvement(gp, cand, max(ys))
        pick = cand[int(ei.argmax())]
        x = (lo + pick * (hi - lo)).tolist()
        xs.append(x)
        ys.append(float(f(x)))
    best = max(range(len(ys)), key=lambda i: ys[i])
    return xs[best], ys[best], list(zip(xs, ys))


def random_search(f: Callable[[Dict[str, object]], float], space: Dict[str, object], n_trials: int, seed: int = 0):
    """Seeded random search over a dict of distributions; returns (best_params, best_score, trials)."""
    rng = XorShift64(seed)
    trials = []
    for _ in range(n_trials):
        params = {k: d.sample(rng) for k, d in space.items()}
        trials.append((params, float(f(params))))
    best = max(trials, key=lambda t: t[1])
    return best[0], best[1], trials


def paired_t_test(a: Sequence[float], b: Sequence[float]) -> Dict[str, float]:
    """Paired t statistic of a - b with n - 1 degrees of freedom and a two-sided p-value from the
    regularised incomplete beta function (lib.rs:2334-2470)."""
    n = len(a)
    d = [x - y for x, y in zip(a, b)]
    mean = sum(d) / n
    var = sum((v - mean) ** 2 for v in d) / (n - 1) if n > 1 else 0.0
    if var <= 0:
        return {"t": 0.0 if mean == 0 else math.copysign(math.inf, mean), "df": n - 1, "p": 1.0 if mean == 0 else 0.0,
                "mean_diff": mean}
    t = mean / math.sqrt(var / n)
    df = n - 1
    xb = df / (df + t * t)
    p = _betainc(df / 2.0, 0.5, xb)
    return {"t": t, "df": df, "p": min(max(p, 0.0), 1.0), "mean_diff": mean}


def _betainc(a: float, b: float, x: float) -> float:
    """Regularised incomplete beta I_x(a, b) by Lentz's continued fraction."""
    if x <= 0:
        return 0.0
    if x >= 1:
        return 1.0
    if x > (a + 1) / (a + b + 2):
        return 1.0 - _betainc(b, a, 1 - x)
    lbeta = math.lgamma(a) + math.lgamma(b) - math.lgamma(a + b)
    front = math.exp(a * math.log(x) + b * math.log(1 - x) - lbeta) / a
    f, c, d = 1.0, 1.0, 0.0
    for i in range(0, 400):
        m = i // 2
        if i == 0:
            num = 1.0
        elif i % 2 == 0:
            num = m * (b - m) * x / ((a + 2 * m - 1) * (a + 2 * m))
        else:
            num = -(a + m) * (a + b + m) * x / ((a + 2 * m) * (a + 2 * m + 1))
        d = 1.0 + num * d
        d = 1.0 / (d if abs(d) > 1e-300 else 1e-300)
        c = 1.0 + num / (c if abs(c) > 1e-300 else 1e-300)
        f *= c * d
        if abs(1.0 - c * d) < 1e-14:
            break
    return front * (f - 1.0)


class ModelEnsemble:
    """Mean, weighted mean or majority vote of fitted models (lib.rs:2477-2610)."""

    def __init__(self, models: Sequence, method: str = "mean", weights: Optional[Sequence[float]] = None):
        self.models, self.method, self.weights = list(models), method, weights

    def predict(self, x):
        preds = torch.stack([m.predict(x) for m in self.models])
        if self.method == "mean":
            return preds.mean(0)
        if self.method == "weighted":
            w = torch.tensor(self.weights, dtype=preds.dtype)
            return (preds * (w / w.sum()).unsqueeze(1)).sum(0)
        if self.method == "vote":
            return preds.round().mode(0).values
        raise ValueError(self.method)


@dataclass
class AutoMLReport:
    best_kind: str
    best_params: Dict[str, object]
    best_score: float
    leaderboard: List[Tuple[str, Dict[str, object], float]]


class AutoML:
    """Tries every model kind with a seeded random search over its space, scores each trial by k-fold
    cross-validation, refits the winner on all data (lib.rs:3176-3400)."""

    def __init__(self, kinds: Sequence[str] = ("ridge", "knn", "mlp"), trials_per_kind: int = 6, k: int = 3,
                 metric: str = "neg_mse", seed: int = 0):
        self.kinds, self.trials, self.k, self.metric, self.seed = kinds, trials_per_kind, k, metric, seed

    def fit(self, x: torch.Tensor, y: torch.Tensor) -> AutoMLReport:
        x, y = x.double(), y.double()
        board = []
        for ki, kind in enumerate(self.kinds):
            splits = k_fold_splits(len(x), self.k, XorShift64(self.seed + 1))

            def score(params, kind=kind):
                return cross_validate(lambda: MODEL_KINDS[kind](**params), x, y, splits, self.metric).mean
            _, _, trials = random_search(score, MODEL_SPACES[kind], self.trials, seed=self.seed + 17 * (ki + 1))
            board += [(kind, p, s) for p, s in trials]
        board.sort(key=lambda t: -t[2])
        kind, params, s = board[0]
        self.scaler = StandardScaler().fit(x)
        self.model = MODEL_KINDS[kind](**params).fit(self.scaler.transform(x), y)
        return AutoMLReport(kind, params, s, board)

    def predict(self, x: torch.Tensor) -> torch.Tensor:
        return self.model.predict(self.scaler.transform(x.double()))


# ------------------------------------------------------------------ architecture search
ACTIVATIONS = ("relu", "gelu", "tanh", "silu")


@dataclass
class LayerSpec:
    kind: str                      # "linear" | "dropout" | "layernorm"
    out_features: int = 0
    activation: str = "relu"
    rate: float = 0.0

    def __str__(self):
        if self.kind == "linear":
            return f"Linear({self.out_features},{self.activation})"
        return f"Dropout({self.rate:.2f})" if self.kind == "dropout" else "LayerNorm"


@dataclass
class Architecture:
    layers: List[LayerSpec]
    fitness: float = 0.0
    params_m: float = 0.0
    flops: float = 0.0
    accuracy: Optional[float] = None

    def __str__(self):
        return "[" + " -> ".join(str(l) for l in self.layers) + f"] (fit={self.fitness:.4f}, {self.params_m:.4f}M params)"


@dataclass
class NasConfig:
    in_features: int = 64
    out_features: int = 10
    min_layers: int = 2
    max_layers: int = 8
    min_hidden: int = 32
    max_hidden: int = 1024
    accuracy_weight: float = 1.0
    params_weight: float = -0.1
    flops_weight: float = -0.05
    max_models: int = 500
    seed: int = 42


class NasSearch:
    """Evolutionary search over stacks of linear / dropout / layer-norm layers (lib.rs:176-370): the top half
    of the population survives, each survivor leaves one mutated child. Fitness is either the reference's
    zero-cost proxy (a bump at about four layers and half a million parameters, minus linear penalties on
    parameters and FLOPs) or a caller's ``score(arch) -> accuracy`` that trains the candidate."""

    def __init__(self, config: NasConfig = NasConfig(), score: Optional[Callable[[Architecture], float]] = None):
        self.config, self.score = config, score
        self.population: List[Architecture] = []
        self.evaluations = 0

    def costs(self, layers: Sequence[LayerSpec]) -> Tuple[float, float]:
        width, params, flops = self.config.in_features, 0.0, 0.0
        for l in layers:
            if l.kind == "linear":
                params += width * l.out_features + l.out_features
                flops += 2.0 * width * l.out_features
                width = l.out_features
            elif l.kind == "layernorm":
                params += 2 * width
        params += width * self.config.out_features + self.config.out_features
        flops += 2.0 * width * self.config.out_features
        return params / 1e6, flops

    def random_architecture(self, seed: int) -> Architecture:
        c = self.config
        rng = XorShift64(seed)
        n = c.min_layers + rng.below(c.max_layers - c.min_layers + 1)
        layers = []
        for _ in range(n):
            r = rng.below(10)
            if r < 7:
                layers.append(LayerSpec("linear", c.min_hidden + rng.below(c.max_hidden - c.min_hidden + 1),
                                        ACTIVATIONS[rng.below(len(ACTIVATIONS))]))
            elif r < 9:
                layers.append(LayerSpec("dropout", rate=0.1 * (1 + rng.below(5))))
            else:
                layers.append(LayerSpec("layernorm"))
        if not any(l.kind == "linear" for l in layers):
            layers[0] = LayerSpec("linear", c.min_hidden, "relu")
        a = Architecture(layers)
        a.params_m, a.flops = self.costs(layers)
        return a

    def evaluate(self, arch: Architecture) -> float:
        c = self.config
        if self.score is not None:
            arch.accuracy = float(self.score(arch))
            quality = arch.accuracy
        else:
            quality = math.exp(-(len(arch.layers) - 4.0) ** 2 / 8.0) * math.exp(-(arch.params_m - 0.5) ** 2 / 0.5)
        self.evaluations += 1
        return c.accuracy_weight * quality + c.params_weight * arch.params_m + c.flops_weight * arch.flops / 1e9

    def mutate(self, parent: Architecture, rng: XorShift64) -> Architecture:
        c = self.config
        layers = [LayerSpec(l.kind, l.out_features, l.activation, l.rate) for l in parent.layers]
        op = rng.below(4)
        i = rng.below(len(layers))
        if op == 0 or layers[i].kind != "linear":
            layers[i] = LayerSpec("linear", c.min_hidden + rng.below(c.max_hidden - c.min_hidden + 1),
                                  ACTIVATIONS[rng.below(len(ACTIVATIONS))])
        elif op == 1:
            layers[i].activation = ACTIVATIONS[rng.below(len(ACTIVATIONS))]
        elif op == 2 and len(layers) < c.max_layers:
            layers.insert(i, LayerSpec("linear", c.min_hidden + rng.below(c.max_hidden - c.min_hidden + 1), "gelu"))
        elif op == 3 and len(layers) > c.min_layers and sum(l.kind == "linear" for l in layers) > 1:
            del layers[i]
        child = Architecture(layers)
        child.params_m, child.flops = self.costs(layers)
        return child

    def evolve(self, generations: int, pop_size: int) -> List[Architecture]:
        c = self.config
        self.population = []
        for i in range(pop_size):
            a = self.random_architecture(((c.seed + i) * 0x9E3779B9) & _MASK)
            a.fitness = self.evaluate(a)
            self.population.append(a)
        self.population.sort(key=lambda a: -a.fitness)
        rng = XorShift64(c.seed ^ 0xA5A5A5A5)
        for _ in range(generations):
            survive = max(1, pop_size // 2)
            self.population = self.population[:survive]
            for i in range(survive):
                if self.evaluations >= c.max_models:
                    break
                child = self.mutate(self.population[i], rng)
                child.fitness = self.evaluate(child)
                self.population.append(child)
            self.population.sort(key=lambda a: -a.fitness)
        return list(self.population)


def build_module(arch: Architecture, in_features: int, out_features: int) -> torch.nn.Module:
    """The candidate as a ``torch.nn.Sequential`` ending in a linear read-out."""
    acts = {"relu": torch.nn.ReLU, "gelu": torch.nn.GELU, "tanh": torch.nn.Tanh, "silu": torch.nn.SiLU}
    mods, width = [], in_features
    for l in arch.layers:
        if l.kind == "linear":
            mods += [torch.nn.Linear(width, l.out_features), acts[l.activation]()]
            width = l.out_features
        elif l.kind == "dropout":
            mods.append(torch.nn.Dropout(l.rate))
        else:
            mods.append(torch.nn.LayerNorm(width))
    mods.append(torch.nn.Linear(width, out_features))
    return torch.nn.Sequential(*mods)

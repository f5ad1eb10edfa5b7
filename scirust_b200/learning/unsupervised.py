"""Clustering, density models and anomaly detectors on ``[n, d]`` tensors; distance matrices and EM steps are single
batched tensor operations, so they run unchanged on a GPU for large ``n``.

``KMeans`` (k-means++ seeding, several restarts evaluated one after another with one seed each), ``Pca`` (SVD of the centred
data), ``Dbscan`` (density-reachable expansion over a boolean neighbourhood matrix; label -1 = noise),
``LocalOutlierFactor`` (k-distance, reachability, local reachability density), ``GaussianMixture`` (full covariances,
log-sum-exp E step, ridge on the covariances, BIC / AIC), ``IsolationForest`` (random axis-parallel splits on
sub-samples; score 2^{-E[h] / c(psi)}), ``AutoencoderDetector`` (reconstruction error of a small MLP trained with Adam).
Reference counterpart: scirust-unsupervised/src/lib.rs (Autoencoder, IsolationForest, Dbscan, LocalOutlierFactor,
GaussianMixtureModel)."""
from __future__ import annotations

import math

import torch

D = torch.float64


def _x(x):
    x = torch.as_tensor(x, dtype=D)
    if x.dim() != 2 or x.shape[0] == 0:
        raise ValueError("expected a non-empty [n, d] matrix")
    return x


class KMeans:
    def __init__(self, k: int, restarts: int = 4, max_iter: int = 100, seed: int = 0):
        self.k, self.restarts, self.max_iter, self.seed = k, restarts, max_iter, seed
        self.centers = None
        self.inertia = math.inf

    def _seed(self, x, g):
        c = [x[int(torch.randint(x.shape[0], (1,), generator=g))]]
        for _ in range(1, self.k):
            d2 = torch.cdist(x, torch.stack(c)).min(1).values ** 2
            tot = float(d2.sum())
            i = int(torch.multinomial(d2 / tot, 1, generator=g)) if tot > 0 else int(torch.randint(x.shape[0], (1,), generator=g))
            c.append(x[i])
        return torch.stack(c)

    def fit(self, x):
        x = _x(x)
        if not 1 <= self.k <= x.shape[0]:
            raise ValueError("1 <= k <= n")
        for r in range(self.restarts):
            g = torch.Generator().manual_seed(self.seed + r)
            c = self._seed(x.cpu(), g).to(x.device)
            lab = None
            for _ in range(self.max_iter):
                new = torch.cdist(x, c).argmin(1)
                if lab is not None and torch.equal(new, lab):
                    break
                lab = new
                one = torch.nn.functional.one_hot(lab, self.k).to(D)
                cnt = one.sum(0)
                c = torch.where(cnt[:, None] > 0, (one.t() @ x) / cnt.clamp_min(1)[:, None], c)
            inertia = float((torch.cdist(x, c).min(1).values ** 2).sum())
            if inertia < self.inertia:
                self.inertia, self.centers = inertia, c
        return self

    def predict(self, x):
        return torch.cdist(_x(x).to(self.centers.device), self.centers).argmin(1)


class Pca:
    def __init__(self, components: int):
        self.components = components

    def fit(self, x):
        x = _x(x)
        self.mean = x.mean(0)
        _, s, vt = torch.linalg.svd(x - self.mean, full_matrices=False)
        self.axes = vt[:self.components]
        var = s ** 2 / max(1, x.shape[0] - 1)
        self.explained_variance = var[:self.components]
        self.explained_ratio = self.explained_variance / var.sum()
        return self

    def transform(self, x):
        return (_x(x) - self.mean) @ self.axes.t()

    def inverse_transform(self, z):
        return z @ self.axes + self.mean


class Dbscan:
    def __init__(self, eps: float, min_points: int = 5):
        if eps <= 0 or min_points < 1:
            raise ValueError("eps > 0 and min_points >= 1")
        self.eps, self.min_points = eps, min_points

    def fit(self, x):
        """-> labels [n] (cluster ids from 0, -1 for noise); ``self.core`` marks the core points."""
        x = _x(x)
        near = torch.cdist(x, x) <= self.eps
        core = near.sum(1) >= self.min_points
        labels = torch.full((x.shape[0],), -1, dtype=torch.long)
        cid = 0
        for i in range(x.shape[0]):
            if not bool(core[i]) or int(labels[i]) != -1:
                continue
            member = torch.zeros(x.shape[0], dtype=torch.bool)
            frontier = torch.zeros_like(member)
            frontier[i] = True
            while bool(frontier.any()):
                member |= frontier
                reach = near[frontier & core].any(0) if bool((frontier & core).any()) else torch.zeros_like(member)
                frontier = reach & ~member
            labels[member & (labels == -1)] = cid
            cid += 1
        self.core, self.n_clusters = core, cid
        return labels


class LocalOutlierFactor:
    def __init__(self, k: int = 20):
        self.k = k

    def fit_predict(self, x):
        """-> LOF score per point (about 1 inside a cluster, well above 1 for outliers)."""
        x = _x(x)
        k = min(self.k, x.shape[0] - 1)
        if k < 1:
            raise ValueError("need at least two points")
        d = torch.cdist(x, x)
        d.fill_diagonal_(math.inf)
        nd, ni = d.topk(k, dim=1, largest=False)
        kdist = nd[:, -1]
        reach = torch.maximum(nd, kdist[ni])
        lrd = 1.0 / reach.mean(1).clamp_min(1e-300)
        return lrd[ni].mean(1) / lrd

    def detect_outliers(self, x, threshold: float = 1.5):
        return torch.nonzero(self.fit_predict(x) > threshold)[:, 0].tolist()


class GaussianMixture:
    def __init__(self, components: int, max_iter: int = 200, tol: float = 1e-8, ridge: float = 1e-6, seed: int = 0):
        self.k, self.max_iter, self.tol, self.ridge, self.seed = components, max_iter, tol, ridge, seed

    def _log_prob(self, x):
        l = torch.linalg.cholesky(self.cov)                                   # [k, d, d]
        diff = x[None, :, :] - self.means[:, None, :]                         # [k, n, d]
        z = torch.linalg.solve_triangular(l, diff.transpose(1, 2), upper=False)
        maha = (z * z).sum(1)                                                 # [k, n]
        logdet = 2 * torch.log(torch.diagonal(l, dim1=1, dim2=2)).sum(1)
        d = x.shape[1]
        return (torch.log(self.weights)[:, None] - 0.5 * (maha + logdet[:, None] + d * math.log(2 * math.pi))).t()

    def fit(self, x):
        x = _x(x)
        n, d = x.shape
        km = KMeans(self.k, restarts=2, seed=self.seed).fit(x)
        self.means = km.centers.clone()
        self.weights = torch.full((self.k,), 1.0 / self.k, dtype=D)
        self.cov = (torch.cov(x.t()).reshape(d, d) + self.ridge * torch.eye(d, dtype=D)).expand(self.k, d, d).clone()
        prev = -math.inf
        self.converged, self.iterations = False, 0
        for it in range(1, self.max_iter + 1):
            lp = self._log_prob(x)
            norm = torch.logsumexp(lp, 1)
            ll = float(norm.mean())
            resp = torch.exp(lp - norm[:, None])
            nk = resp.sum(0).clamp_min(1e-12)
            self.weights = nk / n
            self.means = (resp.t() @ x) / nk[:, None]
            diff = x[None] - self.means[:, None]
            self.cov = torch.einsum("nk,knd,kne->kde", resp, diff, diff) / nk[:, None, None] + self.ridge * torch.eye(d, dtype=D)
            self.iterations = it
            if abs(ll - prev) <= self.tol * (1 + abs(ll)):
                self.converged = True
                break
            prev = ll
        self.n, self.d = n, d
        return self

    def predict_proba(self, x):
        lp = self._log_prob(_x(x))
        return torch.exp(lp - torch.logsumexp(lp, 1, keepdim=True))

    def predict(self, x):
        return self._log_prob(_x(x)).argmax(1)

    def score(self, x) -> float:
        """Mean log-likelihood per observation."""
        return float(torch.logsumexp(self._log_prob(_x(x)), 1).mean())

    def _free_parameters(self):
        return self.k - 1 + self.k * self.d + self.k * self.d * (self.d + 1) // 2

    def bic(self, x) -> float:
        x = _x(x)
        return -2 * self.score(x) * x.shape[0] + self._free_parameters() * math.log(x.shape[0])

    def aic(self, x) -> float:
        x = _x(x)
        return -2 * self.score(x) * x.shape[0] + 2 * self._free_parameters()


def _c_factor(n: int) -> float:
    """Average path length of an unsuccessful search in a binary search tree of n nodes."""
    return 0.0 if n <= 1 else 2.0 * (math.log(n - 1) + 0.5772156649015329) - 2.0 * (n - 1) / n if n > 2 else 1.0


class IsolationForest:
    def __init__(self, trees: int = 100, sample_size: int = 256, seed: int = 0):
        self.trees, self.sample_size, self.seed = trees, sample_size, seed

    def fit(self, x):
        x = _x(x).cpu()
        g = torch.Generator().manual_seed(self.seed)
        psi = min(self.sample_size, x.shape[0])
        limit = max(1, math.ceil(math.log2(max(psi, 2))))
        self.psi, self.forest = psi, []

        def grow(rows, depth):
            if depth >= limit or rows.shape[0] <= 1:
                return ("leaf", rows.shape[0])
            lo, hi = rows.min(0).values, rows.max(0).values
            ok = torch.nonzero(hi > lo)[:, 0]
            if ok.numel() == 0:
                return ("leaf", rows.shape[0])
            f = int(ok[int(torch.randint(ok.numel(), (1,), generator=g))])
            cut = float(lo[f] + (hi[f] - lo[f]) * torch.rand((), generator=g, dtype=D))
            left = rows[:, f] < cut
            return ("node", f, cut, grow(rows[left], depth + 1), grow(rows[~left], depth + 1))

        for _ in range(self.trees):
            self.forest.append(grow(x[torch.randperm(x.shape[0], generator=g)[:psi]], 0))
        return self

    def _depths(self, tree, x, idx, depth, out):
        if tree[0] == "leaf":
            out[idx] += depth + _c_factor(tree[1])
            return
        _, f, cut, l, r = tree
        left = x[idx, f] < cut
        if bool(left.any()):
            self._depths(l, x, idx[left], depth + 1, out)
        if bool((~left).any()):
            self._depths(r, x, idx[~left], depth + 1, out)

    def anomaly_scores(self, x):
        x = _x(x).cpu()
        total = torch.zeros(x.shape[0], dtype=D)
        for t in self.forest:
            self._depths(t, x, torch.arange(x.shape[0]), 0, total)
        return torch.pow(2.0, -(total / len(self.forest)) / _c_factor(self.psi))

    def detect_anomalies(self, x, threshold: float = 0.6):
        return torch.nonzero(self.anomaly_scores(x) > threshold)[:, 0].tolist()


class AutoencoderDetector:
    def __init__(self, in_dim: int, hidden: int = 8, latent: int = 2, seed: int = 0):
        torch.manual_seed(seed)
        self.net = torch.nn.Sequential(torch.nn.Linear(in_dim, hidden), torch.nn.Tanh(), torch.nn.Linear(hidden, latent),
                                       torch.nn.Linear(latent, hidden), torch.nn.Tanh(), torch.nn.Linear(hidden, in_dim)).to(D)
        self.mean = self.std = None

    def train(self, x, epochs: int = 300, lr: float = 1e-2):
        x = _x(x)
        self.mean, self.std = x.mean(0), x.std(0).clamp_min(1e-9)
        z = (x - self.mean) / self.std
        opt = torch.optim.Adam(self.net.parameters(), lr=lr)
        loss = None
        for _ in range(epochs):
            opt.zero_grad()
            loss = ((self.net(z) - z) ** 2).mean()
            loss.backward()
            opt.step()
        return float(loss.detach())

    @torch.no_grad()
    def anomaly_scores(self, x):
        z = (_x(x) - self.mean) / self.std
        return ((self.net(z) - z) ** 2).mean(1)

    def detect_anomalies(self, x, threshold: float):
        return torch.nonzero(self.anomaly_scores(x) > threshold)[:, 0].tolist()

"""Sequence models and alignment.

* ``Hmm``: discrete hidden Markov model in log space: the forward / backward recursions take a BATCH of equal-length
  observation sequences at once (``[batch, T]``), Viterbi decoding, Baum-Welch re-estimation over the batch.
* ``LinearChainCrf``: emission and transition scores as parameters, the log-partition by the forward recursion
  (``logsumexp``), so the negative log-likelihood is differentiable and its gradient comes from autograd (equal to
  expected minus observed feature counts); Viterbi decoding; fitting with any optimizer.
* labelling helpers: BIO spans, validation; alignment: Needleman-Wunsch, edit distance, longest common subsequence,
  dynamic time warping with its path; exact matching: Knuth-Morris-Pratt, Boyer-Moore (bad-character rule).
Reference counterpart: scirust-sequential/src/{hmm,crf,labeling,matching}.rs.
"""
from __future__ import annotations

import math

import torch

D = torch.float64
NEG = -1e30


def _log(p):
    return torch.log(torch.as_tensor(p, dtype=D).clamp_min(1e-300))


class Hmm:
    def __init__(self, initial, transition, emission):
        self.log_pi, self.log_a, self.log_b = _log(initial), _log(transition), _log(emission)
        n = self.log_pi.shape[0]
        if self.log_a.shape != (n, n) or self.log_b.shape[0] != n:
            raise ValueError("shapes: initial [n], transition [n, n], emission [n, symbols]")
        for name, p in (("initial", initial), ("transition", transition), ("emission", emission)):
            if float((torch.as_tensor(p, dtype=D).sum(-1) - 1).abs().max()) > 1e-8:
                raise ValueError(f"{name} probabilities must sum to one")

    @property
    def n_states(self):
        return self.log_pi.shape[0]

    def _obs(self, obs):
        o = torch.as_tensor(obs, dtype=torch.long)
        return o[None] if o.dim() == 1 else o

    def forward(self, obs) -> torch.Tensor:
        """-> log alpha ``[batch, T, n]``."""
        o = self._obs(obs)
        em = self.log_b.t()[o]                                                # [batch, T, n]
        alpha = [self.log_pi + em[:, 0]]
        for t in range(1, o.shape[1]):
            alpha.append(torch.logsumexp(alpha[-1][:, :, None] + self.log_a, 1) + em[:, t])
        return torch.stack(alpha, 1)

    def backward(self, obs) -> torch.Tensor:
        o = self._obs(obs)
        em = self.log_b.t()[o]
        beta = [torch.zeros(o.shape[0], self.n_states, dtype=D)]
        for t in range(o.shape[1] - 1, 0, -1):
            beta.append(torch.logsumexp(self.log_a + (em[:, t] + beta[-1])[:, None, :], 2))
        return torch.stack(beta[::-1], 1)

    def log_probability(self, obs) -> torch.Tensor:
        out = torch.logsumexp(self.forward(obs)[:, -1], 1)
        return out[0] if torch.as_tensor(obs).dim() == 1 else out

    def viterbi(self, obs):
        """-> (best state path, its log probability) for one sequence."""
        o = torch.as_tensor(obs, dtype=torch.long)
        delta = self.log_pi + self.log_b[:, o[0]]
        back = []
        for t in range(1, o.shape[0]):
            cand = delta[:, None] + self.log_a
            best = cand.max(0)
            back.append(best.indices)
            delta = best.values + self.log_b[:, o[t]]
        path = [int(delta.argmax())]
        for b in reversed(back):
            path.append(int(b[path[-1]]))
        return path[::-1], float(delta.max())

    def baum_welch(self, obs, iters: int = 50, tol: float = 1e-8):
        """Re-estimate all three tables on a batch of sequences -> list of total log-likelihoods per iteration."""
        o = self._obs(obs)
        hist = []
        n_sym = self.log_b.shape[1]
        onehot = torch.nn.functional.one_hot(o, n_sym).to(D)                  # [batch, T, symbols]
        for _ in range(iters):
            la, lb = self.forward(o), self.backward(o)
            ll = torch.logsumexp(la[:, -1], 1)
            hist.append(float(ll.sum()))
            gamma = torch.exp(la + lb - ll[:, None, None])                    # [batch, T, n]
            em = self.log_b.t()[o]
            xi = torch.exp(la[:, :-1, :, None] + self.log_a + (em[:, 1:] + lb[:, 1:])[:, :, None, :] - ll[:, None, None, None])
            self.log_pi = _log(gamma[:, 0].mean(0))
            self.log_a = _log(xi.sum((0, 1)) / gamma[:, :-1].sum((0, 1))[:, None])
            self.log_b = _log(torch.einsum("btn,bts->ns", gamma, onehot) / gamma.sum((0, 1))[:, None])
            if len(hist) > 1 and abs(hist[-1] - hist[-2]) <= tol * (1 + abs(hist[-1])):
                break
        return hist

    def sample(self, length: int, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        states, obs = [], []
        s = int(torch.multinomial(self.log_pi.exp(), 1, generator=g))
        for _ in range(length):
            states.append(s)
            obs.append(int(torch.multinomial(self.log_b[s].exp(), 1, generator=g)))
            s = int(torch.multinomial(self.log_a[s].exp(), 1, generator=g))
        return states, obs


class LinearChainCrf(torch.nn.Module):
    """Scores: ``emission_weights [features, labels]`` applied to per-position feature vectors, ``transitions [labels,
    labels]``, ``start`` and ``end`` vectors."""

    def __init__(self, n_features: int, n_labels: int):
        super().__init__()
        self.w = torch.nn.Parameter(torch.zeros(n_features, n_labels, dtype=D))
        self.trans = torch.nn.Parameter(torch.zeros(n_labels, n_labels, dtype=D))
        self.start = torch.nn.Parameter(torch.zeros(n_labels, dtype=D))
        self.end = torch.nn.Parameter(torch.zeros(n_labels, dtype=D))

    def _em(self, feats):
        f = torch.as_tensor(feats, dtype=D)
        return (f[None] if f.dim() == 2 else f) @ self.w                      # [batch, T, labels]

    def log_partition(self, feats) -> torch.Tensor:
        em = self._em(feats)
        alpha = self.start + em[:, 0]
        for t in range(1, em.shape[1]):
            alpha = torch.logsumexp(alpha[:, :, None] + self.trans, 1) + em[:, t]
        return torch.logsumexp(alpha + self.end, 1)

    def score(self, feats, labels) -> torch.Tensor:
        em = self._em(feats)
        y = torch.as_tensor(labels, dtype=torch.long)
        y = y[None] if y.dim() == 1 else y
        s = self.start[y[:, 0]] + self.end[y[:, -1]] + em.gather(2, y[:, :, None])[:, :, 0].sum(1)
        return s + self.trans[y[:, :-1], y[:, 1:]].sum(1)

    def nll(self, feats, labels) -> torch.Tensor:
        return (self.log_partition(feats) - self.score(feats, labels)).mean()

    def marginals(self, feats) -> torch.Tensor:
        """Posterior label probabilities ``[batch, T, labels]`` = gradient of the log-partition w.r.t. the emissions."""
        em = self._em(feats).detach().requires_grad_(True)
        alpha = self.start + em[:, 0]
        for t in range(1, em.shape[1]):
            alpha = torch.logsumexp(alpha[:, :, None] + self.trans, 1) + em[:, t]
        torch.logsumexp(alpha + self.end, 1).sum().backward()
        return em.grad

    @torch.no_grad()
    def decode(self, feats) -> list:
        em = self._em(feats)[0]
        delta, back = self.start + em[0], []
        for t in range(1, em.shape[0]):
            best = (delta[:, None] + self.trans).max(0)
            back.append(best.indices)
            delta = best.values + em[t]
        path = [int((delta + self.end).argmax())]
        for b in reversed(back):
            path.append(int(b[path[-1]]))
        return path[::-1]

    def fit(self, feats, labels, steps: int = 200, lr: float = 0.1, l2: float = 1e-3) -> list:
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        hist = []
        for _ in range(steps):
            opt.zero_grad()
            loss = self.nll(feats, labels) + l2 * sum((p ** 2).sum() for p in self.parameters())
            loss.backward()
            opt.step()
            hist.append(float(loss.detach()))
        return hist


# ------------------------------------------------------------------ labelling
def extract_spans(tags) -> list:
    """BIO tags -> [(type, start, end_exclusive)]; an ``I-`` that does not continue a span of its type opens one."""
    spans, cur = [], None
    for i, t in enumerate(list(tags) + ["O"]):
        kind = t[2:] if t[:2] in ("B-", "I-") else None
        if cur and (t == "O" or t.startswith("B-") or kind != cur[0]):
            spans.append((cur[0], cur[1], i))
            cur = None
        if kind and cur is None:
            cur = (kind, i)
    return spans


def validate_bio(tags) -> list:
    """Positions where an ``I-X`` follows neither ``B-X`` nor ``I-X``, or a tag is malformed."""
    bad, prev = [], "O"
    for i, t in enumerate(tags):
        if t != "O" and t[:2] not in ("B-", "I-") or t in ("B-", "I-"):
            bad.append(i)
        elif t.startswith("I-") and prev[2:] != t[2:]:
            bad.append(i)
        prev = t if t != "O" else "O-"
    return bad


# ------------------------------------------------------------------ alignment and matching
def needleman_wunsch(a, b, match: float = 1.0, mismatch: float = -1.0, gap: float = -1.0):
    """Global alignment -> (score, aligned a, aligned b) with ``None`` for gaps."""
    n, m = len(a), len(b)
    s = [[0.0] * (m + 1) for _ in range(n + 1)]
    for i in range(1, n + 1):
        s[i][0] = i * gap
    for j in range(1, m + 1):
        s[0][j] = j * gap
    for i in range(1, n + 1):
        for j in range(1, m + 1):
            s[i][j] = max(s[i - 1][j - 1] + (match if a[i - 1] == b[j - 1] else mismatch), s[i - 1][j] + gap, s[i][j - 1] + gap)
    i, j, ra, rb = n, m, [], []
    while i or j:
        if i and j and s[i][j] == s[i - 1][j - 1] + (match if a[i - 1] == b[j - 1] else mismatch):
            ra.append(a[i - 1]); rb.append(b[j - 1]); i -= 1; j -= 1
        elif i and s[i][j] == s[i - 1][j] + gap:
            ra.append(a[i - 1]); rb.append(None); i -= 1
        else:
            ra.append(None); rb.append(b[j - 1]); j -= 1
    return s[n][m], ra[::-1], rb[::-1]


def edit_distance(a, b) -> int:
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i]
        for j, y in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[-1] + 1, prev[j - 1] + (x != y)))
        prev = cur
    return prev[-1]


def longest_common_subsequence(a, b) -> list:
    n, m = len(a), len(b)
    l = [[0] * (m + 1) for _ in range(n + 1)]
    for i in range(n):
        for j in range(m):
            l[i + 1][j + 1] = l[i][j] + 1 if a[i] == b[j] else max(l[i][j + 1], l[i + 1][j])
    out, i, j = [], n, m
    while i and j:
        if a[i - 1] == b[j - 1]:
            out.append(a[i - 1]); i -= 1; j -= 1
        elif l[i - 1][j] >= l[i][j - 1]:
            i -= 1
        else:
            j -= 1
    return out[::-1]


def dynamic_time_warping(a, b, with_path: bool = False):
    """Cost of the best monotone alignment of two numeric series (absolute difference as local cost)."""
    x, y = torch.as_tensor(a, dtype=D).reshape(-1), torch.as_tensor(b, dtype=D).reshape(-1)
    cost = (x[:, None] - y[None, :]).abs().tolist()
    n, m = len(cost), len(cost[0])
    acc = [[math.inf] * (m + 1) for _ in range(n + 1)]
    acc[0][0] = 0.0
    for i in range(1, n + 1):
        for j in range(1, m + 1):
            acc[i][j] = cost[i - 1][j - 1] + min(acc[i - 1][j], acc[i][j - 1], acc[i - 1][j - 1])
    if not with_path:
        return acc[n][m]
    path, i, j = [], n, m
    while i and j:
        path.append((i - 1, j - 1))
        step = min((acc[i - 1][j - 1], 0), (acc[i - 1][j], 1), (acc[i][j - 1], 2))[1]
        i, j = (i - 1, j - 1) if step == 0 else (i - 1, j) if step == 1 else (i, j - 1)
    return acc[n][m], path[::-1]


def kmp(text, pattern) -> list:
    """Start positions of every (possibly overlapping) occurrence."""
    if not pattern:
        return list(range(len(text) + 1))
    fail, k = [0] * len(pattern), 0
    for i in range(1, len(pattern)):
        while k and pattern[i] != pattern[k]:
            k = fail[k - 1]
        k += pattern[i] == pattern[k]
        fail[i] = k
    out, k = [], 0
    for i, c in enumerate(text):
        while k and c != pattern[k]:
            k = fail[k - 1]
        k += c == pattern[k]
        if k == len(pattern):
            out.append(i - k + 1)
            k = fail[k - 1]
    return out


def boyer_moore(text, pattern) -> list:
    if not pattern:
        return list(range(len(text) + 1))
    last = {c: i for i, c in enumerate(pattern)}
    out, s, m = [], 0, len(pattern)
    while s <= len(text) - m:
        j = m - 1
        while j >= 0 and pattern[j] == text[s + j]:
            j -= 1
        if j < 0:
            out.append(s)
            s += 1
        else:
            s += max(1, j - last.get(text[s + j], -1))
    return out

"""Weight pruning on tensors of any device: unstructured magnitude pruning, structured row / column pruning by L2
norm, Wanda (|w| times the input-activation norm, per output row), N:M structured sparsity (2:4 is the pattern the
tensor cores' sparse mode consumes) and iterative lottery-ticket pruning with rewinding.

All selections are deterministic: candidates are ordered by score, ties by index (a stable sort of the scores), and
exactly ``floor(n * sparsity)`` entries are removed. Inputs must be finite; sparsity must lie in [0, 1]. Tensors are
pruned IN PLACE and returned. Reference counterpart: scirust-core/src/pruning.rs:26-430 (flat f32 slices, row-major
``(rows, cols)``); N:M pruning has no counterpart there.
"""
from __future__ import annotations

import enum
import math

import torch


class PruningMethod(enum.Enum):
    MAGNITUDE = "magnitude"
    STRUCTURED_COLUMNS = "structured_columns"
    STRUCTURED_ROWS = "structured_rows"


def _check(op, w, sparsity):
    if not isinstance(sparsity, (int, float)) or not math.isfinite(sparsity) or not 0.0 <= sparsity <= 1.0:
        raise ValueError(f"{op}: sparsity must be finite and in [0, 1], got {sparsity}")
    bad = torch.nonzero(~torch.isfinite(w.reshape(-1)))
    if bad.numel():
        i = int(bad[0])
        raise ValueError(f"{op}: weight at index {i} must be finite, got {float(w.reshape(-1)[i])}")


def _count(n: int, sparsity: float) -> int:
    return int(math.floor(n * float(sparsity)))


def _smallest(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k smallest scores, ties to the lower index."""
    return torch.sort(scores, stable=True).indices[:k]


@torch.no_grad()
def prune_magnitude(weights: torch.Tensor, sparsity: float) -> torch.Tensor:
    _check("prune_magnitude", weights, sparsity)
    k = _count(weights.numel(), sparsity)
    if k:
        weights.view(-1)[_smallest(weights.reshape(-1).abs(), k)] = 0.0
    return weights


def _matrix(op, w, rows, cols):
    if rows is None:
        if w.dim() != 2:
            raise ValueError(f"{op}: expected a matrix")
        return w
    if w.numel() != rows * cols:
        raise ValueError(f"{op}: expected {rows * cols} weights for shape ({rows}, {cols}), got {w.numel()}")
    return w.view(rows, cols)


@torch.no_grad()
def prune_structured_columns(weights, rows=None, cols=None, sparsity: float = 0.0) -> torch.Tensor:
    _check("prune_structured_columns", weights, sparsity)
    W = _matrix("prune_structured_columns", weights, rows, cols)
    k = _count(W.shape[1], sparsity)
    if k:
        W[:, _smallest(W.double().pow(2).sum(0).sqrt(), k)] = 0.0
    return weights


@torch.no_grad()
def prune_structured_rows(weights, rows=None, cols=None, sparsity: float = 0.0) -> torch.Tensor:
    _check("prune_structured_rows", weights, sparsity)
    W = _matrix("prune_structured_rows", weights, rows, cols)
    k = _count(W.shape[0], sparsity)
    if k:
        W[_smallest(W.double().pow(2).sum(1).sqrt(), k)] = 0.0
    return weights


@torch.no_grad()
def prune_wanda(weights, input_norms, sparsity: float, out=None, in_features=None) -> torch.Tensor:
    """``weights [out, in]``; per output row, drop the ``floor(in * sparsity)`` entries with the smallest
    ``|w_ij| * ||x_j||`` (``input_norms [in]``: activation norms collected on calibration data)."""
    _check("prune_wanda", weights, sparsity)
    W = _matrix("prune_wanda", weights, out, in_features)
    xn = torch.as_tensor(input_norms, dtype=torch.float32, device=W.device).reshape(-1)
    if xn.numel() != W.shape[1]:
        raise ValueError(f"prune_wanda: expected {W.shape[1]} input norms, got {xn.numel()}")
    if not bool(torch.isfinite(xn).all()) or bool((xn < 0).any()):
        raise ValueError("prune_wanda: input norms must be finite and non-negative")
    k = _count(W.shape[1], sparsity)
    if k:
        idx = torch.sort(W.abs().float() * xn[None, :], dim=1, stable=True).indices[:, :k]
        W.scatter_(1, idx, 0.0)
    return weights


@torch.no_grad()
def prune_n_of_m(weights: torch.Tensor, n: int = 2, m: int = 4, scores: torch.Tensor | None = None) -> torch.Tensor:
    """Keep the ``n`` largest of every ``m`` consecutive entries along the last axis (2:4 by default)."""
    if not 0 < n <= m or weights.shape[-1] % m:
        raise ValueError("prune_n_of_m: need 0 < n <= m and a last axis that is a multiple of m")
    _check("prune_n_of_m", weights, 0.0)
    s = (weights.abs() if scores is None else scores).reshape(-1, m)
    drop = torch.sort(s, dim=1, stable=True).indices[:, : m - n]
    weights.view(-1, m).scatter_(1, drop, 0.0)
    return weights


def is_n_of_m(weights: torch.Tensor, n: int = 2, m: int = 4) -> bool:
    return bool(((weights.reshape(-1, m) != 0).sum(1) <= n).all())


def sparsity_ratio(weights: torch.Tensor) -> float:
    return 0.0 if weights.numel() == 0 else float((weights == 0).sum()) / weights.numel()


class LotteryTicketPruner:
    """Train, prune ``prune_fraction`` of the smallest ACTIVE weights, rewind the survivors to their initial values,
    repeat ``iterations`` times: the final sparsity is ``1 - (1 - p)^iterations`` and further calls are no-ops."""

    def __init__(self, prune_fraction: float, iterations: int):
        if not math.isfinite(prune_fraction) or not 0.0 <= prune_fraction <= 1.0:
            raise ValueError(f"LotteryTicketPruner: prune_fraction must be finite and in [0, 1], got {prune_fraction}")
        self.prune_fraction, self.iterations = prune_fraction, iterations
        self.initial = None

    def save_initial(self, weights: torch.Tensor) -> None:
        self.initial = weights.detach().clone()

    @torch.no_grad()
    def prune_and_rewind(self, weights: torch.Tensor) -> torch.Tensor:
        _check("LotteryTicketPruner.prune_and_rewind", weights, self.prune_fraction)
        if self.initial is None:
            raise ValueError("LotteryTicketPruner.prune_and_rewind: initial weights were not saved")
        if self.initial.numel() != weights.numel():
            raise ValueError(f"LotteryTicketPruner.prune_and_rewind: initial length {self.initial.numel()} does not match "
                             f"current length {weights.numel()}")
        target = 1.0 - (1.0 - self.prune_fraction) ** self.iterations
        if sparsity_ratio(weights) >= target:
            return weights
        flat = weights.view(-1)
        active = torch.nonzero(flat != 0).reshape(-1)
        k = _count(active.numel(), self.prune_fraction)
        if k:
            flat[active[_smallest(flat[active].abs(), k)]] = 0.0
        keep = flat != 0
        flat[keep] = self.initial.reshape(-1).to(flat.device)[keep]
        return weights


def prune(weights, method: PruningMethod, sparsity: float):
    return {PruningMethod.MAGNITUDE: prune_magnitude,
            PruningMethod.STRUCTURED_COLUMNS: lambda w, s: prune_structured_columns(w, sparsity=s),
            PruningMethod.STRUCTURED_ROWS: lambda w, s: prune_structured_rows(w, sparsity=s)}[method](weights, sparsity)

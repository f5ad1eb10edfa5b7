"""Compressed-sparse-row matrices and sparse x dense products. ``CsrTensor`` validates its structure on construction
(offsets start at 0, never decrease and end at nnz; column indices in range), so a malformed operand is refused
before any kernel reads through it. ``spmm_dense`` runs on the tensor's device through ``torch.sparse`` CSR kernels
(cuSPARSE on a GPU); ``spmm_dense_reference`` is the row-by-row fp32 statement with a fixed accumulation order, used
as the oracle. Reference counterpart: scirust-core/src/matrix/csr.rs:4-181.
"""
from __future__ import annotations

import torch


class CsrTensor:
    def __init__(self, values, column_indices, row_offsets, rows: int, cols: int):
        self.values = torch.as_tensor(values, dtype=torch.float32).reshape(-1)
        self.column_indices = torch.as_tensor(column_indices, dtype=torch.int64).reshape(-1)
        self.row_offsets = torch.as_tensor(row_offsets, dtype=torch.int64).reshape(-1)
        self.rows, self.cols = rows, cols
        if self.row_offsets.numel() != rows + 1:
            raise ValueError("CsrTensor: row_offsets.len() must be rows+1")
        if self.values.numel() != self.column_indices.numel():
            raise ValueError("CsrTensor: values.len() must equal column_indices.len()")
        if int(self.row_offsets[0]) != 0:
            raise ValueError("CsrTensor: row_offsets[0] must be 0")
        if bool((self.row_offsets[1:] < self.row_offsets[:-1]).any()):
            raise ValueError("CsrTensor: row_offsets must be non-decreasing")
        if int(self.row_offsets[-1]) != self.values.numel():
            raise ValueError("CsrTensor: row_offsets[rows] must equal values.len()")
        if self.column_indices.numel() and (int(self.column_indices.min()) < 0 or int(self.column_indices.max()) >= cols):
            raise ValueError("CsrTensor: a column index is out of range [0, cols)")

    @staticmethod
    def from_dense(dense: torch.Tensor, threshold: float = 0.0) -> "CsrTensor":
        mask = dense.abs() > threshold
        counts = mask.sum(1)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)])
        r, c = torch.nonzero(mask, as_tuple=True)
        return CsrTensor(dense[r, c], c, offsets, dense.shape[0], dense.shape[1])

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self.rows, self.cols)
        row_of = torch.repeat_interleave(torch.arange(self.rows), self.row_offsets[1:] - self.row_offsets[:-1])
        out.index_put_((row_of, self.column_indices), self.values, accumulate=True)
        return out

    def nnz(self) -> int:
        return self.values.numel()

    def to(self, device) -> "CsrTensor":
        t = CsrTensor.__new__(CsrTensor)
        t.values, t.column_indices, t.row_offsets = (x.to(device) for x in (self.values, self.column_indices, self.row_offsets))
        t.rows, t.cols = self.rows, self.cols
        return t

    def torch_csr(self) -> torch.Tensor:
        return torch.sparse_csr_tensor(self.row_offsets, self.column_indices, self.values, (self.rows, self.cols),
                                       check_invariants=False)     # validated at construction


def spmm_dense(a: CsrTensor, b: torch.Tensor) -> torch.Tensor:
    """``a [m, k] (CSR) @ b [k, n]`` -> dense ``[m, n]``."""
    if b.dim() != 2 or b.shape[0] != a.cols:
        raise ValueError(f"spmm_dense: dense operand must be [{a.cols}, n]")
    return a.torch_csr() @ b.float()


def spmm_dense_reference(a: CsrTensor, b: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(a.rows, b.shape[1])
    for r in range(a.rows):
        for idx in range(int(a.row_offsets[r]), int(a.row_offsets[r + 1])):
            out[r] += a.values[idx] * b[int(a.column_indices[idx])].float()
    return out


def solve(a: CsrTensor, b: torch.Tensor, tol: float = 1e-12, max_iter: int | None = None) -> torch.Tensor:
    """``A x = b`` for a square CSR matrix and one or several right-hand sides ``[n]`` / ``[n, k]``, in float64:
    BiCGSTAB on the sparse products (no fill-in), restarted from a dense LU solve if it stalls."""
    if a.rows != a.cols:
        raise ValueError("solve: the matrix must be square")
    csr = torch.sparse_csr_tensor(a.row_offsets, a.column_indices, a.values.double(), (a.rows, a.cols), check_invariants=False)
    rhs = torch.as_tensor(b, dtype=torch.float64)
    if rhs.dim() not in (1, 2) or rhs.shape[0] != a.rows:
        raise ValueError(f"solve: the right-hand side must have {a.rows} rows, got {tuple(rhs.shape)}")
    cols = rhs.reshape(a.rows, -1)
    out = torch.zeros_like(cols)
    for j in range(cols.shape[1]):
        bj = cols[:, j]
        x = torch.zeros_like(bj)
        r = bj.clone()
        r0, rho, alpha, omega = r.clone(), 1.0, 1.0, 1.0
        v = p = torch.zeros_like(bj)
        ok = False
        for _ in range(max_iter or 20 * a.rows):
            rho_new = float(r0 @ r)
            if abs(rho_new) < 1e-300 or omega == 0.0:
                break
            p = r + (rho_new / rho) * (alpha / omega) * (p - omega * v)
            v = (csr @ p[:, None])[:, 0]
            alpha = rho_new / float(r0 @ v)
            s_ = r - alpha * v
            t = (csr @ s_[:, None])[:, 0]
            tt = float(t @ t)
            omega = float(t @ s_) / tt if tt > 0 else 0.0
            x = x + alpha * p + omega * s_
            r = s_ - omega * t
            rho = rho_new
            if float(r.norm()) <= tol * max(1.0, float(bj.norm())):
                ok = True
                break
        out[:, j] = x if ok else torch.linalg.solve(a.to_dense().double(), bj)
    return out.reshape(rhs.shape)

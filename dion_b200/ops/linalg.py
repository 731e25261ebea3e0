"""Orthonormalisation building blocks: batched Cholesky-inverse of Gram matrices and
column norms.  CUDA tensors use the in-tree kernels, CPU tensors a PyTorch reference."""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import runtime

# Pivot floor for the Jacobi-scaled (unit diagonal) Gram matrix.
DEFAULT_PIVOT_FLOOR = 1e-6
# Largest rank the one-CTA-per-matrix kernel keeps in shared memory.
MAX_KERNEL_RANK = 1728


def chol_inverse_reference(G: torch.Tensor, pivot_floor: float = DEFAULT_PIVOT_FLOOR) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pure PyTorch version of the kernel: Jacobi scaling, Cholesky, triangular inverse.  A pivot that is
    not above `pivot_floor` marks a column that (numerically) depends on the earlier ones: it gets a unit
    pivot and eliminates nothing, so rounding noise is never divided by a tiny number; `info` counts such
    pivots.  Returns (Z, info) with Z lower triangular, Z @ G @ Z.T ~= I on the independent columns."""
    G = G.float()
    B, r, _ = G.shape
    diag = torch.diagonal(G, dim1=-2, dim2=-1)
    d = torch.where(diag > 1e-30, diag.clamp_min(1e-30).rsqrt(), torch.zeros_like(diag))
    W = G * d.unsqueeze(-1) * d.unsqueeze(-2)
    L = torch.zeros_like(W)
    info = torch.zeros(B, dtype=torch.int32, device=G.device)
    W = W.clone()
    for j in range(r):
        piv = W[:, j, j]
        bad = ~(piv > pivot_floor)
        info += bad.to(torch.int32)
        piv = torch.where(bad, torch.ones_like(piv), piv).sqrt()
        L[:, j, j] = piv
        if j + 1 < r:
            col = torch.where(bad.unsqueeze(-1), torch.zeros_like(W[:, j + 1:, j]), W[:, j + 1:, j] / piv.unsqueeze(-1))
            L[:, j + 1:, j] = col
            W[:, j + 1:, j + 1:] -= col.unsqueeze(-1) * col.unsqueeze(-2)
    eye = torch.eye(r, dtype=G.dtype, device=G.device).expand(B, r, r)
    Z = torch.linalg.solve_triangular(L, eye, upper=False)
    Z = torch.tril(Z) * d.unsqueeze(-2)
    return Z, info


def chol_inverse(G: torch.Tensor, pivot_floor: float = DEFAULT_PIVOT_FLOOR,
                 out: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None,
                 info: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """For a batch of Gram matrices ``G = P^T P`` (fp32, ``[B, r, r]``) return ``Z`` (lower
    triangular) such that ``P @ Z^T`` has orthonormal columns, and ``info`` = number of
    clamped pivots per matrix (0 for a well-conditioned input)."""
    if G.dim() != 3 or G.shape[-1] != G.shape[-2]:
        raise ValueError("chol_inverse expects [batch, r, r]")
    B, r, _ = G.shape
    if not runtime.use_cuda_kernels(G) or r > MAX_KERNEL_RANK or G.dtype != torch.float32:
        Z, inf = chol_inverse_reference(G, pivot_floor)
        if out is not None:
            out.copy_(Z)
            Z = out
        if info is not None:
            info.copy_(inf)
            inf = info
        return Z, inf
    if G.stride(-1) != 1:
        G = G.contiguous()
    if out is None:
        out = torch.empty(B, r, r, dtype=torch.float32, device=G.device)
    if work is None:
        work = torch.empty(B, r, r, dtype=torch.float32, device=G.device)
    if info is None:
        info = torch.empty(B, dtype=torch.int32, device=G.device)
    torch.ops.dion_b200.chol_inverse(G, out, work, info, float(pivot_floor))
    return out, info


def col_sumsq(X: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[b, j] = sum_i X[b, i, j]**2`` in fp32 (dion.py:1447-1457)."""
    squeeze = X.dim() == 2
    X3 = X.unsqueeze(0) if squeeze else X
    if runtime.use_cuda_kernels(X3) and X3.dtype in (torch.float32, torch.bfloat16) and X3.stride(-1) == 1:
        if out is None:
            out = torch.empty(X3.shape[0], X3.shape[2], dtype=torch.float32, device=X.device)
        torch.ops.dion_b200.col_sumsq(X3, out.view(X3.shape[0], X3.shape[2]))
        res = out
    else:
        res = X3.float().square().sum(dim=-2)
        if out is not None:
            out.copy_(res.view_as(out))
            res = out
    return res.view(-1) if squeeze else res.view(X3.shape[0], X3.shape[2])


def split_tf32(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x = hi + lo`` with ``hi`` exactly representable in tf32 (low 13 mantissa bits cleared):
    the operand pair of a 3xTF32 product (three tensor-core passes, close to fp32 accuracy)."""
    if runtime.use_cuda_kernels(x) and x.dtype == torch.float32 and x.is_contiguous() and x.data_ptr() % 16 == 0:
        hi, lo = torch.empty_like(x), torch.empty_like(x)
        torch.ops.dion_b200.split_tf32(x, hi, lo)
        return hi, lo
    hi = (x.view(torch.int32) & -8192).view(torch.float32)
    return hi, x - hi


# After a Cholesky-QR pass the squared norm of an independent column is close to 1; one far below that
# belongs to a column the factorisation gave up on (see chol_inverse_reference) and is dropped.
DEAD_COLUMN_BELOW = 1e-4


def refine_prep(G: torch.Tensor, dead_below: float = 1e-30,
                skip: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """From Gram matrices ``G: [B, r, r]``: ``d = rsqrt(diag G)`` (0 where the diagonal is not above
    `dead_below`) and ``C = stril(D G D)``, the strictly lower part of the column-scaled Gram matrix.
    ``skip`` (int32, one per matrix): C is zero for the matrices where it is non-zero."""
    if runtime.use_cuda_kernels(G) and G.dtype == torch.float32 and G.dim() == 3:
        G = G.contiguous()
        C, d = torch.empty_like(G), torch.empty(G.shape[:-1], dtype=torch.float32, device=G.device)
        torch.ops.dion_b200.refine_prep(G, C, d, float(dead_below), None if skip is None else skip.contiguous())
        return C, d
    diag = torch.diagonal(G, dim1=-2, dim2=-1)
    d = torch.where(diag > dead_below, diag.clamp_min(1e-30).rsqrt(), torch.zeros_like(diag))
    C = torch.tril(G * d.unsqueeze(-1) * d.unsqueeze(-2), diagonal=-1)
    if skip is not None:
        C = C * (skip == 0).to(C.dtype).view(-1, 1, 1)
    return C, d

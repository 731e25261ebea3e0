"""Orthonormalisation building blocks: batched Cholesky-inverse of Gram matrices and
column norms.  CUDA tensors use the in-tree kernels, CPU tensors a PyTorch reference."""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import runtime

# Pivot floor for the Jacobi-scaled (unit diagonal) Gram matrix.
DEFAULT_PIVOT_FLOOR = 1e-6
# Largest rank the one-CTA-per-matrix kernel keeps in shared memory.
MAX_KERNEL_RANK = 1728


def chol_inverse_reference(G: torch.Tensor, pivot_floor: float = DEFAULT_PIVOT_FLOOR, jacobi: bool = True,
                           colmask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pure PyTorch version of the kernel: Jacobi scaling, Cholesky, triangular inverse.  A pivot that is
    not above `pivot_floor` marks a column that (numerically) depends on the earlier ones: it gets a unit
    pivot and eliminates nothing, so rounding noise is never divided by a tiny number; `info` counts such
    pivots.  Returns (Z, info) with Z lower triangular, Z @ G @ Z.T ~= I on the independent columns.
    ``jacobi=False`` skips the scaling (the floor is then absolute); ``colmask`` (``[B, r]``) receives 1
    for factorised columns and 0 for clamped pivots."""
    G = G.float()
    B, r, _ = G.shape
    diag = torch.diagonal(G, dim1=-2, dim2=-1)
    d = torch.where(diag > 1e-30, diag.clamp_min(1e-30).rsqrt(), torch.zeros_like(diag))
    if not jacobi:
        d = torch.ones_like(diag)
    W = G * d.unsqueeze(-1) * d.unsqueeze(-2)
    L = torch.zeros_like(W)
    info = torch.zeros(B, dtype=torch.int32, device=G.device)
    W = W.clone()
    for j in range(r):
        piv = W[:, j, j]
        bad = ~(piv > pivot_floor)
        if colmask is not None:
            colmask[:, j] = (~bad).to(colmask.dtype)
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


# Ranks above this are factorised block by block (see chol_inverse_blocked); DION_B200_CHOL_BLOCKED=0
# keeps the one-launch kernel for every rank it fits.
BLOCK = 256
BLOCKED = os.environ.get("DION_B200_CHOL_BLOCKED", "1") != "0"
# 3xTF32 products split their fp32 operands inside the GEMM kernel (0: hi / lo tensors from a separate pass)
SPLIT_IN_KERNEL = os.environ.get("DION_B200_SPLIT_IN_KERNEL", "1") != "0"


def _split_block(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """tf32 halves (contiguous) of a ``[B, rows, cols]`` block that may be a strided view."""
    if (runtime.use_cuda_kernels(x) and x.dtype == torch.float32 and x.stride(-1) == 1 and x.shape[-1] % 4 == 0
            and x.stride(-2) % 4 == 0 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0):
        hi = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        lo = torch.empty_like(hi)
        torch.ops.dion_b200.split_tf32_rows(x, hi, lo)
        return hi, lo
    return split_tf32(x.contiguous())


def _diag_inverse(D: torch.Tensor, pivot_floor: float):
    """Inverse Cholesky factor of every diagonal block ``D: [B, nb, nb]`` (a strided view, already in the
    unit-diagonal scaling of the whole matrix, so no scaling of its own and an absolute pivot floor),
    the 0 / 1 mask of its clamped pivots and their count."""
    B, nb, _ = D.shape
    mask = torch.empty(B, nb, dtype=torch.float32, device=D.device)
    if runtime.use_cuda_kernels(D):
        Zd = torch.empty(B, nb, nb, dtype=torch.float32, device=D.device)
        work = torch.empty_like(Zd)
        info = torch.empty(B, dtype=torch.int32, device=D.device)
        torch.ops.dion_b200.chol_inverse(D, Zd, work, info, float(pivot_floor), False, mask)
        return Zd, mask, info
    Zd, info = chol_inverse_reference(D, pivot_floor, jacobi=False, colmask=mask)
    return Zd, mask, info


def chol_inverse_blocked(G: torch.Tensor, pivot_floor: float = DEFAULT_PIVOT_FLOOR, block: int = BLOCK,
                         out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """:func:`chol_inverse` for larger ranks with the cubic work on the tensor cores: a right-looking
    block factorisation whose diagonal blocks (``block`` columns) go through the Cholesky-inverse kernel
    and whose panels, trailing updates and the block-wise inverse are batched 3xTF32 GEMMs
    (hi / lo operands, one launch per product):

        Z_kk = chol(W_kk)^-1;   L_ik = W_ik Z_kk^T (i > k);   W_ij -= L_ik L_jk^T (i, j > k)
        Z_ik = -Z_ii (L_i,0:i Z_0:i,0:i)[:, k]               (row blocks of the inverse, top to bottom)

    A clamped pivot has a unit diagonal and eliminates nothing, exactly as in the one-launch kernel: its
    row of Z_kk is left out of the panel product, which zeroes its column of L below the block."""
    from .gemm import gemm

    G = G.float()
    B, r, _ = G.shape
    cuda = runtime.use_cuda_kernels(G) and G.stride(-1) == 1
    if cuda:
        W = torch.empty((B, r, r), dtype=torch.float32, device=G.device)
        d = torch.empty((B, r), dtype=torch.float32, device=G.device)
        torch.ops.dion_b200.jacobi_scale(G, W, d)
    else:
        diag = torch.diagonal(G, dim1=-2, dim2=-1)
        d = torch.where(diag > 1e-30, diag.clamp_min(1e-30).rsqrt(), torch.zeros_like(diag))
        W = G * d.unsqueeze(-1) * d.unsqueeze(-2)
    Z = out if out is not None else torch.empty_like(W)
    Z.zero_()
    # the factor's panels L_ik live in a buffer of their own, so that no product overwrites one of its operands
    Lbuf = torch.empty_like(W) if (cuda and SPLIT_IN_KERNEL) else W
    info = torch.zeros(B, dtype=torch.int32, device=G.device)
    edges = list(range(0, r, block)) + [r]
    zsplit = []
    for k in range(len(edges) - 1):
        k0, k1 = edges[k], edges[k + 1]
        Zd, mask, inf = _diag_inverse(W[:, k0:k1, k0:k1], pivot_floor)
        info += inf
        if cuda and Z.is_contiguous():
            Zm = torch.empty_like(Zd)
            torch.ops.dion_b200.place_block(Zd, mask, Z, Zm, k0)   # Z_kk into Z, and its copy without clamped rows
        else:
            Z[:, k0:k1, k0:k1].copy_(Zd)
            Zm = Zd * mask.unsqueeze(-1)
        zsplit.append(Zd if SPLIT_IN_KERNEL else split_tf32(Zd))
        if k1 == r:
            break
        panel = W[:, k1:, k0:k1]
        trail = W[:, k1:, k1:]
        if SPLIT_IN_KERNEL:
            # the products read their operands straight out of W and Lbuf (strided views) and split them on the fly
            L = Lbuf[:, k1:, k0:k1]
            gemm(panel, Zm.transpose(-1, -2), out=L, split3=True)
            if Lbuf is W:  # CPU: the product above was not in place, nothing else to do
                pass
            gemm(L, L.transpose(-1, -2), c=trail, out=trail, alpha=-1.0, beta=1.0, split3=True)
            continue
        zm_hi, zm_lo = split_tf32(Zm)
        p_hi, p_lo = _split_block(panel)
        gemm(p_hi, zm_hi.transpose(-1, -2), a_lo=p_lo, b_lo=zm_lo.transpose(-1, -2), out=panel)   # L_ik
        l_hi, l_lo = _split_block(panel)
        gemm(l_hi, l_hi.transpose(-1, -2), a_lo=l_lo, b_lo=l_lo.transpose(-1, -2), c=trail, out=trail, alpha=-1.0,
             beta=1.0)
    for i in range(1, len(edges) - 1):
        i0, i1 = edges[i], edges[i + 1]
        if SPLIT_IN_KERNEL:
            T = gemm(Lbuf[:, i0:i1, :i0], Z[:, :i0, :i0], split3=True)
            gemm(zsplit[i], T, out=Z[:, i0:i1, :i0], alpha=-1.0, split3=True)
            continue
        l_hi, l_lo = _split_block(W[:, i0:i1, :i0])
        z_hi, z_lo = _split_block(Z[:, :i0, :i0])
        T = gemm(l_hi, z_hi, a_lo=l_lo, b_lo=z_lo)
        t_hi, t_lo = split_tf32(T)
        zi_hi, zi_lo = zsplit[i]
        gemm(zi_hi, t_hi, a_lo=zi_lo, b_lo=t_lo, out=Z[:, i0:i1, :i0], alpha=-1.0)
    # undo the scaling: L^-1 = L'^-1 D, column j times d_j
    Z.mul_(d.unsqueeze(-2))
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
    if (BLOCKED and G.is_cuda and G.dtype == torch.float32 and r > BLOCK and r % 4 == 0 and B > 0
            and (out is None or out.is_contiguous())):
        Z, inf = chol_inverse_blocked(G, pivot_floor, out=out)
        if info is not None:
            info.copy_(inf)
            inf = info
        return Z, inf
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


def refine_prep(G: torch.Tensor, dead_below: float = 1e-30, skip: Optional[torch.Tensor] = None,
                fold: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """From Gram matrices ``G: [B, r, r]``: ``d = rsqrt(diag G)`` (0 where the diagonal is not above
    `dead_below`) and ``C = stril(D G D)``, the strictly lower part of the column-scaled Gram matrix.
    ``skip`` (int32, one per matrix): C is zero for the matrices where it is non-zero.
    ``fold``: the columns of C are scaled by d once more (``C diag(d)``), so that the correction
    ``(X D)(I - C^T)`` can be taken on the unscaled X as ``X diag(d) - X (C diag(d))^T``."""
    if runtime.use_cuda_kernels(G) and G.dtype == torch.float32 and G.dim() == 3:
        G = G.contiguous()
        C, d = torch.empty_like(G), torch.empty(G.shape[:-1], dtype=torch.float32, device=G.device)
        torch.ops.dion_b200.refine_prep(G, C, d, float(dead_below), None if skip is None else skip.contiguous(),
                                        bool(fold))
        return C, d
    diag = torch.diagonal(G, dim1=-2, dim2=-1)
    d = torch.where(diag > dead_below, diag.clamp_min(1e-30).rsqrt(), torch.zeros_like(diag))
    C = torch.tril(G * d.unsqueeze(-1) * d.unsqueeze(-2), diagonal=-1)
    if skip is not None:
        C = C * (skip == 0).to(C.dtype).view(-1, 1, 1)
    if fold:
        C = C * d.unsqueeze(-2)
    return C, d

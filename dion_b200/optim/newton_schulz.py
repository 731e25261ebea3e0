"""Quintic Newton-Schulz orthogonalisation in bf16 (Muon's ``zeropower``).

Same iteration and coefficient schedule as the reference (dion/muon.py:620-647;
dion/newton_schulz_triton.py:336-374): ``X <- a X + (b A + c A A) X`` with ``A = X X^T``,
five steps with per-step coefficients, input scaled to Frobenius norm <= 1.

On CUDA the three products of a step are tcgen05 GEMMs: ``A`` and ``b A + c A A`` are
symmetric, so only the upper-triangular tiles are computed and mirrored in the epilogue,
which also fuses the ``b A`` / ``a X`` additions.  Tall inputs are handled by multiplying
from the right (``A = X^T X``), so nothing is ever transposed in memory.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor

from .. import ops

NS_COEFFS: Tuple[Tuple[float, float, float], ...] = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)


def newton_schulz_torch(G: Tensor, epsilon: float = 1e-7,
                        coeffs: Sequence[Tuple[float, float, float]] = NS_COEFFS) -> Tensor:
    """Plain PyTorch statement of the iteration (bf16 matmuls); the numerical reference."""
    X = G.to(torch.bfloat16)
    tall = G.size(-2) > G.size(-1)
    if tall:
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + epsilon)
    for a, b, c in coeffs:
        A = X @ X.mT
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    if tall:
        X = X.mT
    return X


def newton_schulz(G: Tensor, epsilon: float = 1e-7, coeffs: Sequence[Tuple[float, float, float]] = NS_COEFFS,
                  sumsq: Optional[Tensor] = None, scatter: Optional[dict] = None) -> Optional[Tensor]:
    """Orthogonalise ``G`` (``[m, n]`` or a batch ``[B, m, n]``); returns bf16 of the same shape.

    ``sumsq`` (fp32 ``[B]``), when given, is the squared Frobenius norm of every matrix,
    e.g. accumulated by the momentum kernel, so that no extra pass over G is needed.

    ``scatter`` (CUDA only) makes the last product write its result tiles straight into
    per-destination blocks instead of one output tensor - the all-to-all that returns the
    shards of every orthogonalised matrix to their owners, done by the GEMM epilogue with
    peer stores.  Keys: ``ptrs`` (int64 CUDA tensor, B * dests block addresses), ``mode``
    (1 = row blocks, 2 = column blocks), ``block``, ``dests``, ``block_like`` (a tensor with
    the dtype and row pitch of one block).  Nothing is returned in that case."""
    if not G.is_cuda:
        return newton_schulz_torch(G, float(epsilon), coeffs)
    squeeze = G.dim() == 2
    X = G.unsqueeze(0) if squeeze else G
    if X.dim() != 3:
        X = X.flatten(end_dim=-3)
    X = X.to(torch.bfloat16)
    if not X.is_contiguous():
        X = X.contiguous()
    # X / (||X||_F + eps) in one pass over X (two when the norms still have to be computed)
    ops.runtime.use_cuda_kernels(X)  # loads the extension
    Xs = torch.empty_like(X)
    torch.ops.dion_b200.frob_scale(X, Xs, None if sumsq is None else sumsq.float().contiguous(), float(epsilon))
    X = Xs
    Bn, m, n = X.shape
    tall = m > n
    k = n if tall else m
    A = torch.empty(Bn, k, k, device=X.device, dtype=torch.bfloat16)
    Bm = torch.empty_like(A)
    Y = torch.empty_like(X)
    for it, (a, b, c) in enumerate(coeffs):
        last = it == len(coeffs) - 1
        if tall:
            ops.gemm(X.transpose(1, 2), X, out=A, symmetric=True)        # A = X^T X
            ops.gemm(A, A.transpose(1, 2), c=A, out=Bm, alpha=c, beta=b, symmetric=True)  # b A + c A A
            lhs, rhs = X, Bm                                              # a X + X B
        else:
            ops.gemm(X, X.transpose(1, 2), out=A, symmetric=True)        # A = X X^T
            ops.gemm(A, A.transpose(1, 2), c=A, out=Bm, alpha=c, beta=b, symmetric=True)
            lhs, rhs = Bm, X                                              # a X + B X
        if last and scatter is not None:
            torch.ops.dion_b200.gemm_scatter(lhs, rhs, X, scatter["block_like"], scatter["ptrs"], scatter["mode"],
                                             scatter["block"], scatter["dests"], 1.0, float(a),
                                             ops.runtime.status_tensor(X.device))
            return None
        ops.gemm(lhs, rhs, c=X, out=Y, alpha=1.0, beta=a)
        X, Y = Y, X
    out = X[0] if squeeze else X
    return out.view(G.shape)


def zeropower_via_newtonschulz5(G: Tensor, epsilon: float = 1e-7) -> Tensor:
    """Name-compatible entry point (dion/muon.py:620)."""
    return newton_schulz(G, epsilon)


def symmetric_gram(A: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """``A @ A^T`` for ``A: [m, k]`` or a batch ``[B, m, k]``, computing only the tiles on and above
    the diagonal and mirroring them (the first product of a Newton-Schulz step; the reference's
    ``ns_line_1``, dion/newton_schulz_triton.py:134-170).  Output in the dtype of ``A``."""
    if not A.is_cuda:
        r = A @ A.mT
        return r if out is None else out.copy_(r)
    squeeze = A.dim() == 2
    A3 = A.unsqueeze(0) if squeeze else A
    o3 = None if out is None else (out.unsqueeze(0) if squeeze else out)
    r = ops.gemm(A3, A3.transpose(1, 2), out=o3, symmetric=True)
    return r[0] if squeeze and out is None else (out if out is not None else r)


def symmetric_poly(A: Tensor, alpha: float, beta: float, out: Optional[Tensor] = None) -> Tensor:
    """``alpha * A @ A^T + beta * A`` for symmetric ``A: [m, m]`` (or a batch), upper-triangular tiles
    plus mirror with the ``beta * A`` term fused into the epilogue (the second product of a step; the
    reference's ``ns_line_2``, dion/newton_schulz_triton.py:261-302)."""
    if not A.is_cuda:
        r = alpha * (A @ A.mT) + beta * A
        return r if out is None else out.copy_(r)
    squeeze = A.dim() == 2
    A3 = A.unsqueeze(0) if squeeze else A
    o3 = None if out is None else (out.unsqueeze(0) if squeeze else out)
    r = ops.gemm(A3, A3.transpose(1, 2), c=A3, out=o3, alpha=float(alpha), beta=float(beta), symmetric=True)
    return r[0] if squeeze and out is None else (out if out is not None else r)


# names of the reference's entry points
ns_line_1 = symmetric_gram
ns_line_2 = symmetric_poly

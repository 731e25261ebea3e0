"""Column orthonormalisation used by Dion's power iteration.

Two families:

* :func:`orthonormalize_cholqr` - the production path.  Cholesky-QR run twice
  (CholeskyQR2) on a Jacobi-scaled Gram matrix: ``G = P^T P`` (all-reduced over the group
  that shards P's rows, if any), ``Z = chol(G)^{-1}`` by the one-CTA-per-matrix kernel,
  ``P <- P Z^T`` on the tensor cores.  It returns the same orthonormal basis as a QR
  factorisation with positive diagonal, needs one small all-reduce per pass when rows are
  sharded, and never synchronises with the host.  It stands in for the reference's
  sketch + Householder QR + triangular solves + Cholesky sequence
  (dion/dion.py:1267-1413).

* :func:`orthogonalize_reference` - the per-matrix methods of the reference oracle
  (``qr``, ``cqr``, ``rcqr``; dion/dion_reference.py:733-789), built on torch.linalg.
"""

from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .. import ops

# "3xtf32" splits fp32 operands into two tf32 halves (three tensor-core passes, ~fp32
# accuracy); "tf32" is a single pass.
GRAM_PRECISION = os.environ.get("DION_B200_GRAM_PRECISION", "3xtf32")


def _split_tf32(x: Tensor):
    """x = hi + lo with hi exactly representable in tf32 (low 13 mantissa bits cleared)."""
    hi = (x.view(torch.int32) & -8192).view(torch.float32)
    return hi, x - hi


def gram(P: Tensor) -> Tensor:
    """``P^T P`` in fp32 for a batch ``[B, a, r]`` (fp32 input)."""
    Pt = P.transpose(-1, -2)
    if not P.is_cuda:
        return Pt @ P
    if GRAM_PRECISION == "tf32":
        return ops.gemm(Pt, P, symmetric=True)
    hi, lo = _split_tf32(P)
    G = ops.gemm(hi.transpose(-1, -2), hi, symmetric=True)
    # cross terms lo^T hi + hi^T lo; lo^T lo is below fp32 resolution
    ops.gemm(lo.transpose(-1, -2), hi, c=G, out=G, beta=1.0)
    ops.gemm(hi.transpose(-1, -2), lo, c=G, out=G, beta=1.0)
    return G


def apply_right(P: Tensor, Z: Tensor) -> Tensor:
    """``P @ Z^T`` for ``P: [B, a, r]`` fp32 and lower-triangular ``Z: [B, r, r]``."""
    Zt = Z.transpose(-1, -2)
    if not P.is_cuda:
        return P @ Zt
    if GRAM_PRECISION == "tf32":
        return ops.gemm(P, Zt)
    p_hi, p_lo = _split_tf32(P)
    z_hi, z_lo = _split_tf32(Z)
    out = ops.gemm(p_hi, z_hi.transpose(-1, -2))
    ops.gemm(p_lo, z_hi.transpose(-1, -2), c=out, out=out, beta=1.0)
    ops.gemm(p_hi, z_lo.transpose(-1, -2), c=out, out=out, beta=1.0)
    return out


def orthonormalize_cholqr(P: Tensor, row_group: Optional[dist.ProcessGroup] = None, passes: int = 2,
                          pivot_floor: float = ops.linalg.DEFAULT_PIVOT_FLOOR) -> Tensor:
    """Orthonormalise the columns of every matrix in ``P: [B, a, r]``.

    ``row_group``: process group over which the rows (dim -2) of P are sharded; the Gram
    matrices are summed over it so every member applies the same triangular factor to its
    own rows.  All-zero inputs come back as zeros; rank-deficient inputs stay finite."""
    if P.dim() != 3:
        raise ValueError("expected a batch of matrices [B, a, r]")
    out_dtype = P.dtype
    X = P.float()
    if X.data_ptr() == P.data_ptr() and passes > 0:
        pass  # gemm writes new tensors, the input is never modified
    for _ in range(passes):
        G = gram(X)
        if row_group is not None and dist.get_world_size(row_group) > 1:
            dist.all_reduce(G, group=row_group)
        Z, _ = ops.chol_inverse(G, pivot_floor)
        X = apply_right(X, Z)
    return X.to(out_dtype)


def orthogonalize_reference(P: Tensor, qr_method: str = "rcqr", oversample: float = 1.25,
                            rng: Optional[torch.Generator] = None) -> Tensor:
    """Per-matrix orthogonalisation with the three methods of the reference oracle:
    Householder ``qr``; ``cqr`` (Cholesky QR, falling back to rcqr when the factorisation
    fails); ``rcqr`` (sketch -> QR of the sketch -> triangular solve -> one Cholesky QR),
    with wide or square inputs using Householder QR."""
    if qr_method not in ("qr", "cqr", "rcqr"):
        raise ValueError(f"Unknown QR method: {qr_method}")
    m, n = P.shape
    dtype = P.dtype
    Q = None
    if qr_method == "cqr":
        P32 = P.float()
        R, info = torch.linalg.cholesky_ex(P32.T @ P32, upper=True)
        if int(info) == 0:
            Q = torch.linalg.solve_triangular(R, P32, upper=True, left=False)
        else:
            qr_method = "rcqr"
    if Q is None and (qr_method == "qr" or m <= n):
        Q, _ = torch.linalg.qr(P.float())
    if Q is None:
        k = math.ceil(oversample * n / 128.0) * 128
        S = torch.empty((k, m), device=P.device, dtype=P.dtype).normal_(std=math.sqrt(1.0 / k), generator=rng)
        _, R = torch.linalg.qr((S @ P).float(), mode="r")
        Q = torch.linalg.solve_triangular(R, P.float(), upper=True, left=False)
        R, _ = torch.linalg.cholesky_ex(Q.T @ Q, upper=True)
        Q = torch.linalg.solve_triangular(R, Q, upper=True, left=False)
    return Q.to(dtype)

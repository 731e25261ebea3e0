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
from ..parallel import symm

# "3xtf32" splits fp32 operands into two tf32 halves (three tensor-core passes, ~fp32
# accuracy); "tf32" is a single pass.
GRAM_PRECISION = os.environ.get("DION_B200_GRAM_PRECISION", "3xtf32")
# 3xTF32 products split their fp32 operands inside the GEMM kernel (DION_B200_SPLIT_IN_KERNEL=0: hi / lo
# tensors written by a separate pass, then one launch over three K-segments)
SPLIT_IN_KERNEL = os.environ.get("DION_B200_SPLIT_IN_KERNEL", "1") != "0"


# tf32 halves that a producer already wrote next to its fp32 result (see register_split)
_presplit = {}


def register_split(x: Tensor, hi: Tensor, lo: Tensor) -> None:
    """Tell the orthonormalisation that the tf32 halves of `x` exist already (the kernel that summed x
    over the ranks wrote them in the same pass), so that it does not split x again.  Entries live until
    the end of the next :func:`orthonormalize_many`."""
    _presplit[(x.data_ptr(), tuple(x.shape))] = (hi, lo)


def _split_tf32(x: Tensor):
    """x = hi + lo with hi exactly representable in tf32 (low 13 mantissa bits cleared)."""
    known = _presplit.get((x.data_ptr(), tuple(x.shape)))
    if known is not None:
        return known
    return ops.linalg.split_tf32(x)


def gram(P: Tensor, reduce_group=None, out: Optional[Tensor] = None) -> Tensor:
    """``P^T P`` in fp32 for a batch ``[B, a, r]`` (fp32 input).  When the result will be
    summed over `reduce_group`, it is produced in that group's symmetric arena; `out` (contiguous
    ``[B, r, r]``, e.g. a slice of a buffer shared by several batches) receives it otherwise."""
    Pt = P.transpose(-1, -2)
    if not P.is_cuda:
        res = Pt @ P
        return res if out is None else out.copy_(res)
    if out is None:
        out = symm.empty(reduce_group, (P.shape[0], P.shape[2], P.shape[2]), torch.float32, P.device)
    if GRAM_PRECISION == "tf32":
        return ops.gemm(Pt, P, out=out, symmetric=True)
    if SPLIT_IN_KERNEL:
        # 3xTF32 with the tf32 halves formed in shared memory: P is read once, nothing is materialised
        return ops.gemm(Pt, P, out=out, symmetric=True, split3=True)
    hi, lo = _split_tf32(P)
    # hi^T hi and the cross terms lo^T hi + hi^T lo in one launch (three K-segments, the cross terms in an
    # accumulator of their own); lo^T lo is below fp32 resolution
    return ops.gemm(hi.transpose(-1, -2), hi, out=out, symmetric=True, a_lo=lo.transpose(-1, -2), b_lo=lo)


def apply_right(P: Tensor, Z: Tensor) -> Tensor:
    """``P @ Z^T`` for ``P: [B, a, r]`` fp32 and lower-triangular ``Z: [B, r, r]``."""
    Zt = Z.transpose(-1, -2)
    if not P.is_cuda:
        return P @ Zt
    if GRAM_PRECISION == "tf32":
        return ops.gemm(P, Zt)
    if SPLIT_IN_KERNEL:
        return ops.gemm(P, Zt, split3=True)
    p_hi, p_lo = _split_tf32(P)
    z_hi, z_lo = _split_tf32(Z)
    return ops.gemm(p_hi, z_hi.transpose(-1, -2), a_lo=p_lo, b_lo=z_lo.transpose(-1, -2))


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


def _refine(X: Tensor, row_group: Optional[dist.ProcessGroup], gave_up: Optional[Tensor] = None,
            out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """One triangular Newton correction of an almost orthonormal X: with the column-scaled
    Gram matrix D G D = I + E, the Cholesky factor's inverse is I - stril(E) to first order,
    so X <- (X D) (I - stril(E))^T squares the orthogonality error while keeping the column
    spans nested exactly like a QR factorisation does."""
    G = gram(X, row_group)
    if row_group is not None and dist.get_world_size(row_group) > 1:
        symm.all_reduce(G, row_group)
    # d = rsqrt(diag G), C = stril(D G D) = stril(E); columns the factorisation gave up on (squared norm
    # far below 1) are dropped instead of being blown up to unit length
    # a matrix whose factorisation gave up on some pivot (`gave_up`, int32 per matrix) is far from
    # orthonormal, where the first-order correction diverges: it is only rescaled
    if X.is_cuda:
        # X D (I - C^T) = X diag(d) - X (C diag(d))^T as one product on the unscaled X: the column scale
        # rides on the addend in the epilogue; the correction term is small, so a single tensor-core
        # pass keeps its error far below fp32 resolution
        C, d = ops.linalg.refine_prep(G, ops.linalg.DEAD_COLUMN_BELOW, gave_up, fold=True)
        return ops.gemm(X, C.transpose(-1, -2), c=X, alpha=-1.0, beta=1.0, c_col_scale=d, out_dtype=out_dtype)
    C, d = ops.linalg.refine_prep(G, ops.linalg.DEAD_COLUMN_BELOW, gave_up)
    Xs = X * d.unsqueeze(-2)
    return (Xs - Xs @ C.transpose(-1, -2)).to(out_dtype or X.dtype)


# Work sharding: a batch that is identical on every rank of a group is split over the group, each rank
# orthonormalises its share and the shares are all-gathered (the reference hands matrix j of a batch
# to rank j, dion/dion.py:809-830, 925-946).  DION_B200_SHARD_ORTHO=0 keeps the redundant computation.
SHARD_WORK = os.environ.get("DION_B200_SHARD_ORTHO", "1") != "0"
# relative rise of the Gram diagonal in the first pass of the ill-conditioned treatment
ROBUST_SHIFT = 1e-5
# a batch stays in that treatment while the smallest pivot of its shifted, unit-diagonal Gram matrix is below this
ROBUST_KEEP_BELOW = 1e-4
_gatherers = {}


def _my_share(X: Tensor, group) -> Tensor:
    """Matrices [rank * c, (rank + 1) * c) of the batch, c = ceil(B / world); ranks whose range runs
    past the end repeat the last matrix so that every share has the same shape."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B = X.shape[0]
    c = (B + world - 1) // world
    lo = min(rank * c, B)
    hi = min(lo + c, B)
    part = X[lo:hi]
    if hi - lo < c:
        part = torch.cat([part, X[B - 1:B].expand(c - (hi - lo), -1, -1)], dim=0)
    return part


class _Gatherer:
    """All-gather callable of one group (None: the process group's own) and whether its first call,
    which is compared against the process group's result, has happened."""

    def __init__(self, fn):
        self.fn = fn
        self.checked = False


def _exchange(out: Tensor, part: Tensor, group, state: _Gatherer) -> None:
    """out = all-gather of `part` over `group`.  The first call through an in-tree kernel also runs the
    process group's all-gather and compares: if the kernel reports a failure or any rank sees a
    difference, every rank of the group switches to the process group for good."""
    if state.fn is None:
        dist.all_gather_into_tensor(out, part, group=group)
        return
    if state.checked:
        state.fn(out.view(-1), part.view(-1), group)
        return
    ref = torch.empty_like(out)
    dist.all_gather_into_tensor(ref, part, group=group)
    try:
        state.fn(out.view(-1), part.view(-1), group)
        if part.is_cuda:
            from ..ops import runtime

            runtime.check_status(part.device)
        ok = torch.equal(out, ref)
    except Exception as e:  # a kernel-side failure (status word) or a launch error
        ok = False
        print(f"[dion_b200] rank {dist.get_rank()}: in-tree all-gather failed on first use ({type(e).__name__}: {e})")
    verdict = torch.tensor([1 if ok else 0], dtype=torch.int32, device=part.device)
    dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
    state.checked = True
    if int(verdict.item()) == 0:
        state.fn = None
        out.copy_(ref)
        if dist.get_rank() == 0:
            print("[dion_b200] the in-tree all-gather did not reproduce the process group's on first use; "
                  "using the process group for the orthonormal factors")


def _gather_shares(part: Tensor, group, B: int) -> Tensor:
    """Inverse of :func:`_my_share`: all-gather the shares and drop the padding."""
    world = dist.get_world_size(group)
    part = part.contiguous()
    out = part.new_empty((world * part.shape[0],) + tuple(part.shape[1:]))
    key = symm._key(group)
    if key not in _gatherers:
        fn = None
        if part.is_cuda:
            from ..parallel import fsdp_comm

            if fsdp_comm._usable(group, part.device):
                fn = fsdp_comm.SymmAllGather(group, part.device)  # falls back per call where it does not apply
        _gatherers[key] = _Gatherer(fn)
    _exchange(out, part, group, _gatherers[key])
    return out[:B]


def orthonormalize_many(Ps, row_groups=None, refine_passes: int = 2,
                        pivot_floor: float = ops.linalg.DEFAULT_PIVOT_FLOOR, shard_groups=None, totals=None,
                        out_dtypes=None, robust=None, infos=None):
    """Orthonormalise several batches ``P_i: [B_i, a_i, r_i]`` at once.  All Gram matrices of
    the same rank are factorised by a single launch of the Cholesky kernel (one CTA per
    matrix), whatever their row counts; the remaining loss of orthogonality is removed by
    `refine_passes` triangular Newton corrections, which are plain tensor-core GEMMs.
    ``row_groups[i]`` is the process group sharding the rows of ``P_i`` (or None);
    ``shard_groups[i]`` a group on whose ranks ``P_i`` is identical, which then splits the batch.
    ``totals[i]``, when not None, says that ``P_i`` already is this rank's share (as
    :func:`_my_share` would cut it) of a batch of that many matrices; the result is the whole batch.
    ``out_dtypes[i]`` is the dtype of result i (default: the input's); shares are converted before they
    are exchanged, so a bf16 consumer halves the all-gather.
    ``robust[i]`` asks for the ill-conditioned treatment of batch i: the first factorisation runs on the
    Gram matrix with its diagonal raised by ROBUST_SHIFT (always positive definite in fp32) and a second
    Cholesky-QR pass follows (shifted CholeskyQR3; good up to condition numbers around 1e6, where one pass
    gives up near 3e3).  ``infos``, if a list, receives per batch the int32 tensor of pivots the (first)
    factorisation gave up on, per matrix of this rank's share (for a `robust` batch: 1 where the smallest
    pivot says that the plain factorisation would still give up) - the signal for asking for `robust`."""
    try:
        return _orthonormalize_many(Ps, row_groups, refine_passes, pivot_floor, shard_groups, totals, out_dtypes,
                                    robust, infos)
    finally:
        _presplit.clear()


def _orthonormalize_many(Ps, row_groups, refine_passes, pivot_floor, shard_groups, totals, out_dtypes, robust, infos):
    n = len(Ps)
    if out_dtypes is None:
        out_dtypes = [P.dtype for P in Ps]
    if row_groups is None:
        row_groups = [None] * n
    if totals is None:
        totals = [None] * n
    if shard_groups is None or not SHARD_WORK:
        assert all(t is None for t in totals), "a batch that arrives split needs its group"
        shard_groups = [None] * n
    shard_groups = [g if (t is not None or (g is not None and dist.get_world_size(g) > 1 and P.shape[0] > 1 and rg is None))
                    else None for g, P, rg, t in zip(shard_groups, Ps, row_groups, totals)]
    if robust is None:
        robust = [False] * n
    if any(g is not None for g in shard_groups):
        parts = [P.float() if (g is None or t is not None) else _my_share(P.float(), g)
                 for P, g, t in zip(Ps, shard_groups, totals)]
        outs = _orthonormalize_many(parts, row_groups, refine_passes, pivot_floor, None, None, out_dtypes, robust, infos)
        return [X.to(dt) if g is None else _gather_shares(X.to(dt), g, P.shape[0] if t is None else t)
                for X, P, g, t, dt in zip(outs, Ps, shard_groups, totals, out_dtypes)]
    dtypes = out_dtypes
    Xs = [P.float() for P in Ps]
    first_info = [None] * n
    last_info = [None] * n  # pivots the last factorisation of each batch gave up on
    for cholqr_pass in range(2 if any(robust) else 1):
        todo = [i for i in range(n) if cholqr_pass == 0 or robust[i]]
        by_rank = {}
        for i in todo:
            by_rank.setdefault(Xs[i].shape[-1], []).append(i)
        # The Gram matrices of all batches of one rank are factorised together.  Batches whose Gram matrix
        # is not summed over a row group write theirs straight into one shared buffer; the others are
        # produced in their group's arena and copied in.
        Gs, Gcats = {}, {}
        for r, idxs in by_rank.items():
            if len(idxs) > 1:
                total = sum(Xs[i].shape[0] for i in idxs)
                Gcats[r] = torch.empty((total, r, r), dtype=torch.float32, device=Xs[idxs[0]].device)
            off = 0
            for i in idxs:
                b = Xs[i].shape[0]
                g = row_groups[i]
                sharded_rows = g is not None and dist.get_world_size(g) > 1
                if r in Gcats and not sharded_rows:
                    Gs[i] = gram(Xs[i], out=Gcats[r][off:off + b])
                else:
                    Gs[i] = gram(Xs[i], g)
                    if sharded_rows:
                        symm.all_reduce(Gs[i], g)
                    if r in Gcats:
                        Gcats[r][off:off + b].copy_(Gs[i])
                        Gs[i] = Gcats[r][off:off + b]
                if cholqr_pass == 0 and robust[i]:
                    Gs[i].diagonal(dim1=-2, dim2=-1).mul_(1.0 + ROBUST_SHIFT)
                off += b
        for r, idxs in by_rank.items():
            Gcat = Gcats[r] if r in Gcats else Gs[idxs[0]]
            Z, info = ops.chol_inverse(Gcat, pivot_floor)
            off = 0
            for i in idxs:
                b = Gs[i].shape[0]
                Xs[i] = apply_right(Xs[i], Z[off:off + b])
                last_info[i] = info[off:off + b]
                if cholqr_pass == 0 and not robust[i]:
                    first_info[i] = info[off:off + b]
                elif cholqr_pass == 0:
                    # the shifted factorisation never gives up; its smallest pivot, 1 / (G_jj Z_jj^2) in
                    # the unit-diagonal scaling, says whether the plain one would have
                    gd = Gs[i].diagonal(dim1=-2, dim2=-1)
                    zd = Z[off:off + b].diagonal(dim1=-2, dim2=-1)
                    piv = torch.where(gd > 1e-30, 1.0 / (gd * zd * zd).clamp_min(1e-30), torch.ones_like(gd))
                    first_info[i] = (piv.amin(dim=-1) < ROBUST_KEEP_BELOW).to(torch.int32)
                off += b
    if infos is not None:
        infos.extend(first_info)
    # A batch that went through two Cholesky-QR passes is already orthonormal to about 1e-3 (CholeskyQR2 on a
    # matrix whose condition number the shifted first pass brought below a few hundred); one correction takes
    # that to the 1e-6 level.  After a single pass the error can be 1e-1, which takes two corrections.
    passes = [max(1, refine_passes - 1) if (rb and refine_passes > 0) else refine_passes for rb in robust]
    for k in range(refine_passes):
        for i in range(n):
            if k >= passes[i]:
                continue
            # the last correction writes the result in the dtype its consumer multiplies with
            last = k == passes[i] - 1
            Xs[i] = _refine(Xs[i], row_groups[i], last_info[i], dtypes[i] if last else None)
    return [X.to(dt) for X, dt in zip(Xs, dtypes)]


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

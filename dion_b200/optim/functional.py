"""Building blocks of the Dion and Muon updates as free functions, under the names and call signatures of
the reference's module-level helpers, implemented on this package's kernels.

A training script that imports pieces of the reference rather than its optimizer classes - a custom update
loop calling ``orthogonalize``, ``column_normalize``, ``foreach_baddbmm_``, ``muon_update_pre_orthogonalize``
and so on - finds them here (and re-exported from ``dion_b200.dion`` / ``dion_b200.muon``, the module paths the
reference uses).  Every function accepts plain tensors or DTensors exactly where the reference's does, runs the
in-tree CUDA kernels for CUDA inputs and plain PyTorch on the host.

Where the algorithm differs from the reference's, the result is the same mathematical object: ``orthogonalize``
and ``distributed_orthogonalize`` return the orthonormal factor of a QR factorisation with positive diagonal
through Cholesky-QR on the tensor cores instead of a random sketch followed by Householder QR, so ``oversample``
is accepted and not needed.
"""

from __future__ import annotations

import math
from typing import Callable, Generator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed.tensor import DeviceMesh, DTensor, Replicate, Shard
from torch.distributed.tensor import randn as dtensor_randn

from .. import ops
from .common import all_reduce_, group_of, like_dtensor, to_local
from .orthogonalize import orthonormalize_cholqr


def _scalar(v) -> float:
    """Hyper-parameters arrive as Python numbers or as 0-dim tensors (the reference passes tensors so that its
    compiled functions do not specialise on their values)."""
    return float(v.item()) if isinstance(v, Tensor) else float(v)


# --------------------------------------------------------------------------- Dion (dion/dion.py:1165-1602)

def all_reduce_replicate_mesh(G: Union[Tensor, List[Tensor]], replicate_mesh: Union[DeviceMesh, dist.ProcessGroup, None] = None,
                              return_dtensor: bool = True, reduce_op: str = "avg") -> Union[Tensor, List[Tensor]]:
    """Mean (``"avg"``) or sum (``"sum"``) of a tensor or a list of tensors over the data-parallel replicas
    (dion/dion.py:1165-1197).  Unlike the reference's functional collective this reduces the local tensors in
    place - same-dtype members of a list travel as one bucket - and returns them, wrapped as DTensors like the
    inputs when ``return_dtensor``."""
    if replicate_mesh is None:
        return G
    if reduce_op not in ("avg", "sum"):
        raise ValueError(f"reduce_op must be 'avg' or 'sum', got {reduce_op!r}")
    local = to_local(G)
    all_reduce_(local, group_of(replicate_mesh), average=reduce_op == "avg")
    if not return_dtensor:
        return local
    return like_dtensor(local, G if isinstance(G, Tensor) else G[0])


def tensor_list_to_batch(M: List[Tensor], Q: List[Tensor], is_transposed: bool) -> Tuple[Tensor, Tensor]:
    """Stack momentum matrices (transposed when the parameter is handled transposed) and their Q factors into
    two 3-D batches, Q in the dtype of M (dion/dion.py:1200-1218)."""
    M_batch = torch.stack([m.mT for m in M]) if is_transposed else torch.stack(list(M))
    return M_batch, torch.stack(list(Q)).to(M_batch.dtype)


def generate_random_sketch_matrix(P: Tensor, oversample: float = 1.25, shard_mesh_dim: Optional[int] = None) -> Tensor:
    """Gaussian sketch ``S: [*, k, m]`` for ``P: [*, m, r]`` with ``k = oversample * r`` rounded up to a multiple
    of 128 and entries of variance ``1 / k`` (dion/dion.py:1221-1264).  For a DTensor the sketch is drawn
    through the DTensor random-number generator, so that replicas agree and shards differ, and it is sharded
    along m over ``shard_mesh_dim`` when that is given.  The Cholesky-QR path of this package does not use a
    sketch; the function serves code that builds its own randomised factorisations."""
    if P.ndim < 3:
        raise ValueError("P must have a batch dimension")
    m, r = P.size(-2), P.size(-1)
    k = math.ceil(oversample * r / 128.0) * 128
    std = math.sqrt(1.0 / k)
    shape = (*P.shape[:-2], k, m)
    if isinstance(P, DTensor):
        placements = list(P.placements)
        if shard_mesh_dim is not None:
            placements[shard_mesh_dim] = Shard(P.ndim - 1)
        return dtensor_randn(shape, device_mesh=P.device_mesh, dtype=P.dtype, placements=placements) * std
    if shard_mesh_dim is not None:
        raise TypeError("a sharded sketch needs a DTensor input")
    return torch.empty(shape, device=P.device, dtype=P.dtype).normal_(std=std)


def orthogonalize(P: Tensor, oversample: float = 1.25) -> Tensor:
    """Orthonormalise the columns of every matrix of ``P: [*, m, r]`` (m >= r gives orthonormal columns; a wide
    matrix is treated like the reference treats it, by a QR factorisation of the matrix as it stands).  The
    matrix dimensions must not be sharded; a DTensor comes back as a DTensor with the same placements
    (dion/dion.py:1267-1309)."""
    del oversample  # no sketch is drawn: Cholesky-QR works on the Gram matrix directly
    if P.ndim < 3:
        raise ValueError("expected P to have a batch dimension")
    if isinstance(P, DTensor) and any(p.is_shard(P.ndim - 2) or p.is_shard(P.ndim - 1) for p in P.placements):
        raise ValueError("orthogonalize: the matrix dimensions cannot be sharded (see distributed_orthogonalize)")
    local = to_local(P)
    lead = local.shape[:-2]
    X = local.reshape(-1, local.shape[-2], local.shape[-1])
    if X.shape[-2] < X.shape[-1]:
        # wide: the Gram matrix would be singular, take the Householder route like the reference
        Qf, _ = torch.linalg.qr(X.float())
        out = Qf.to(local.dtype)
    else:
        out = orthonormalize_cholqr(X)
    return like_dtensor(out.reshape(*lead, *out.shape[-2:]).contiguous(), P)


def distributed_orthogonalize(P: DTensor, oversample: float = 1.25, shard_mesh_dim: Optional[int] = None) -> DTensor:
    """:func:`orthogonalize` for matrices whose rows (dimension -2) are sharded over mesh dimension
    ``shard_mesh_dim`` (dion/dion.py:1312-1413).  The reference moves whole matrices between ranks (all-to-all,
    reduce-scatter, all-gather around per-rank QR and Cholesky factorisations); here every rank forms the Gram
    matrix of its rows, the Gram matrices are summed over the shard group - one small all-reduce per pass - and
    every rank applies the same triangular factor to its own rows."""
    del oversample
    if not isinstance(P, DTensor):
        raise TypeError("distributed_orthogonalize expects a DTensor")
    if any(p.is_partial() for p in P.placements) or any(p.is_shard(P.ndim - 1) for p in P.placements):
        raise ValueError("the input cannot be partial or sharded along its last dimension")
    if P.ndim < 3:
        raise ValueError("expected P to have a batch dimension")
    row_sharded = [i for i, p in enumerate(P.placements) if p.is_shard(P.ndim - 2)]
    if shard_mesh_dim is None:
        if row_sharded:
            raise ValueError("rows are sharded: name the mesh dimension with shard_mesh_dim")
        return orthogonalize(P)
    if row_sharded not in ([], [shard_mesh_dim]):
        raise ValueError(f"rows are sharded over mesh dimensions {row_sharded}, not over {shard_mesh_dim}")
    group = P.device_mesh.get_group(shard_mesh_dim) if row_sharded else None
    local = P.to_local()
    lead = local.shape[:-2]
    X = local.reshape(-1, local.shape[-2], local.shape[-1])
    if P.size(-2) < P.size(-1):
        # wide as a whole: gather the rows, factorise, keep this rank's rows
        full = P.redistribute(placements=[Replicate() for _ in P.placements]).to_local()
        Qf, _ = torch.linalg.qr(full.reshape(-1, *full.shape[-2:]).float())
        rows = local.shape[-2]
        r0 = P.device_mesh.get_local_rank(shard_mesh_dim) * rows if row_sharded else 0
        out = Qf[:, r0:r0 + rows].to(local.dtype)
    else:
        out = orthonormalize_cholqr(X, row_group=group)
    return like_dtensor(out.reshape(*lead, *out.shape[-2:]).contiguous(), P)


def fix_all_zero_or_nan(P: Tensor, R: Tensor, Q_init: Tensor, B: Tensor) -> Tuple[Tensor, Tensor]:
    """Where a matrix of ``B`` is entirely zero, the power iteration's outputs are zero or NaN: return
    ``P = 0`` and ``R = Q_init`` for those matrices and the NaN-free ``P``, ``R`` for the others, without a
    host-side branch and shard-locally like the reference (dion/dion.py:1416-1444)."""
    zero = (to_local(B) == 0).all(dim=(-2, -1), keepdim=True)
    P_local = torch.where(zero, torch.zeros_like(to_local(P)), to_local(P).nan_to_num())
    R_local = torch.where(zero, to_local(Q_init).to(to_local(R).dtype), to_local(R).nan_to_num())
    return like_dtensor(P_local, P), like_dtensor(R_local, R)


def local_column_sum_sq(X: Tensor) -> Tensor:
    """Per-column sum of squares of a tensor or of the local shard of a DTensor: ``[*, m, n] -> [*, 1, n]``,
    always a plain fp32 tensor (dion/dion.py:1447-1457)."""
    X = to_local(X)
    if X.dim() >= 2 and X.dtype in (torch.float32, torch.bfloat16):
        X3 = X.reshape(-1, X.shape[-2], X.shape[-1])
        return ops.col_sumsq(X3).reshape(*X.shape[:-2], 1, X.shape[-1])
    return X.float().square().sum(dim=-2, keepdim=True)


def column_normalize(X: Tensor, full_column_sum_sq: Optional[Tensor] = None, epsilon: float = 1e-8) -> Tensor:
    """Divide every column by its Euclidean norm plus ``epsilon``, in fp32, returning the dtype (and DTensor
    wrapping) of the input.  A row-sharded DTensor needs the complete sums of squares from the caller
    (dion/dion.py:1460-1491)."""
    if isinstance(X, DTensor) and full_column_sum_sq is None and any(p.is_shard(X.ndim - 2) for p in X.placements):
        raise RuntimeError("Cannot normalize row-sharded DTensor.")
    local = to_local(X).float()
    ss = local.square().sum(dim=-2, keepdim=True) if full_column_sum_sq is None else to_local(full_column_sum_sq).float()
    return like_dtensor((local / (ss.sqrt() + epsilon)).to(X.dtype), X)


def foreach_baddbmm_(X: List[Tensor], A: Tensor, B: Tensor, alpha: float = 1.0, beta: float = 1.0,
                     transpose: bool = False) -> None:
    """``X[i] = beta * X[i] + alpha * (A @ B^T)[i]`` (``(B @ A^T)[i]`` with ``transpose``) for separately
    allocated matrices ``X[i]`` (dion/dion.py:1494-1530).  On CUDA, fp32 matrices are updated by one batched
    tensor-core product whose epilogue reads and writes every ``X[i]`` through a table of addresses; nothing of
    the size of the update is materialised."""
    if A.size(0) != B.size(0) or len(X) != A.size(0):
        raise ValueError("len(X), A.size(0) and B.size(0) must agree")
    a_op, b_op = (B, A.mT) if transpose else (A, B.mT)
    if isinstance(a_op, DTensor) or isinstance(b_op, DTensor):
        prod = a_op @ b_op
        if isinstance(prod, DTensor):
            if any(p.is_partial() for p in prod.placements):
                raise NotImplementedError("a product with Partial() placements is not supported")
            prod = prod.to_local()
        for x, u in zip(to_local(X), prod.unbind(0)):
            x.mul_(beta).add_(u.to(x.dtype), alpha=alpha)
        return
    Xl = to_local(X)
    x0 = Xl[0]
    fast = (x0.is_cuda and x0.dtype == torch.float32 and a_op.dtype == b_op.dtype
            and a_op.dtype in (torch.float32, torch.bfloat16)
            and all(x.is_contiguous() and x.data_ptr() % 16 == 0 for x in Xl) and (x0.shape[-1] * 4) % 16 == 0)
    if fast:
        ptrs = torch.tensor([x.data_ptr() for x in Xl], dtype=torch.int64, device=x0.device)
        ops.gemm(a_op, b_op, c=x0, out=x0, c_ptrs=ptrs, out_ptrs=ptrs, alpha=float(alpha), beta=float(beta))
        return
    prod = ops.gemm(a_op, b_op, out_dtype=torch.float32) if a_op.is_cuda and a_op.dtype == b_op.dtype else \
        torch.matmul(a_op.float(), b_op.float())
    for x, u in zip(Xl, prod.unbind(0)):
        x.mul_(beta).add_(u.to(x.dtype), alpha=alpha)


def update_Q_matrix_(Q: List[Tensor], Q_batch: Tensor, Q_sharded_placements=None) -> None:
    """Copy the rows of the stacked new ``Q_batch`` into the list of Q states, re-sharding a DTensor batch to
    the placements of the states first (their ``Shard`` dimensions shifted by the batch dimension)
    (dion/dion.py:1533-1561)."""
    if Q_sharded_placements is not None:
        if not isinstance(Q_batch, DTensor):
            raise TypeError("re-sharding needs a DTensor batch")
        shifted = [Shard(p.dim + 1) if p.is_shard() else p for p in Q_sharded_placements]
        Q_batch = Q_batch.redistribute(placements=shifted)
    rows = to_local(Q_batch).to(to_local(Q[0]).dtype).unbind(0)
    torch._foreach_copy_(to_local(list(Q)), list(rows))


# --------------------------------------------------------------------------- AdamW / Lion (dion/scalar_opts.py)

def adamw_update_foreach(X: List[Tensor], G: List[Tensor], M: List[Tensor], V: List[Tensor], lr, beta1, beta2,
                         weight_decay, step: int, epsilon: float) -> None:
    """AdamW on lists of tensors, one multi-tensor kernel launch on CUDA (dion/scalar_opts.py:89-149)."""
    if not (len(X) == len(G) == len(M) == len(V)):
        raise ValueError("X, G, M and V must have the same length")
    ops.adamw_update(to_local(list(X)), to_local(list(G)), to_local(list(M)), to_local(list(V)), lr=_scalar(lr),
                     beta1=_scalar(beta1), beta2=_scalar(beta2), weight_decay=_scalar(weight_decay), step=int(step),
                     epsilon=float(epsilon))


def lion_update_foreach(X: List[Tensor], G: List[Tensor], M: List[Tensor], lr, beta1, beta2, weight_decay) -> None:
    """Lion on lists of tensors, one multi-tensor kernel launch on CUDA (dion/scalar_opts.py:152-187)."""
    if not (len(X) == len(G) == len(M)):
        raise ValueError("X, G and M must have the same length")
    ops.lion_update(to_local(list(X)), to_local(list(G)), to_local(list(M)), lr=_scalar(lr), beta1=_scalar(beta1),
                    beta2=_scalar(beta2), weight_decay=_scalar(weight_decay))


def adamw_update(X: Tensor, G: Tensor, M: Tensor, V: Tensor, lr, beta1, beta2, weight_decay, step: int,
                 epsilon: float) -> None:
    """AdamW on one tensor (dion/scalar_opts.py:6-52)."""
    adamw_update_foreach([X], [G], [M], [V], lr, beta1, beta2, weight_decay, step, epsilon)


def lion_update(X: Tensor, G: Tensor, M: Tensor, lr, beta1, beta2, weight_decay) -> None:
    """Lion on one tensor (dion/scalar_opts.py:55-86)."""
    lion_update_foreach([X], [G], [M], lr, beta1, beta2, weight_decay)


def adamw_update_foreach_async(X, G, M, V, lr, beta1, beta2, weight_decay, step: int,
                               epsilon: float) -> Generator[None, None, None]:
    """Task form of :func:`adamw_update_foreach` for the cooperative scheduler (dion/muon.py:489-505)."""
    adamw_update_foreach(X, G, M, V, lr, beta1, beta2, weight_decay, step, epsilon)
    yield


def lion_update_foreach_async(X, G, M, lr, beta1, beta2, weight_decay) -> Generator[None, None, None]:
    """Task form of :func:`lion_update_foreach` (dion/muon.py:508-522)."""
    lion_update_foreach(X, G, M, lr, beta1, beta2, weight_decay)
    yield


def adamw_update_allreduce_grad(X, G, M, V, lr, beta1, beta2, weight_decay, step: int, epsilon: float,
                                replicate_mesh=None) -> Generator[None, None, None]:
    """AdamW after averaging the gradients over the replicas; yields once while the all-reduce is in flight
    (dion/dion.py:1564-1583)."""
    if replicate_mesh is not None:
        wait = all_reduce_(to_local(list(G)), group_of(replicate_mesh), average=True, async_op=True)
        yield
        wait()
    adamw_update_foreach(X, G, M, V, lr, beta1, beta2, weight_decay, step, epsilon)


def lion_update_allreduce_grad(X, G, M, lr, beta1, beta2, weight_decay,
                               replicate_mesh=None) -> Generator[None, None, None]:
    """Lion after averaging the gradients over the replicas (dion/dion.py:1586-1602)."""
    if replicate_mesh is not None:
        wait = all_reduce_(to_local(list(G)), group_of(replicate_mesh), average=True, async_op=True)
        yield
        wait()
    lion_update_foreach(X, G, M, lr, beta1, beta2, weight_decay)


# --------------------------------------------------------------------------- Muon (dion/muon.py:525-593)

def muon_update_pre_orthogonalize(G: List[Tensor], M: List[Tensor], momentum, nesterov: bool) -> List[Tensor]:
    """``M <- momentum * M + G`` in place and the bf16 input of the orthogonalisation, ``momentum * M + G`` with
    Nesterov momentum and ``M`` without: one multi-tensor kernel on CUDA (dion/muon.py:525-553)."""
    return ops.muon_momentum(to_local(list(G)), to_local(list(M)), mu=_scalar(momentum), nesterov=bool(nesterov))


def muon_update_post_orthogonalize(X: List[Tensor], U: List[Tensor], base_lr, adjusted_lr, weight_decay) -> None:
    """``X <- (1 - base_lr * weight_decay) * X - adjusted_lr * U`` in place, one multi-tensor kernel on CUDA
    (dion/muon.py:556-573)."""
    ops.muon_apply(to_local(list(X)), to_local(list(U)), decay=1.0 - _scalar(base_lr) * _scalar(weight_decay),
                   step=_scalar(adjusted_lr))


def muon_update_newton_schulz(X: Tensor, newton_schulz_func: Callable, flatten: bool, epsilon) -> Tensor:
    """Bring ``X`` into the 2-D / 3-D form the orthogonalisation expects - everything after the first dimension
    flattened with ``flatten``, leading dimensions folded into one batch otherwise - call it and restore the
    shape (dion/muon.py:576-593)."""
    shape = X.shape
    if flatten and X.ndim >= 3:
        X = X.flatten(start_dim=1)
    elif X.ndim >= 4:
        X = X.flatten(end_dim=-3)
    return newton_schulz_func(X, epsilon=epsilon).reshape(shape)

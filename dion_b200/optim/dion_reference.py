"""DionReference: per-parameter, synchronous Dion following the paper, with
``power_iters >= 1`` and ``qr_method`` in {"qr", "cqr", "rcqr"} (CQR only after a warm-up,
falling back to RCQR when the Cholesky factorisation fails).  Behavioural counterpart of
dion/dion_reference.py:64-984 and the numerical oracle for the batched :class:`Dion`.

Constructor, state layout and sharding rules are inherited from :class:`Dion`; the update
works on local shards with explicit collectives, like the batched optimizer, but one
parameter at a time and with the library factorizations of torch.linalg.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor
from torch.optim.optimizer import ParamsT

from ..ops import nn as nn_ops
from .common import all_reduce_, group_of, to_local
from .dion import Dion, DionMixedPrecisionConfig, validate_dion_args, validate_dion_meshes
from .orthogonalize import orthogonalize_reference
from .scalar import adamw_update, lion_update


def _gather_rows(P: Tensor, group: Optional[ProcessGroup]) -> Tensor:
    if group is None:
        return P
    parts = [torch.empty_like(P) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, P.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def orthogonalize_row_sharded(P: Tensor, qr_method: str, oversample: float, group: Optional[ProcessGroup],
                              rng: Optional[torch.Generator]) -> Tensor:
    """Orthonormalise the columns of a matrix whose rows are sharded over `group`
    (dion/dion_reference.py:792-885); returns this rank's rows."""
    if group is None or dist.get_world_size(group) == 1:
        return orthogonalize_reference(P, qr_method, oversample, rng)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    a_loc, r = P.shape
    a = a_loc * world
    dtype = P.dtype
    P32 = P.float()
    if qr_method == "cqr":
        G = P32.T @ P32
        dist.all_reduce(G, group=group)
        R, info = torch.linalg.cholesky_ex(G, upper=True)
        if int(info) == 0:
            return torch.linalg.solve_triangular(R, P32, upper=True, left=False).to(dtype)
        qr_method = "rcqr"
    if qr_method == "qr" or a <= r:
        Q, _ = torch.linalg.qr(_gather_rows(P32, group))
        return Q[rank * a_loc:(rank + 1) * a_loc].to(dtype).contiguous()
    k = math.ceil(oversample * r / 128.0) * 128
    S = torch.empty((k, a), device=P.device, dtype=P.dtype).normal_(std=math.sqrt(1.0 / k), generator=rng)
    SP = (S[:, rank * a_loc:(rank + 1) * a_loc] @ P).float()
    dist.all_reduce(SP, group=group)
    _, R = torch.linalg.qr(SP, mode="r")
    Q = torch.linalg.solve_triangular(R, P32, upper=True, left=False)
    G = Q.T @ Q
    dist.all_reduce(G, group=group)
    R, _ = torch.linalg.cholesky_ex(G, upper=True)
    return torch.linalg.solve_triangular(R, Q, upper=True, left=False).to(dtype)


def power_iteration(B: Tensor, Q_init: Tensor, power_iters: int, qr_method: str, oversample: float,
                    compressed_all_reduce: bool, replicate_mesh: Union[DeviceMesh, ProcessGroup, None] = None,
                    inner_shard_mesh_dim: Optional[int] = None, rng: Optional[torch.Generator] = None, *,
                    row_group: Optional[ProcessGroup] = None,
                    column_group: Optional[ProcessGroup] = None) -> Tuple[Tensor, Tensor]:
    """Low-rank factors of ``B ~ P Q^T`` by ``power_iters`` rounds of ``P = orth(B Q)``, ``Q = B^T P``
    (dion/dion_reference.py:690-730).

    ``B`` and ``Q_init`` are one matrix each, in the same dtype.  Sharding is described either the reference's
    way - ``B`` a DTensor whose rows are sharded over mesh dimension ``inner_shard_mesh_dim``; P comes back
    sharded like B's rows and Q replicated - or on local shards with explicit groups: ``row_group`` shards the
    rows of B (and of P), ``column_group`` its columns (and the rows of Q).  With ``compressed_all_reduce`` the
    factors are averaged over ``replicate_mesh`` instead of the gradient having been averaged beforehand."""
    if B.dtype != Q_init.dtype:
        raise TypeError(f"Expected inputs to have the same dtype, but got {B.dtype} and {Q_init.dtype}.")
    wrap = None
    if isinstance(B, DTensor):
        for i, pl in enumerate(B.placements):
            if pl.is_partial() or pl.is_shard(1) or (pl.is_shard(0) and i != inner_shard_mesh_dim):
                raise ValueError("a DTensor B may only have its rows sharded, over inner_shard_mesh_dim")
        if inner_shard_mesh_dim is not None and B.placements[inner_shard_mesh_dim].is_shard(0):
            row_group = B.device_mesh.get_group(inner_shard_mesh_dim)
        wrap = B
        B, Q_init = B.to_local(), to_local(Q_init)
    replicate = group_of(replicate_mesh) if compressed_all_reduce else None
    P, Q = None, Q_init
    for _ in range(power_iters):
        P = B @ Q
        if column_group is not None:
            dist.all_reduce(P, group=column_group)
        if replicate is not None:
            all_reduce_(P, replicate, average=True)
        P = orthogonalize_row_sharded(P, qr_method, oversample, row_group, rng)
        Q = B.T @ P
        if row_group is not None:
            dist.all_reduce(Q, group=row_group)
        if replicate is not None:
            all_reduce_(Q, replicate, average=True)
    if wrap is not None:
        from torch.distributed.tensor import Replicate

        P = DTensor.from_local(P, device_mesh=wrap.device_mesh, placements=wrap.placements, run_check=False)
        Q = DTensor.from_local(Q, device_mesh=wrap.device_mesh, placements=[Replicate()] * wrap.device_mesh.ndim,
                               run_check=False)
    return P, Q


def dion_update(X: Tensor, G: Tensor, M: Tensor, Q: Tensor, lr, mu, weight_decay, epsilon: float, transpose: bool,
                power_iters: int, qr_method: str, oversample: float = 1.25, compressed_all_reduce: bool = True,
                replicate_mesh: Union[DeviceMesh, ProcessGroup, None] = None,
                inner_shard_mesh_dim: Optional[int] = None, rng: Optional[torch.Generator] = None, *,
                row_group: Optional[ProcessGroup] = None, column_group: Optional[ProcessGroup] = None,
                full_shape: Optional[Tuple[int, int]] = None) -> Tensor:
    """One Dion step on one matrix (dion/dion_reference.py:614-687): momentum accumulation, power iteration,
    all-zero / NaN guard, error feedback, column-normalised new Q, weight decay and the scaled update.
    ``X`` and ``M`` are updated in place and the new Q (all columns, in the dtype of M) is returned for the
    caller to store.

    ``X``, ``G``, ``M`` are local shards and ``Q`` holds all of its columns; ``row_group`` / ``column_group``
    (keyword only) name the process groups that shard the rows / columns of the matrix the power iteration
    works on (``M``, or ``M^T`` with ``transpose``), and ``full_shape`` the unsharded (fan_out, fan_in) that
    scales the learning rate.  ``inner_shard_mesh_dim`` belongs to the reference's DTensor calling convention
    and is not used on local shards."""
    del inner_shard_mesh_dim
    lr, mu, weight_decay = float(lr), float(mu), float(weight_decay)
    Q_init = Q.to(M.dtype)
    M.add_(G.to(M.dtype))
    A = M.T if transpose else M
    P, R = power_iteration(A, Q_init, power_iters, qr_method, oversample, compressed_all_reduce, replicate_mesh,
                           rng=rng, row_group=row_group, column_group=column_group)
    # all-zero momentum shard: no update, keep the previous Q (shard-local check)
    is_zero = bool((M == 0).all())
    P = P.nan_to_num() * (0.0 if is_zero else 1.0)
    R = Q_init.clone() if is_zero else R.nan_to_num()

    M.add_((R @ P.T) if transpose else (P @ R.T), alpha=-(1 - mu))

    R32 = R.float()
    ss = R32.square().sum(dim=0, keepdim=True)
    if column_group is not None:
        dist.all_reduce(ss, group=column_group)
    Q_new = (R32 / (ss.sqrt() + epsilon)).to(P.dtype)

    X.mul_(1 - lr * weight_decay)
    fan_out, fan_in = full_shape if full_shape is not None else X.shape
    scaled_lr = ((fan_out / fan_in) ** 0.5) * lr
    upd = (Q_new @ P.T) if transpose else (P @ Q_new.T)
    X.add_(upd.to(X.dtype), alpha=-scaled_lr)
    return Q_new


class DionReference(Dion):
    def __init__(
        self,
        params: ParamsT,
        replicate_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        outer_shard_mesh: Optional[DeviceMesh] = None,
        inner_shard_mesh: Optional[DeviceMesh] = None,
        replicate_mesh_grad_sync: bool = True,
        rank_fraction: float = 1.0,
        rank_multiple_of: int = 1,
        lr: float = 0.01,
        mu: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: float = 0.01,
        epsilon: float = 1e-8,
        power_iters: int = 1,
        qr_method: str = "rcqr",
        cqr_warmup_steps: int = 150,
        rcqr_oversample: float = 1.25,
        mixed_precision_config: Optional[DionMixedPrecisionConfig] = None,
    ):
        validate_dion_args(lr, mu, betas, weight_decay, rank_fraction, rank_multiple_of)
        if power_iters <= 0:
            raise ValueError(f"Invalid power iterations: {power_iters}")
        if qr_method not in ("qr", "cqr", "rcqr"):
            raise ValueError(f"Unknown QR method: {qr_method}")
        validate_dion_meshes(replicate_mesh, outer_shard_mesh, inner_shard_mesh)
        super().__init__(params, replicate_mesh=replicate_mesh, outer_shard_mesh=outer_shard_mesh,
                         inner_shard_mesh=inner_shard_mesh, replicate_mesh_grad_sync=replicate_mesh_grad_sync,
                         rank_fraction=rank_fraction, rank_multiple_of=rank_multiple_of, lr=lr, mu=mu, betas=betas,
                         weight_decay=weight_decay, epsilon=epsilon, power_iters=1, qr_method="rcqr",
                         cqr_warmup_steps=cqr_warmup_steps, rcqr_oversample=rcqr_oversample,
                         mixed_precision_config=mixed_precision_config)
        self._power_iters = power_iters
        self._qr_method = qr_method
        self._cqr_warmup_steps = cqr_warmup_steps
        self._rng: Optional[torch.Generator] = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        replicate = group_of(self._replicate_mesh)
        if replicate is not None and dist.get_world_size(replicate) == 1:
            replicate = None
        for group in self.param_groups:
            algo = group["algorithm"]
            group["step"] += 1
            step = group["step"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self._get_or_initialize_state(p, group)
                cfg = self._get_dion_param_config(p)
                grad = to_local(p.grad)
                if self._replicate_mesh_grad_sync and not cfg.compressed_all_reduce and replicate is not None:
                    grad = grad.clone()
                    all_reduce_(grad, replicate, average=True)
                if algo == "dion":
                    qr_method = self._qr_method
                    if qr_method == "cqr" and step <= self._cqr_warmup_steps:
                        qr_method = "rcqr"  # CQR only once the matrices are well conditioned
                    self._dion_update(p, grad, state, cfg, group, qr_method, replicate)
                elif algo == "adamw":
                    adamw_update(to_local(p), grad, to_local(state["momentum"]), to_local(state["variance"]),
                                 group["lr"], group["beta1"], group["beta2"], group["weight_decay"], step,
                                 group["epsilon"])
                elif algo == "lion":
                    lion_update(to_local(p), grad, to_local(state["momentum"]), group["lr"], group["beta1"],
                                group["beta2"], group["weight_decay"])
                else:
                    raise ValueError(f"Unknown algorithm: {algo}")
                nn_ops.mark_shadow_stale(p)
        return loss

    def _dion_update(self, p, grad, state, cfg, group, qr_method, replicate) -> None:
        lr, mu, wd, eps = group["lr"], group["mu"], group["weight_decay"], group["epsilon"]
        X = to_local(p)
        M = to_local(state["momentum"])
        Q_loc = to_local(state["Q"])
        outer = self._mesh_dim_group(p, cfg.outer_shard_mesh_dim)
        inner = self._mesh_dim_group(p, cfg.inner_shard_mesh_dim)
        compressed = self._replicate_mesh_grad_sync and cfg.compressed_all_reduce and replicate is not None
        if self._rng is None:
            self._rng = torch.Generator(device=X.device)
            self._rng.manual_seed(0)

        if inner is not None:
            parts = [torch.empty_like(Q_loc) for _ in range(dist.get_world_size(inner))]
            dist.all_gather(parts, Q_loc.contiguous(), group=inner)
            Q_full = torch.cat(parts, dim=1)
        else:
            Q_full = Q_loc
        Q_init = Q_full.to(M.dtype)

        Q_new = dion_update(X, grad, M, Q_init, lr, mu, wd, eps, cfg.is_transposed, self._power_iters, qr_method,
                            group["oversample"], compressed, replicate, rng=self._rng, row_group=inner,
                            column_group=outer, full_shape=tuple(p.shape))

        if inner is not None:
            r_loc = Q_loc.shape[1]
            i0 = dist.get_rank(inner) * r_loc
            Q_new = Q_new[:, i0:i0 + r_loc]
        Q_loc.copy_(Q_new.to(Q_loc.dtype))

    @torch.no_grad()
    def synchronize_for_checkpoint(self):
        if self._replicate_mesh is None or not self._replicate_mesh_grad_sync:
            return
        group = group_of(self._replicate_mesh)
        for state in self.state.values():
            for val in state.values():
                if isinstance(val, Tensor):
                    all_reduce_(to_local(val), group, average=True)

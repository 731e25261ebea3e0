"""The reference's ``dion.dion_reference`` import path (dion/dion_reference.py:23-984): the per-parameter Dion as
``Dion`` and the free functions of its update.  ``orthogonalize`` here is the oracle's per-matrix routine with
its three methods (``qr``, ``cqr``, ``rcqr``), unlike the batched Cholesky-QR of ``dion_b200.dion.orthogonalize``."""

from __future__ import annotations

from typing import Optional

import torch
from torch.distributed.tensor import DTensor

from .optim.dion import DionMixedPrecisionConfig, _DionParamConfig  # noqa: F401
from .optim.dion_reference import (  # noqa: F401
    DionReference,
    dion_update,
    orthogonalize_row_sharded,
    power_iteration,
)
from .optim.functional import all_reduce_replicate_mesh, fix_all_zero_or_nan  # noqa: F401
from .optim.orthogonalize import orthogonalize_reference

Dion = DionReference
orthogonalize = orthogonalize_reference

_sketch_calls = 0


def distributed_orthogonalize(P: DTensor, qr_method: str = "rcqr", oversample: float = 1.25,
                              shard_mesh_dim: Optional[int] = None) -> DTensor:
    """Orthonormalise the columns of one matrix whose rows are sharded over mesh dimension ``shard_mesh_dim``
    with the chosen method, returning a DTensor sharded like the input (dion/dion_reference.py:792-885).  The
    random sketch of ``rcqr`` has to be the same on every rank of the shard group: it is drawn from a generator
    seeded with the number of calls made so far, which ranks that call in step share."""
    global _sketch_calls
    if not isinstance(P, DTensor) or P.ndim != 2:
        raise TypeError("expected a 2-D DTensor")
    if any(p.is_partial() or p.is_shard(1) for p in P.placements):
        raise ValueError("the input cannot be partial or sharded along its columns")
    sharded = [i for i, p in enumerate(P.placements) if p.is_shard(0)]
    if sharded not in ([], [shard_mesh_dim]):
        raise ValueError(f"rows are sharded over mesh dimensions {sharded}, not over {shard_mesh_dim}")
    group = P.device_mesh.get_group(shard_mesh_dim) if sharded else None
    local = P.to_local()
    rng = torch.Generator(device=local.device)
    rng.manual_seed(_sketch_calls)
    _sketch_calls += 1
    out = orthogonalize_row_sharded(local, qr_method, oversample, group, rng)
    return DTensor.from_local(out.contiguous(), device_mesh=P.device_mesh, placements=P.placements, run_check=False)


def all_reduce(tensor, reduce_mesh, reduce_op: str = "avg"):
    """Mean or sum of a tensor (or of a DTensor's local shard) over ``reduce_mesh``; ``None`` returns the input
    (dion/dion_reference.py:945-984)."""
    if isinstance(tensor, DTensor) and any(p.is_partial() for p in tensor.placements):
        from torch.distributed.tensor import Replicate

        tensor = tensor.redistribute(placements=[Replicate() if p.is_partial() else p for p in tensor.placements])
    return all_reduce_replicate_mesh(tensor, reduce_mesh, return_dtensor=True, reduce_op=reduce_op)

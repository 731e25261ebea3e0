"""Dion: distributed orthonormalised updates with low-rank power iteration and error feedback.

Same constructor, parameter-group keys, optimizer-state layout and update rule as the
reference's ``Dion`` (dion/dion.py:75-739 for the class, 742-1162 for the three update
functions), executed differently:

* all matrices of one (shape, placements, dtype) class are processed together: their
  momentum and Q states live in one packed buffer each (``state["momentum"]`` / ``["Q"]``
  are views into it, so checkpoints look the same), and every stage of the algorithm is
  one batched kernel launch over the whole class instead of one task per ``world_size``
  matrices;
* one local-shard formulation covers the unsharded (DDP), outer-sharded (FSDP2) and
  inner+outer-sharded (FSDP2 x TP) cases; the only things that differ are which process
  groups the partial products are reduced over;
* orthonormalisation is CholeskyQR2 on device (see optim/orthogonalize.py) instead of the
  sketch + Householder QR + triangular-solve sequence.

Notation: a weight X is m x n; "A" is M (or M^T when transposed) of shape a x b; Q is
b x r, P = A Q is a x r, R = A^T P is b x r.  The outer (FSDP) mesh shards b, the inner
(TP) mesh shards a and the columns of Q.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Generator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor, Placement, Replicate, Shard
from torch.optim.optimizer import Optimizer, ParamsT

from .. import ops
from ..ops import nn as nn_ops
from ..parallel import symm
from .common import Scheduler, all_reduce_, group_of, group_size, to_local
from .orthogonalize import SHARD_WORK, orthonormalize_many, register_split

import os

# The fused paths: partial products pushed into the consumers' symmetric memory by the GEMM epilogue and
# summed by the kernel that needs them (DION_B200_FUSED_REDUCE=0: GEMM, then a collective kernel), and
# the guard / norm / new-Q chain after R as one kernel (DION_B200_FUSED_POST=0: element-wise torch ops).
FUSED_REDUCE = os.environ.get("DION_B200_FUSED_REDUCE", "1") != "0"
FUSED_POST = os.environ.get("DION_B200_FUSED_POST", "1") != "0"
# an all-reduce by pushing to every rank costs (world - 1) times the data; beyond this group size the
# product is reduced by the all-reduce kernel instead
_MAX_PUSH_WORLD = 4

try:  # pragma: no cover - depends on the torch build
    from torch.distributed.tensor.placement_types import _StridedShard
except ImportError:  # pragma: no cover
    _StridedShard = None


@dataclass
class DionMixedPrecisionConfig:
    """dtypes of the optimizer states; ``None`` keeps the parameter's dtype
    (dion/dion.py:59-72)."""

    momentum_dtype: Optional[torch.dtype] = None
    Q_dtype: Optional[torch.dtype] = None
    variance_dtype: Optional[torch.dtype] = None


@dataclass
class _DionParamConfig:
    """How one parameter is sharded and which orientation the power iteration uses.
    Recomputed from the live tensors, never checkpointed (dion/dion.py:33-56, 194-196)."""

    outer_shard_tensor_dim: Optional[int] = None
    inner_shard_tensor_dim: Optional[int] = None
    outer_shard_mesh_dim: Optional[int] = None
    inner_shard_mesh_dim: Optional[int] = None
    is_transposed: bool = False
    compressed_all_reduce: bool = False
    Q_sharded_placements: Optional[Tuple[Placement, ...]] = None
    Q_inner_unsharded_placements: Optional[Tuple[Placement, ...]] = None


def validate_dion_args(lr, mu, betas, weight_decay, rank_fraction, rank_multiple_of):
    if lr < 0.0:
        raise ValueError(f"Invalid learning rate: {lr}")
    if mu < 0.0:
        raise ValueError(f"Invalid momentum factor (mu): {mu}")
    if len(betas) != 2 or betas[0] < 0.0 or betas[1] < 0.0:
        raise ValueError(f"Invalid betas: {betas}")
    if weight_decay < 0.0:
        raise ValueError(f"Invalid weight_decay value: {weight_decay}")
    if rank_fraction <= 0 or rank_fraction > 1:
        raise ValueError(f"Invalid rank fraction: {rank_fraction}")
    if rank_multiple_of <= 0:
        raise ValueError(f"Invalid rank multiple of: {rank_multiple_of}")


def validate_dion_meshes(replicate_mesh, outer_shard_mesh, inner_shard_mesh):
    if replicate_mesh is not None and not isinstance(replicate_mesh, (DeviceMesh, ProcessGroup)):
        raise TypeError(f"Replicate mesh must be a DeviceMesh or ProcessGroup, but got {type(replicate_mesh)}.")
    for name, mesh in (("Outer", outer_shard_mesh), ("Inner", inner_shard_mesh)):
        if mesh is None:
            continue
        if not isinstance(mesh, DeviceMesh):
            raise TypeError(f"{name} shard mesh must be a DeviceMesh, but got {type(mesh)}.")
        if mesh.ndim != 1:
            raise ValueError(f"{name} shard mesh must be 1D, but got {mesh.ndim}D. Try using a 1D sub-mesh.")
        if mesh == replicate_mesh:
            raise ValueError(f"{name} shard mesh must be different from replicate mesh.")
    if inner_shard_mesh is not None and inner_shard_mesh == outer_shard_mesh:
        raise ValueError("Outer and inner shard meshes must be different.")


def low_rank_dim(m: int, n: int, rank_fraction: float, rank_multiple_of: int) -> int:
    """r = rank_fraction * min(m, n), rounded up to a multiple, clamped (dion.py:673-676)."""
    r = rank_fraction * min(m, n)
    r = rank_multiple_of * math.ceil(r / rank_multiple_of)
    return int(min(r, m, n))


# steps the shifted two-pass orthonormalisation stays on after the last step that needed it
ROBUST_STEPS = 20


class _PackedClass:
    """All Dion parameters of one (shape, placements, dtype, group) class with their states
    packed into ``M: [B, m_loc, n_loc]`` and ``Q: [B, q_rows_loc, r_loc]``."""

    def __init__(self, params: List[Tensor], cfg: _DionParamConfig, M: Tensor, Q: Tensor):
        self.params = params
        self.cfg = cfg
        self.M = M
        self.Q = Q
        self.x_ptrs: Optional[Tensor] = None
        self.x_ptr_list: Optional[List[int]] = None
        self.shadow_ptrs: Optional[Tensor] = None
        self.shadow_ptr_list: Optional[List[int]] = None
        self.nonzero: Optional[Tensor] = None
        self.ptr_cache: Dict[tuple, Tensor] = {}  # device tables of push destinations, by buffer placement
        # conditioning of P: steps the ill-conditioned treatment of the orthonormalisation stays on, and
        # the (asynchronously fetched) count of matrices that asked for it in the last step
        self.robust_left = 0
        self.cond_host: Optional[Tensor] = None
        self.cond_event = None


class _ClassWork:
    """Per-step working set of one parameter class between the two phases of the update."""

    __slots__ = ("cls", "params", "group", "replicate", "outer", "inner", "sync", "compressed", "A", "Qm", "P", "P_total")


class Dion(Optimizer):
    """Distributed Dion optimizer (https://arxiv.org/abs/2504.05295).

    Args mirror the reference: ``replicate_mesh`` (DeviceMesh or ProcessGroup, data-parallel
    replicas), ``outer_shard_mesh`` (FSDP dimension, replicated during orthogonalisation),
    ``inner_shard_mesh`` (TP dimension, sharded during orthogonalisation),
    ``replicate_mesh_grad_sync`` (the optimizer synchronises gradients - compressed to the
    low-rank factors where that is cheaper), ``rank_fraction`` / ``rank_multiple_of``,
    ``lr`` (scaled by sqrt(fan_out/fan_in) for matrices), ``mu``, ``betas`` (for the
    ``adamw`` / ``lion`` parameter groups), ``weight_decay``, ``epsilon``,
    ``mixed_precision_config``.  Only ``power_iters=1`` and ``qr_method="rcqr"`` are
    accepted, as in the reference (``cqr_warmup_steps`` and ``rcqr_oversample`` are kept for
    signature and checkpoint compatibility; the device-side CholeskyQR2 needs neither).

    Parameters are either all DTensors (with DeviceMesh arguments) or all plain tensors
    (with a ProcessGroup ``replicate_mesh``), sharded uniformly.
    """

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
        if power_iters != 1:
            raise ValueError("Async Dion only supports power_iters=1")
        if qr_method != "rcqr":
            raise ValueError("Async Dion only supports qr_method='rcqr'")
        validate_dion_meshes(replicate_mesh, outer_shard_mesh, inner_shard_mesh)

        defaults = dict(
            rank_fraction=rank_fraction,
            rank_multiple_of=rank_multiple_of,
            lr=lr,
            mu=mu,
            beta1=betas[0],
            beta2=betas[1],
            weight_decay=weight_decay,
            epsilon=epsilon,
            oversample=rcqr_oversample,
            algorithm="dion",
            step=0,
        )
        super().__init__(params, defaults)

        self._param_config: Dict[Tensor, _DionParamConfig] = {}
        self._packed: Dict[tuple, _PackedClass] = {}
        self._replicate_mesh = replicate_mesh
        self._outer_shard_mesh = outer_shard_mesh
        self._inner_shard_mesh = inner_shard_mesh
        self._replicate_mesh_grad_sync = replicate_mesh_grad_sync
        self._replicate_world_size = group_size(replicate_mesh)
        self._outer_shard_ranks = (dist.get_process_group_ranks(outer_shard_mesh.get_group())
                                   if outer_shard_mesh is not None else None)
        self._inner_shard_ranks = (dist.get_process_group_ranks(inner_shard_mesh.get_group())
                                   if inner_shard_mesh is not None else None)
        self._mixed_precision_config = mixed_precision_config or DionMixedPrecisionConfig()
        # how often P left a reduction as this rank's share of the batch (reduce-scatter instead of all-reduce)
        self.p_reduce_scatters = 0
        # how often a class of matrices went into the ill-conditioned treatment of the orthonormalisation
        self.robust_switches = 0
        # Q factors are drawn from this generator so that every rank draws the same values
        self._q_seed = 0x0D10

    # ------------------------------------------------------------------ public API

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        dion_groups, lion_groups, adamw_groups = [], [], []
        for group in self.param_groups:
            group["step"] += 1
            algo = group["algorithm"]
            if algo == "dion":
                dion_groups.append(group)
            elif algo == "lion":
                lion_groups.append(group)
            elif algo == "adamw":
                adamw_groups.append(group)
            else:
                raise ValueError(f"Unknown algorithm: {algo}")

        # The update of every (shape, placements, dtype) class runs in two phases around one
        # joint orthonormalisation, so that the Gram matrices of all classes are factorised
        # by a single kernel launch.  Within a phase the classes are interleaved by the
        # scheduler: while one waits for a collective, the others issue their kernels.
        work: List[_ClassWork] = []
        for group in dion_groups:
            work.extend(self._dion_classes(group))

        def phase1():
            for w in work:
                yield lambda w=w: self._dion_phase1(w)
            for group in lion_groups:
                yield lambda g=group: self._scalar_task(g, "lion")
            for group in adamw_groups:
                yield lambda g=group: self._scalar_task(g, "adamw")

        if work:
            # Arena creation is collective over each group, so every rank must walk its groups in an
            # order that is consistent across the whole job: by mesh role (replicate, outer, inner),
            # never by group name, which differs between the sub-groups of one mesh dimension.
            groups = []
            for pick in (lambda w: w.replicate if w.compressed else None, lambda w: w.outer, lambda w: w.inner):
                for w in work:
                    g = pick(w)
                    if g is not None and all(g is not h for h in groups):
                        groups.append(g)
            symm.begin_step(groups, work[0].cls.M.device)
        Scheduler(phase1(), max_in_flight=3).run()
        if work:
            # P is the same on every rank of the outer (or else the replicate) group by now: each rank
            # orthonormalises its share of every batch and the shares are all-gathered
            infos: List[Tensor] = []
            ortho = orthonormalize_many([w.P for w in work], [w.inner for w in work],
                                        shard_groups=[w.outer if w.outer is not None else w.replicate for w in work],
                                        totals=[w.P_total for w in work],
                                        out_dtypes=[w.cls.M.dtype for w in work],  # what phase 2 multiplies with
                                        robust=[w.cls.robust_left > 0 for w in work], infos=infos)
            for w, info in zip(work, infos):
                self._note_conditioning(w.cls, info)
            for w, P in zip(work, ortho):
                w.P = P
            Scheduler((lambda w=w: self._dion_phase2(w) for w in work), max_in_flight=3).run()
        return loss

    def _note_conditioning(self, cls: _PackedClass, info: Tensor) -> None:
        """Switch the ill-conditioned treatment of a class on for ROBUST_STEPS steps when its
        factorisation gave up on a pivot (or, while the treatment is on, reports that it still would).
        On GPUs the count travels to the host asynchronously and is read one step later - by then the
        copy has long finished, so the read does not stall the GPU, and every rank that factorised the
        same matrices (the ranks of a tensor-parallel group, whose Gram matrices are all-reduced) takes
        the same decision at the same step.  The step that discovers the problem runs the plain path
        (bounded, columns dropped)."""
        count = None
        if not info.is_cuda:
            count = int(info.sum())
        else:
            if cls.cond_event is not None:
                cls.cond_event.synchronize()          # recorded a whole step ago
                count = int(cls.cond_host.item())
            if cls.cond_host is None:
                cls.cond_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
                cls.cond_event = torch.cuda.Event()
            cls.cond_host.copy_(info.sum(dtype=torch.int32).view(1), non_blocking=True)
            cls.cond_event.record()
        if count is not None:
            if count > 0:
                if cls.robust_left == 0:
                    self.robust_switches += 1
                cls.robust_left = ROBUST_STEPS
            elif cls.robust_left > 0:
                cls.robust_left -= 1

    @torch.no_grad()
    def synchronize_for_checkpoint(self):
        """Average every optimizer-state tensor over the replicate mesh.  With compressed
        gradient synchronisation the momentum is decoupled across data-parallel replicas, so
        this must run before a distributed checkpoint is written (dion/dion.py:273-311).  A
        no-op without a replicate mesh or when the optimizer does not own gradient sync."""
        if self._replicate_mesh is None or not self._replicate_mesh_grad_sync:
            return
        tensors: List[Tensor] = []
        seen = set()
        for cls in self._packed.values():
            for t in (cls.M, cls.Q):
                tensors.append(t)
                seen.add(t.untyped_storage().data_ptr())
        for state in self.state.values():
            for val in state.values():
                if isinstance(val, Tensor):
                    loc = to_local(val)
                    if loc.untyped_storage().data_ptr() not in seen:
                        tensors.append(loc)
        group = group_of(self._replicate_mesh)
        # bucketed: one collective per ~256 MB
        bucket, size = [], 0
        for t in tensors:
            bucket.append(t)
            size += t.numel() * t.element_size()
            if size >= (256 << 20):
                all_reduce_(bucket, group, average=True)
                bucket, size = [], 0
        if bucket:
            all_reduce_(bucket, group, average=True)

    def load_state_dict(self, state_dict) -> None:
        """torch casts loaded floating-point state to the parameter dtype; restore the dtypes
        of the mixed-precision configuration afterwards so a resumed run keeps its numerics."""
        super().load_state_dict(state_dict)
        self._packed.clear()
        mp = self._mixed_precision_config
        wanted = {"momentum": mp.momentum_dtype, "Q": mp.Q_dtype, "variance": mp.variance_dtype}
        for state in self.state.values():
            for key, dtype in wanted.items():
                val = state.get(key)
                if dtype is not None and isinstance(val, Tensor) and val.dtype != dtype:
                    state[key] = val.to(dtype)

    # ------------------------------------------------------------------ parameter classification

    def _get_dion_param_config(self, x: Tensor) -> _DionParamConfig:
        """Sharding facts of one parameter (rules of dion/dion.py:498-607)."""
        cfg = self._param_config.get(x)
        if cfg is not None:
            return cfg
        if x.ndim > 2:
            raise NotImplementedError(
                f"Tensors with more than 2 dimensions are not supported. Got {x.ndim}D tensor.")
        using_device_mesh = any(isinstance(m, DeviceMesh)
                                for m in (self._replicate_mesh, self._outer_shard_mesh, self._inner_shard_mesh))
        using_process_group = isinstance(self._replicate_mesh, ProcessGroup)
        if using_device_mesh and not isinstance(x, DTensor):
            raise TypeError("When using DeviceMesh, all parameters must be DTensor.")
        if using_process_group and isinstance(x, DTensor):
            raise TypeError("When using DTensor parameters, the data parallel group must be specified by a "
                            "DeviceMesh instead of ProcessGroup.")

        cfg = _DionParamConfig()
        if x.ndim == 2:
            m, n = x.shape
            cfg.is_transposed = m < n

        if isinstance(x, DTensor) and x.ndim == 2:
            mesh = x.device_mesh
            placements = x.placements
            assert len(placements) == mesh.ndim
            owner_of_dim: List[Optional[int]] = [None, None]
            for mesh_dim, placement in enumerate(placements):
                if _StridedShard is not None and isinstance(placement, _StridedShard):
                    raise NotImplementedError(
                        "StridedShard is not supported. Ensure that FSDP and TP shard different dimensions of "
                        "each matrix.")
                if not placement.is_shard():
                    continue
                tdim = placement.dim
                if owner_of_dim[tdim] is not None:
                    raise RuntimeError(f"Got double-sharded DTensor for tensor dimension {tdim}.")
                owner_of_dim[tdim] = mesh_dim
                ranks = dist.get_process_group_ranks(mesh.get_group(mesh_dim))
                is_outer = ranks == self._outer_shard_ranks
                is_inner = ranks == self._inner_shard_ranks
                if is_outer:
                    cfg.outer_shard_tensor_dim, cfg.outer_shard_mesh_dim = tdim, mesh_dim
                if is_inner:
                    cfg.inner_shard_tensor_dim, cfg.inner_shard_mesh_dim = tdim, mesh_dim
                if is_outer and is_inner:
                    raise RuntimeError("Cannot have outer and inner sharding over the same process group.")
                if mesh.size(mesh_dim) > 1 and not is_outer and not is_inner:
                    raise RuntimeError(
                        f"Got DTensor sharded on unrecognized {mesh_dim=}, which does not match outer_shard_mesh "
                        f"or inner_shard_mesh.")
            # orthogonalise along the inner-sharded dimension
            if cfg.inner_shard_tensor_dim == 0 or cfg.outer_shard_tensor_dim == 1:
                cfg.is_transposed = False
            if cfg.outer_shard_tensor_dim == 0 or cfg.inner_shard_tensor_dim == 1:
                cfg.is_transposed = True

        self._param_config[x] = cfg
        return cfg

    def _split_params_by_sharding(self, params: List[Tensor]) -> Dict[str, List[Tensor]]:
        out: Dict[str, List[Tensor]] = {"inner_sharded": [], "outer_sharded": [], "non_sharded": []}
        for p in params:
            cfg = self._get_dion_param_config(p)
            if cfg.inner_shard_mesh_dim is not None:
                out["inner_sharded"].append(p)
            elif cfg.outer_shard_mesh_dim is not None:
                out["outer_sharded"].append(p)
            else:
                out["non_sharded"].append(p)
        return out

    # ------------------------------------------------------------------ state

    def _init_opt_state_momentum(self, param: Tensor, state: Dict[str, Any]):
        state["momentum"] = torch.zeros_like(param, dtype=self._mixed_precision_config.momentum_dtype)

    def _init_opt_state_adam(self, param: Tensor, state: Dict[str, Any]):
        self._init_opt_state_momentum(param, state)
        state["variance"] = torch.zeros_like(param, dtype=self._mixed_precision_config.variance_dtype)

    def _draw_q(self, shape: Tuple[int, int], device, dtype) -> Tensor:
        """Full (unsharded) random Q, identical on every rank: seeded generator on the
        device, then broadcast from the first rank of the replicate group / world."""
        gen = torch.Generator(device=device)
        gen.manual_seed(self._q_seed)
        self._q_seed += 1
        q = torch.randn(shape, device=device, dtype=torch.float32, generator=gen).to(dtype)
        return q

    def _init_opt_state_dion(self, param: Tensor, state: Dict[str, Any], rank_fraction: float,
                             rank_multiple_of: int):
        """momentum like the parameter; Q of shape (m, r) if transposed else (n, r), as a
        DTensor sharded Shard(0) on the outer and Shard(1) on the inner mesh dimension
        (dion/dion.py:649-721)."""
        if param.ndim != 2:
            raise ValueError(
                f"Expected Dion parameters to be 2D matrix, but got {param.ndim}D. "
                f"For scalar parameters, set 'algorithm' to 'lion' or 'adamw' when creating param group.")
        cfg = self._get_dion_param_config(param)
        self._init_opt_state_momentum(param, state)
        m, n = param.shape
        r = low_rank_dim(m, n, rank_fraction, rank_multiple_of)
        q_shape = (m, r) if cfg.is_transposed else (n, r)
        if rank_fraction < 1 and (m + n) * r < m * n:
            cfg.compressed_all_reduce = True
        q_dtype = self._mixed_precision_config.Q_dtype or param.dtype

        local_param = to_local(param)
        q_full = self._draw_q(q_shape, local_param.device, q_dtype)
        if isinstance(param, DTensor):
            placements: List[Placement] = [Replicate() for _ in range(param.device_mesh.ndim)]
            if cfg.outer_shard_mesh_dim is not None:
                placements[cfg.outer_shard_mesh_dim] = Shard(0)
            if cfg.inner_shard_mesh_dim is not None:
                placements[cfg.inner_shard_mesh_dim] = Shard(1)
            cfg.Q_sharded_placements = tuple(placements)
            if cfg.inner_shard_mesh_dim is not None:
                unsharded = list(placements)
                unsharded[cfg.inner_shard_mesh_dim] = Replicate()
                cfg.Q_inner_unsharded_placements = tuple(unsharded)
            else:
                cfg.Q_inner_unsharded_placements = None
            if dist.is_initialized():
                dist.broadcast(q_full, src=0)
            q_local = q_full
            mesh = param.device_mesh
            for mesh_dim, pl in enumerate(placements):
                if pl.is_shard():
                    size = mesh.size(mesh_dim)
                    if q_local.size(pl.dim) % size != 0:
                        hint = ("use rank_multiple_of to round the rank" if pl.dim == 1 else
                                "the sharded dimension of the weight has to be a multiple of the mesh size "
                                "(uneven shards are not supported)")
                        raise ValueError(
                            f"Q dimension {pl.dim} of size {q_local.size(pl.dim)} is not divisible by the mesh "
                            f"size {size}; {hint}.")
                    idx = mesh.get_local_rank(mesh_dim)
                    q_local = q_local.chunk(size, dim=pl.dim)[idx]
            state["Q"] = DTensor.from_local(q_local.contiguous(), device_mesh=mesh, placements=placements,
                                            run_check=False)
        else:
            self._replicate_mesh_broadcast(q_full)
            state["Q"] = q_full

    def _replicate_mesh_broadcast(self, tensor: Tensor):
        if self._replicate_mesh is None:
            return
        if isinstance(self._replicate_mesh, DeviceMesh):
            for group in self._replicate_mesh.get_all_groups():
                dist.broadcast(tensor, group=group, group_src=0)
        elif isinstance(self._replicate_mesh, ProcessGroup):
            dist.broadcast(tensor, group=self._replicate_mesh, group_src=0)
        else:
            raise TypeError("Data parallel mesh must be either a DeviceMesh or ProcessGroup.")

    def _get_or_initialize_state(self, param: Tensor, group: dict) -> dict:
        state = self.state[param]
        if not state:
            algo = group["algorithm"]
            if algo == "dion":
                self._init_opt_state_dion(param, state, group["rank_fraction"], group["rank_multiple_of"])
            elif algo == "adamw":
                self._init_opt_state_adam(param, state)
            elif algo in ("lion", "clion"):
                self._init_opt_state_momentum(param, state)
            else:
                raise ValueError(f"Unknown algorithm: {algo}")
        return state

    # ------------------------------------------------------------------ packing

    def _pack(self, key: tuple, params: List[Tensor], group: dict) -> _PackedClass:
        """Make the states of `params` views of two packed buffers (copying current values),
        reusing the existing pack while membership and storage are unchanged."""
        cls = self._packed.get(key)
        states = [self._get_or_initialize_state(p, group) for p in params]
        cfg = self._get_dion_param_config(params[0])
        if cls is not None and len(cls.params) == len(params) and all(a is b for a, b in zip(cls.params, params)):
            intact = True
            for i, s in enumerate(states):
                m_loc, q_loc = to_local(s["momentum"]), to_local(s["Q"])
                if m_loc.data_ptr() != cls.M[i].data_ptr() or q_loc.data_ptr() != cls.Q[i].data_ptr() \
                        or m_loc.dtype != cls.M.dtype or q_loc.dtype != cls.Q.dtype:
                    intact = False
                    break
            if intact:
                return cls
        m0, q0 = to_local(states[0]["momentum"]), to_local(states[0]["Q"])
        M = torch.empty((len(params), *m0.shape), dtype=m0.dtype, device=m0.device)
        Q = torch.empty((len(params), *q0.shape), dtype=q0.dtype, device=q0.device)
        for i, (p, s) in enumerate(zip(params, states)):
            M[i].copy_(to_local(s["momentum"]))
            Q[i].copy_(to_local(s["Q"]))
            mom, q = s["momentum"], s["Q"]
            if isinstance(mom, DTensor):
                s["momentum"] = DTensor.from_local(M[i], device_mesh=mom.device_mesh, placements=mom.placements,
                                                   run_check=False, shape=mom.shape, stride=mom.stride())
            else:
                s["momentum"] = M[i]
            if isinstance(q, DTensor):
                s["Q"] = DTensor.from_local(Q[i], device_mesh=q.device_mesh, placements=q.placements,
                                            run_check=False, shape=q.shape, stride=q.stride())
            else:
                s["Q"] = Q[i]
        cls = _PackedClass(list(params), cfg, M, Q)
        self._packed[key] = cls
        return cls

    # ------------------------------------------------------------------ Dion update

    def _dion_classes(self, group: dict) -> List["_ClassWork"]:
        """Parameters of `group` that have gradients, split into classes of identical
        (shape, placements, dtype) with their packed states and process groups resolved."""
        params = [p for p in group["params"] if p.grad is not None]
        classes: Dict[tuple, List[Tensor]] = {}
        for p in params:
            placements = tuple(p.placements) if isinstance(p, DTensor) else None
            transposed = self._get_dion_param_config(p).is_transposed
            classes.setdefault((tuple(p.shape), placements, p.dtype, id(group), transposed), []).append(p)
        replicate = group_of(self._replicate_mesh)
        if replicate is not None and dist.get_world_size(replicate) == 1:
            replicate = None
        out = []
        for key, members in classes.items():
            cls = self._pack(key, members, group)
            w = _ClassWork()
            w.cls, w.params, w.group = cls, members, group
            w.replicate = replicate
            w.outer = self._mesh_dim_group(members[0], cls.cfg.outer_shard_mesh_dim)
            w.inner = self._mesh_dim_group(members[0], cls.cfg.inner_shard_mesh_dim)
            w.sync = self._replicate_mesh_grad_sync and replicate is not None
            w.compressed = w.sync and cls.cfg.compressed_all_reduce
            out.append(w)
        return out

    @staticmethod
    def _reduce(t: Tensor, group: ProcessGroup, average: bool):
        """All-reduce `t` over `group`.  Buffers that live in the group's symmetric arena are
        reduced by the in-tree kernel on the current stream (returns None); anything else
        starts the library collective asynchronously and returns its wait() callable."""
        arena = symm.arena_for(group)
        if arena is not None and t.is_cuda and arena.offset_of(t) is not None:
            symm.all_reduce(t, group, average=average)
            return None
        return all_reduce_(t, group, average=average, async_op=True)

    def _q_gatherer(self, group: ProcessGroup, device):
        """All-gather object for the columns of Q over the inner (tensor-parallel) group
        (dion/dion.py:1063-1070 redistributes Q with a DTensor all-gather), or None where the symmetric
        memory kernels do not apply (CPU tensors, gloo, more than eight ranks)."""
        if device.type != "cuda":
            return None
        key = symm._key(group)
        cache = self.__dict__.setdefault("_q_gatherers", {})
        if key not in cache:
            from ..parallel import fsdp_comm

            cache[key] = fsdp_comm.SymmAllGather(group, device) if fsdp_comm._usable(group, device) else None
        return cache[key]

    def _mesh_dim_group(self, p: Tensor, mesh_dim: Optional[int]) -> Optional[ProcessGroup]:
        if mesh_dim is None or not isinstance(p, DTensor):
            return None
        g = p.device_mesh.get_group(mesh_dim)
        return g if dist.get_world_size(g) > 1 else None

    def _dion_phase1(self, w: "_ClassWork") -> Generator[None, None, None]:
        """Gradient sync, momentum accumulation and P = A Q reduced over the meshes."""
        cls, cfg = w.cls, w.cls.cfg
        B = len(w.params)
        M, Qs = cls.M, cls.Q
        G = [to_local(p.grad) for p in w.params]

        # 0. full-gradient synchronisation when compression does not pay (dion.py:785-791)
        if w.sync and not w.compressed:
            wait = all_reduce_(G, w.replicate, average=True, async_op=True)
            yield
            wait()

        # 1. momentum accumulation, remembering which matrices are entirely zero
        if cls.nonzero is None:
            cls.nonzero = torch.zeros(B, dtype=torch.int32, device=M.device)
        else:
            cls.nonzero.zero_()
        ops.dion_accumulate(G, list(M.unbind(0)), cls.nonzero)

        # 2. Q with all of its columns (gathered over the inner mesh), in the momentum dtype
        if w.inner is not None:
            w_in = dist.get_world_size(w.inner)
            gathered = torch.empty((w_in * B, Qs.shape[1], Qs.shape[2]), dtype=Qs.dtype, device=Qs.device)
            gather = self._q_gatherer(w.inner, Qs.device)
            if gather is not None:
                # the all-gather kernel over symmetric memory (it uses the process group by itself for
                # sizes or alignments it does not cover); blocking in stream order, so nothing to wait for
                before = gather.kernel_calls
                gather(gathered.view(-1), Qs.contiguous().view(-1), w.inner)
                symm.count("dion_q_gather", gather.kernel_calls > before)
            else:
                work = dist.all_gather_into_tensor(gathered, Qs.contiguous(), group=w.inner, async_op=True)
                yield
                work.wait()
            Q_full = gathered.view(w_in, B, Qs.shape[1], Qs.shape[2]).permute(1, 2, 0, 3).reshape(
                B, Qs.shape[1], w_in * Qs.shape[2])
        else:
            Q_full = Qs
        w.Qm = Q_full.to(M.dtype)

        # 3. P = A Q, partial over the outer mesh
        w.A = M.transpose(1, 2) if cfg.is_transposed else M
        a_loc = w.A.shape[1]
        first = w.outer if w.outer is not None else (w.replicate if w.compressed else None)
        w.P_total = None
        if first is not None and FUSED_REDUCE and M.is_cuda:
            second = w.replicate if (w.outer is not None and w.compressed) else None
            P = self._p_pushed(w, first, second, B, a_loc, w.Qm.shape[2])
            if P is not None:
                symm.count("dion_p_exchange", True)
                w.P = P
                return
            symm.count("dion_p_exchange", False)
        # the GEMM writes straight into the symmetric arena of the group that reduces P first
        P = symm.empty(first, (B, a_loc, w.Qm.shape[2]), torch.float32, M.device)
        ops.gemm(w.A, w.Qm, out=P)
        # The ranks of the first reducing group are the ones that divide the orthonormalisation among
        # themselves (see step()).  When the batch splits evenly, a reduce-scatter leaves every rank with
        # exactly the matrices it is going to orthonormalise (dion/dion.py:806-815, 925-929) instead of an
        # all-reduce of which it would drop all but its share.
        share_world = dist.get_world_size(first) if first is not None else 1
        if (SHARD_WORK and first is not None and w.inner is None and B > 1 and B % share_world == 0
                and (P[0].numel() * 4) % 16 == 0):
            w.P_total = B
            self.p_reduce_scatters += 1
            share = symm.empty(w.replicate if (w.outer is not None and w.compressed) else None,
                               (B // share_world, a_loc, w.Qm.shape[2]), torch.float32, M.device)
            symm.reduce_scatter(P, first, average=w.outer is None, out=share)
            P = share
            if w.outer is not None and w.compressed:
                wait = self._reduce(P, w.replicate, average=True)
                if wait is not None:
                    yield
                    wait()
        else:
            if w.outer is not None:
                wait = self._reduce(P, w.outer, average=False)
                if wait is not None:
                    yield
                    wait()
            if w.compressed:
                wait = self._reduce(P, w.replicate, average=True)
                if wait is not None:
                    yield
                    wait()
        w.P = P  # 4. is the joint orthonormalisation in step()

    def _dion_phase2(self, w: "_ClassWork") -> Generator[None, None, None]:
        """R = A^T P, error feedback, new Q and the weight update."""
        cls, cfg, group = w.cls, w.cls.cfg, w.group
        params = w.params
        p0 = params[0]
        lr, mu, wd, eps = group["lr"], group["mu"], group["weight_decay"], group["epsilon"]
        B = len(params)
        M, Qs, A, Qm = cls.M, cls.Q, w.A, w.Qm
        X = [to_local(p) for p in params]
        Pm = w.P.to(M.dtype)

        # 5. R = A^T P, partial over the inner mesh
        first = w.inner if w.inner is not None else (w.replicate if w.compressed else None)
        n_loc, r = A.shape[2], Pm.shape[2]
        fan_out, fan_in = p0.shape[0], p0.shape[1]
        scaled_lr = ((fan_out / fan_in) ** 0.5) * lr
        alpha = -(1.0 - mu)
        beta = 1.0 - lr * wd
        r_loc = Qs.shape[2]
        i0 = dist.get_rank(w.inner) * r_loc if w.inner is not None else 0

        if M.is_cuda and FUSED_POST:
            # 5.-8. on GPUs: the partial products go into slots (pushed to the ranks that need the sum where
            # there are several), and one kernel sums them, applies the all-zero / NaN guard to R and P,
            # writes R in the momentum dtype, the column sums of squares and - unless those still have to
            # be completed over the outer mesh - the new Q, including this rank's columns of the Q state
            slots, scale, wait = None, 1.0, None
            if first is not None and FUSED_REDUCE:
                second = w.replicate if (w.inner is not None and w.compressed) else None
                pushed = self._r_pushed(w, first, second, B, n_loc, r, Pm)
                symm.count("dion_r_exchange", pushed is not None)
                if pushed is not None:
                    slots, scale, wait = pushed
            if slots is None:
                R = symm.empty(first, (B, n_loc, r), torch.float32, M.device)
                ops.gemm(A.transpose(1, 2), Pm, out=R)
                if w.inner is not None:
                    wait_fn = self._reduce(R, w.inner, average=False)
                    if wait_fn is not None:
                        yield
                        wait_fn()
                if w.compressed:
                    wait_fn = self._reduce(R, w.replicate, average=True)
                    if wait_fn is not None:
                        yield
                        wait_fn()
                slots = R.unsqueeze(0)
            finish = w.outer is None
            Rm = torch.empty((B, n_loc, r), dtype=M.dtype, device=M.device)
            # the new Q doubles as the Q state when that holds all columns in the dtype the update multiplies with
            q_is_state = w.inner is None and Qs.dtype == M.dtype
            Qn = Qs if q_is_state else torch.empty((B, n_loc, r), dtype=M.dtype, device=M.device)
            ss = symm.empty(w.outer, (B, r), torch.float32, M.device)
            R32 = None if finish else torch.empty((B, n_loc, r), dtype=torch.float32, device=M.device)
            ops.dion_r_post(slots, scale, cls.nonzero, Qm, Pm, R32, Rm, ss, finish, eps,
                            None if q_is_state else Qn, Qs, i0, wait)
            if not finish:
                wait_fn = self._reduce(ss, w.outer, average=False)
                if wait_fn is not None:
                    yield
                    wait_fn()
                ops.dion_q_norm(R32, ss, Qm, eps, None if q_is_state else Qn, Qs, i0)
            # 7. error feedback  M -= (1 - mu) P R^T, 9. weight decay and update
            if cfg.is_transposed:
                ops.gemm(Rm, Pm.transpose(1, 2), c=M, out=M, alpha=alpha, beta=1.0)
                a_op, b_op = Qn, Pm.transpose(1, 2)
            else:
                ops.gemm(Pm, Rm.transpose(1, 2), c=M, out=M, alpha=alpha, beta=1.0)
                a_op, b_op = Pm, Qn.transpose(1, 2)
            self._apply_update(cls, params, X, a_op, b_op, -scaled_lr, beta)
            w.A = w.Qm = w.P = w.P_total = None
            return

        R = symm.empty(first, (B, n_loc, r), torch.float32, M.device)
        ops.gemm(A.transpose(1, 2), Pm, out=R)
        if w.inner is not None:
            wait = self._reduce(R, w.inner, average=False)
            if wait is not None:
                yield
                wait()
        if w.compressed:
            wait = self._reduce(R, w.replicate, average=True)
            if wait is not None:
                yield
                wait()

        # 6. all-zero / NaN guard, shard-local like the reference (dion.py:1416-1444):
        #    an all-zero momentum gives P = 0 and keeps the previous Q
        nz = (cls.nonzero != 0).view(B, 1, 1)
        Pm = torch.where(nz, Pm.nan_to_num(), torch.zeros_like(Pm))
        R = torch.where(nz, R.nan_to_num(), Qm.float())
        Rm = R.to(M.dtype)

        # 7. error feedback  M -= (1 - mu) P R^T
        if cfg.is_transposed:
            ops.gemm(Rm, Pm.transpose(1, 2), c=M, out=M, alpha=alpha, beta=1.0)
        else:
            ops.gemm(Pm, Rm.transpose(1, 2), c=M, out=M, alpha=alpha, beta=1.0)

        # 8. new Q: column-normalised R (sum of squares completed over the outer mesh)
        ss = ops.col_sumsq(R, out=symm.empty(w.outer, (B, R.shape[2]), torch.float32, M.device))
        if w.outer is not None:
            wait = self._reduce(ss, w.outer, average=False)
            if wait is not None:
                yield
                wait()
        Qn = (R / (ss.sqrt().unsqueeze(1) + eps)).to(M.dtype)
        # a column of P that the orthonormalisation dropped (P was rank deficient) leaves a zero column
        # in R: it keeps its previous Q, like a whole matrix whose momentum is zero does
        Qn = torch.where((ss > 0).unsqueeze(1), Qn, Qm)

        # 9. weight decay and update  X = (1 - lr wd) X - lr sqrt(fan_out / fan_in) P Qn^T
        if cfg.is_transposed:
            a_op, b_op = Qn, Pm.transpose(1, 2)
        else:
            a_op, b_op = Pm, Qn.transpose(1, 2)
        self._apply_update(cls, params, X, a_op, b_op, -scaled_lr, beta)

        # 10. keep this rank's columns of the new Q (dion.py:1533-1561)
        if w.inner is not None:
            Qs.copy_(Qn[:, :, i0:i0 + r_loc])
        else:
            Qs.copy_(Qn)
        w.A = w.Qm = w.P = w.P_total = None

    # ------------------------------------------------------------------ pushed partial products

    @staticmethod
    def _ptr_table(cls: _PackedClass, key: tuple, make) -> Tensor:
        t = cls.ptr_cache.get(key)
        if t is None:
            if len(cls.ptr_cache) > 64:  # arenas were replaced: drop tables of buffers that no longer exist
                cls.ptr_cache.clear()
            t = cls.ptr_cache[key] = torch.tensor(make(), dtype=torch.int64, device=cls.M.device)
        return t

    def _p_pushed(self, w: "_ClassWork", first: ProcessGroup, second: Optional[ProcessGroup], B: int, a_loc: int,
                  r: int) -> Optional[Tensor]:
        """P = A Q summed over `first` (and then averaged over `second`) without a collective between the
        product and its consumer (the reduce-scatter / all-reduce of dion/dion.py:806-815, 925-929,
        1076-1079): the GEMM epilogue stores every tile of this rank's partial product into slot `rank` of
        a buffer in the memory of the rank(s) that need the sum, while the other tiles are still being
        multiplied; the next kernel announces that, waits for the other ranks' announcements, adds the
        slots in rank order and writes P together with the tf32 halves the Gram product needs.
        When the batch can be split (no tensor-parallel rows), matrix i goes only to rank i // per: every
        rank receives exactly the matrices it will orthonormalise.  Returns None (nothing launched) when
        the arenas cannot serve the buffers; sets w.P_total like the unfused path.

        Slot buffers sit at the same arena offsets in every step and no message says that a consumer has
        finished reading.  Rewriting them a step later is safe because every step passes through at least two
        synchronising operations on the arena (this exchange, then the R exchange or the all-reduce of the
        column sums): a rank that is about to push for step n + 1 has completed a consumer kernel that waited
        for its peers' announcements of the later operation of step n, which those peers launch behind their
        readers of this buffer (utils/protocol_check.py enumerates the interleavings)."""
        cls = w.cls
        dev = cls.M.device
        ar1 = symm.arena_for(first)
        ar2 = symm.arena_for(second) if second is not None else None
        mat = a_loc * r
        if mat % 4 != 0:
            return None
        if ar1 is None or (second is not None and ar2 is None):
            # an arena that does not exist yet is asked for, so that the next step can take this path
            nbytes = 8 * B * mat * 4
            symm.request(first, nbytes, dev)
            if second is not None:
                symm.request(second, nbytes, dev)
            return None
        W1 = ar1.world
        split = SHARD_WORK and w.inner is None and B > 1
        if not split and W1 > _MAX_PUSH_WORLD:
            return None
        per = (B + W1 - 1) // W1 if split else B
        cnt = max(0, min(per, B - ar1.rank * per)) if split else B
        push2 = ar2 is not None and ar2.world <= _MAX_PUSH_WORLD
        slots = ar1.alloc_slots((per, a_loc, r))
        slots2 = ar2.alloc_slots((per, a_loc, r)) if push2 else None
        if slots is None or (push2 and slots2 is None):
            return None
        if split:
            table = self._ptr_table(cls, ("p_split", ar1.peers[0], ar1.offset_of(slots), B, per, mat), lambda: [
                ar1.slot_address(i // per, slots, ar1.rank, (i % per) * mat) for i in range(B)])
            ops.gemm(w.A, w.Qm, out=slots[0, 0], out_ptrs=table)
            w.P_total = B
            self.p_reduce_scatters += 1
        else:
            table = self._ptr_table(cls, ("p_all", ar1.peers[0], ar1.offset_of(slots), B, mat), lambda: [
                ar1.slot_address(k, slots, ar1.rank, i * mat) for i in range(B) for k in range(W1)])
            ops.gemm(w.A, w.Qm, out=slots[0, 0], out_ptrs=table, out_dup=W1)
        scale1 = 1.0 if w.outer is not None else 1.0 / W1   # a sum over shards, a mean over replicas
        if ar2 is not None and not push2:
            # large replicate group: the first sum lands in its arena and the all-reduce kernel averages it
            share = symm.empty(second, (per, a_loc, r), torch.float32, dev)
            if cnt < per:
                share[cnt:].zero_()
            ops.slot_reduce(slots[:, :cnt], share[:cnt], None, None, [], scale1, ar1.wait_args())
            wait_fn = self._reduce(share, second, average=True)
            if wait_fn is not None:
                wait_fn()
            return share
        share = torch.empty((per, a_loc, r), dtype=torch.float32, device=dev)
        hi, lo = torch.empty_like(share), torch.empty_like(share)
        if cnt < per:  # shares are padded to equal size with zero matrices, which orthonormalise to zero
            for t in (share, hi, lo):
                t[cnt:].zero_()
        if push2:
            dests = [ar2.slot_address(q, slots2, ar2.rank) for q in range(ar2.world)]
            ops.slot_reduce(slots[:, :cnt], None, None, None, dests, scale1, ar1.wait_args())
            ops.slot_reduce(slots2[:, :cnt], share[:cnt], hi[:cnt], lo[:cnt], [], 1.0 / ar2.world, ar2.wait_args())
        else:
            ops.slot_reduce(slots[:, :cnt], share[:cnt], hi[:cnt], lo[:cnt], [], scale1, ar1.wait_args())
        register_split(share, hi, lo)
        return share

    def _r_pushed(self, w: "_ClassWork", first: ProcessGroup, second: Optional[ProcessGroup], B: int, n_loc: int,
                  r: int, Pm: Tensor):
        """R = A^T P pushed by the GEMM epilogue into slot `rank` of a buffer on every rank of `first`
        (the all-reduces of dion/dion.py:839-844, 951-960, 1098-1110).  With a `second` group (tensor
        parallel sum, then mean over the replicas) one reduction kernel adds the slots and hands the sum
        on to the slots of the second group.  Returns (slots, scale, wait arguments) for the kernel that
        consumes R, or None (nothing launched) when the arenas cannot serve the buffers."""
        cls = w.cls
        ar1 = symm.arena_for(first)
        ar2 = symm.arena_for(second) if second is not None else None
        mat = n_loc * r
        if mat % 4 != 0:
            return None
        if ar1 is None or (second is not None and ar2 is None):
            dev = cls.M.device
            symm.request(first, 8 * B * mat * 4, dev)
            if second is not None:
                symm.request(second, 8 * B * mat * 4, dev)
            return None
        if ar1.world > _MAX_PUSH_WORLD or (ar2 is not None and ar2.world > _MAX_PUSH_WORLD):
            return None
        slots = ar1.alloc_slots((B, n_loc, r))
        slots2 = ar2.alloc_slots((B, n_loc, r)) if ar2 is not None else None
        if slots is None or (ar2 is not None and slots2 is None):
            return None
        W1 = ar1.world
        table = self._ptr_table(cls, ("r_all", ar1.peers[0], ar1.offset_of(slots), B, mat), lambda: [
            ar1.slot_address(k, slots, ar1.rank, i * mat) for i in range(B) for k in range(W1)])
        ops.gemm(w.A.transpose(1, 2), Pm, out=slots[0, 0], out_ptrs=table, out_dup=W1)
        scale1 = 1.0 if w.inner is not None else 1.0 / W1
        if ar2 is None:
            return slots, scale1, ar1.wait_args()
        dests = [ar2.slot_address(q, slots2, ar2.rank) for q in range(ar2.world)]
        ops.slot_reduce(slots, None, None, None, dests, scale1, ar1.wait_args())
        return slots2, 1.0 / ar2.world, ar2.wait_args()

    def _apply_update(self, cls: _PackedClass, params: List[Tensor], X: List[Tensor], a_op: Tensor, b_op: Tensor,
                      alpha: float, beta: float) -> None:
        """X[i] = beta * X[i] + alpha * (a_op @ b_op)[i] for separately allocated X[i]."""
        x0 = X[0]
        fast = (x0.is_cuda and x0.dtype == torch.float32 and a_op.dtype in (torch.float32, torch.bfloat16)
                and all(x.is_contiguous() and x.data_ptr() % 16 == 0 for x in X)
                and (x0.shape[1] * 4) % 16 == 0)
        if fast:
            ptr_list = [x.data_ptr() for x in X]
            if cls.x_ptr_list != ptr_list:
                cls.x_ptr_list = ptr_list
                cls.x_ptrs = torch.tensor(ptr_list, dtype=torch.int64, device=x0.device)
            shadows = [nn_ops.shadow_for_update(p) for p in params]
            shadow0, shadow_ptrs = None, None
            if all(s is not None for s in shadows):
                sp_list = [s.data_ptr() for s in shadows]
                if cls.shadow_ptr_list != sp_list:
                    cls.shadow_ptr_list = sp_list
                    cls.shadow_ptrs = torch.tensor(sp_list, dtype=torch.int64, device=x0.device)
                shadow0, shadow_ptrs = shadows[0], cls.shadow_ptrs
            ops.gemm(a_op, b_op, c=x0, out=x0, c_ptrs=cls.x_ptrs, out_ptrs=cls.x_ptrs, shadow=shadow0,
                     shadow_ptrs=shadow_ptrs, alpha=alpha, beta=beta)
            for p in params:
                if shadow0 is not None:
                    nn_ops.mark_shadow_fresh(p)
                else:
                    nn_ops.mark_shadow_stale(p)
            return
        upd = torch.matmul(a_op.float(), b_op.float()) if not a_op.is_cuda else ops.gemm(a_op, b_op,
                                                                                        out_dtype=torch.float32)
        for i, x in enumerate(X):
            x.mul_(beta).add_(upd[i].to(x.dtype), alpha=alpha)

    # ------------------------------------------------------------------ scalar (AdamW / Lion) groups

    def _scalar_task(self, group: dict, algo: str) -> Generator[None, None, None]:
        params = [p for p in group["params"] if p.grad is not None]
        if not params:
            return
        states = [self._get_or_initialize_state(p, group) for p in params]
        X = to_local(params)
        G = to_local([p.grad for p in params])
        Ms = to_local([s["momentum"] for s in states])
        replicate = group_of(self._replicate_mesh) if self._replicate_mesh_grad_sync else None
        if replicate is not None and dist.get_world_size(replicate) > 1:
            wait = all_reduce_(G, replicate, average=True, async_op=True)
            yield
            wait()
        shadows = [nn_ops.shadow_for_update(p) for p in params]
        shadow_arg = shadows if all(s is not None for s in shadows) and X[0].is_cuda else None
        if algo == "adamw":
            Vs = to_local([s["variance"] for s in states])
            ops.adamw_update(X, G, Ms, Vs, lr=group["lr"], beta1=group["beta1"], beta2=group["beta2"],
                             weight_decay=group["weight_decay"], step=group["step"], epsilon=group["epsilon"],
                             shadow=shadow_arg)
        else:
            ops.lion_update(X, G, Ms, lr=group["lr"], beta1=group["beta1"], beta2=group["beta2"],
                            weight_decay=group["weight_decay"], shadow=shadow_arg)
        for p in params:
            if shadow_arg is not None:
                nn_ops.mark_shadow_fresh(p)
            else:
                nn_ops.mark_shadow_stale(p)

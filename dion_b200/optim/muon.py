"""Muon: momentum orthogonalised by Newton-Schulz, for single GPU, DDP, FSDP2 and HSDP.

Constructor, parameter-group keys, state layout (``momentum`` [+ ``variance``], fp32 like
the parameter) and update rule follow the reference's ``Muon`` (dion/muon.py:25-353 and
356-486).  Execution differs: all matrices of one (shape, placements, dtype) class are
handled together - one multi-tensor momentum kernel writing a packed bf16 buffer and the
squared norms, one exchange that gives every rank whole matrices, batched Newton-Schulz on
the tensor cores, one exchange back, one multi-tensor apply kernel.  Work is split over the
ranks of ``distributed_mesh`` by matrix, as in the reference, but without padding batches
to the world size with dummy matrices.
"""

from __future__ import annotations

import math
from typing import Callable, Dict, Generator, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor
from torch.optim.optimizer import Optimizer, ParamsT

from .. import ops
from ..ops import nn as nn_ops
from ..parallel import symm
from .common import Scheduler, to_local
from .newton_schulz import newton_schulz, newton_schulz_torch, zeropower_via_newtonschulz5  # noqa: F401


def adjust_lr_rms_norm(lr, param_shape):
    """Constant element-wise RMS (https://arxiv.org/abs/2502.16982): 0.2 sqrt(max(A, B))."""
    A, B = param_shape[-2:]
    return lr * 0.2 * math.sqrt(max(A, B))


def adjust_lr_spectral_norm(lr, param_shape):
    """Spectral norm 1 -> RMS operator norm 1 (https://arxiv.org/abs/2310.17813)."""
    fan_out, fan_in = param_shape[-2:]
    return lr * math.sqrt(fan_out / fan_in)


def adjust_lr_keller_muon(lr, param_shape):
    """sqrt(max(1, fan_out / fan_in)), the modded-nanogpt scaling."""
    fan_out, fan_in = param_shape[-2:]
    return lr * max(1, fan_out / fan_in) ** 0.5


_ADJUST = {None: lambda lr, shape: lr, "spectral_norm": adjust_lr_spectral_norm, "rms_norm": adjust_lr_rms_norm,
           "keller_muon": adjust_lr_keller_muon}


def _exchange(out: Tensor, inp: Tensor, group: ProcessGroup) -> None:
    """all_to_all_single with equal splits; backends without all-to-all (gloo) gather
    everything and keep their slice."""
    world = dist.get_world_size(group)
    try:
        dist.all_to_all_single(out, inp, group=group)
        return
    except (RuntimeError, NotImplementedError):
        pass
    gathered = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(gathered, inp.contiguous(), group=group)
    rank = dist.get_rank(group)
    chunk = inp.shape[0] // world
    for s in range(world):
        out[s * chunk:(s + 1) * chunk].copy_(gathered[s][rank * chunk:(rank + 1) * chunk])


class _ArenaTooSmall(Exception):
    """The symmetric arena cannot hold this step's exchange buffers yet."""


class Muon(Optimizer):
    """Distributed Muon (https://kellerjordan.github.io/posts/muon/).

    Args: ``distributed_mesh`` (1-D DeviceMesh for FSDP2 / HSDP sub-mesh, or ProcessGroup for
    DDP), ``lr`` (scaled per matrix according to ``adjust_lr``), ``mu``, ``betas`` (AdamW /
    Lion groups), ``weight_decay``, ``epsilon``, ``nesterov``, ``adjust_lr`` in
    {"spectral_norm", "rms_norm", "keller_muon", None}, ``flatten`` (3-D+ tensors become 2-D
    matrices instead of batches), ``use_triton`` (accepted for compatibility; the tcgen05
    Newton-Schulz is always used on CUDA unless ``newton_schulz_func`` is given),
    ``newton_schulz_func(input, epsilon) -> Tensor``.
    """

    def __init__(
        self,
        params: ParamsT,
        distributed_mesh: Optional[Union[DeviceMesh, ProcessGroup]] = None,
        lr: float = 0.01,
        mu: float = 0.95,
        betas: Tuple[float, float] = (0.9, 0.95),
        weight_decay: float = 0.01,
        epsilon: float = 1e-8,
        nesterov: bool = False,
        adjust_lr: Optional[str] = "spectral_norm",
        flatten: bool = False,
        use_triton: bool = False,
        newton_schulz_func: Optional[Callable] = None,
    ):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if mu < 0.0:
            raise ValueError(f"Invalid momentum factor (mu): {mu}")
        if len(betas) != 2 or betas[0] < 0.0 or betas[1] < 0.0:
            raise ValueError(f"Invalid betas: {betas}")
        if adjust_lr not in ("spectral_norm", "rms_norm", "keller_muon", None):
            raise ValueError(
                f"Invalid adjust_lr value: {adjust_lr}. Must be 'spectral_norm', 'rms_norm', 'keller_muon', or None.")
        defaults = dict(lr=lr, mu=mu, beta1=betas[0], beta2=betas[1], weight_decay=weight_decay, algorithm="muon",
                        step=0, epsilon=epsilon, nesterov=nesterov, flatten=flatten, adjust_lr=adjust_lr)
        super().__init__(params, defaults)

        if isinstance(distributed_mesh, DeviceMesh):
            if distributed_mesh.ndim != 1:
                raise ValueError(
                    f"Only 1D DeviceMesh is supported, but got {distributed_mesh.ndim}D. For HSDP, provide the 1D "
                    f"sharded sub-mesh.")
            self._device_rank = distributed_mesh.get_local_rank()
            self._world_size = distributed_mesh.size()
            self._process_group = distributed_mesh.get_group()
        elif isinstance(distributed_mesh, ProcessGroup):
            self._device_rank = dist.get_rank(distributed_mesh)
            self._world_size = dist.get_world_size(distributed_mesh)
            self._process_group = distributed_mesh
        elif distributed_mesh is None:
            self._device_rank, self._world_size, self._process_group = 0, 1, None
        else:
            raise TypeError(
                f"Invalid distributed_mesh type: {type(distributed_mesh)}. Expected DeviceMesh or ProcessGroup.")
        self._distributed_mesh = distributed_mesh

        if newton_schulz_func is not None:
            if not callable(newton_schulz_func):
                raise TypeError(f"newton_schulz_func must be a callable function, got {type(newton_schulz_func)}")
            self._newton_schulz_func = newton_schulz_func
            self._custom_ns = True
        else:
            self._newton_schulz_func = newton_schulz
            self._custom_ns = False
        self._use_triton = use_triton

    # ------------------------------------------------------------------ step

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        muon_groups, lion_groups, adamw_groups = [], [], []
        for group in self.param_groups:
            group["step"] += 1
            algo = group["algorithm"]
            if algo == "muon":
                muon_groups.append(group)
            elif algo == "lion":
                lion_groups.append(group)
            elif algo == "adamw":
                adamw_groups.append(group)
            else:
                raise ValueError(f"Unknown algorithm: {algo}")

        if muon_groups and self._process_group is not None and self._world_size > 1:
            first = next((p for g in muon_groups for p in g["params"] if p.grad is not None), None)
            if first is not None:
                symm.begin_step([self._process_group], to_local(first).device)

        def tasks():
            for group in muon_groups:
                yield from self._muon_tasks(group)
            for group in lion_groups:
                yield lambda g=group: self._scalar_task(g, "lion")
            for group in adamw_groups:
                yield lambda g=group: self._scalar_task(g, "adamw")

        Scheduler(tasks(), max_in_flight=3).run()
        return loss

    def _get_or_initialize_state(self, param: Tensor, algo: str) -> dict:
        state = self.state[param]
        if not state:
            state["momentum"] = torch.zeros_like(param)
            if algo == "adamw":
                state["variance"] = torch.zeros_like(param)
        return state

    # ------------------------------------------------------------------ Muon groups

    def _shard_info(self, p: Tensor) -> Optional[int]:
        """Tensor dim along which a DTensor parameter is sharded over the optimizer's mesh
        (None when unsharded); validation as in dion/muon.py:226-253."""
        if not isinstance(p, DTensor):
            return None
        if not isinstance(self._distributed_mesh, DeviceMesh):
            raise RuntimeError("Must create optimizer with DeviceMesh if using DTensor parameters.")
        shards = [(i, pl) for i, pl in enumerate(p.placements) if pl.is_shard() and p.device_mesh.size(i) > 1]
        if not shards:
            return None
        if len(shards) > 1:
            raise NotImplementedError("Muon does not support parameters with multiple sharded dimensions.")
        mesh_dim, placement = shards[0]
        if p.device_mesh.get_group(mesh_dim) != self._process_group:
            raise RuntimeError(
                f"Got DTensor sharded over mesh dimension {mesh_dim} different from the optimizer's device mesh")
        return placement.dim

    def _muon_tasks(self, group: dict):
        assert all(p.ndim >= 2 for p in group["params"]), "Muon optimizer only supports matrix parameters."
        params = [p for p in group["params"] if p.grad is not None]
        classes: Dict[tuple, List[Tensor]] = {}
        for p in params:
            placements = tuple(p.placements) if isinstance(p, DTensor) else None
            classes.setdefault((tuple(p.shape), placements, p.dtype), []).append(p)
        for members in classes.values():
            yield lambda ms=members: self._muon_update_class(ms, group)

    def _orthogonalize(self, U: Tensor, sumsq: Optional[Tensor], flatten: bool, epsilon: float) -> Tensor:
        """U: [k, *matrix_shape] bf16 -> orthogonalised, same shape (dion/muon.py:576-593)."""
        shape = U.shape
        X = U
        if flatten and X.dim() >= 4:
            X = X.flatten(start_dim=2)       # [k, d0, rest]
            sumsq_ok = True
        elif X.dim() >= 4:
            X = X.flatten(end_dim=-3)        # batches of 2-D matrices
            sumsq_ok = False
        else:
            sumsq_ok = True
        if self._custom_ns:
            out = torch.stack([self._newton_schulz_func(X[i], epsilon=epsilon) for i in range(X.shape[0])]) \
                if X.dim() == 3 and not sumsq_ok else self._newton_schulz_func(X, epsilon=epsilon)
        else:
            out = newton_schulz(X, epsilon, sumsq=sumsq if (sumsq_ok and sumsq is not None and X.is_cuda) else None)
        return out.reshape(shape)

    def _muon_update_class(self, params: List[Tensor], group: dict) -> Generator[None, None, None]:
        lr, mu, wd, eps = group["lr"], group["mu"], group["weight_decay"], group["epsilon"]
        nesterov, flatten, adjust = group["nesterov"], group["flatten"], group["adjust_lr"]
        states = [self._get_or_initialize_state(p, "muon") for p in params]
        X = to_local(params)
        G = to_local([p.grad for p in params])
        M = to_local([s["momentum"] for s in states])
        shard_dim = self._shard_info(params[0])
        W = self._world_size
        pg = self._process_group
        distributed = pg is not None and W > 1
        B = len(params)
        Bp = ((B + W - 1) // W) * W if distributed else B   # matrices, rounded up to a multiple of W
        per = Bp // W if distributed else B                   # matrices owned by each rank
        local_shape = X[0].shape

        if distributed and shard_dim is not None and params[0].size(shard_dim) % W != 0:
            raise AssertionError(
                f"Shard dimension {shard_dim} size {params[0].size(shard_dim)} is not divisible by world size {W}.")
        if distributed and shard_dim is not None and self._fused_exchange_ok(params[0], X[0], shard_dim):
            # shards travel by peer stores issued from the momentum kernel and from the epilogue of
            # the last Newton-Schulz product; see _muon_update_class_fused (which gives up, before
            # it touches the momentum, when the arena cannot hold its buffers yet)
            try:
                self._muon_update_class_fused(params, X, G, M, group, shard_dim, per, Bp)
                return
            except _ArenaTooSmall:
                pass  # the arena grows at the next step; this step uses the library collectives

        # momentum, Nesterov, bf16 cast and squared norms in one launch (dion/muon.py:525-552)
        U = torch.zeros((Bp, *local_shape), dtype=torch.bfloat16, device=X[0].device) if Bp != B else \
            torch.empty((Bp, *local_shape), dtype=torch.bfloat16, device=X[0].device)
        use_sumsq = X[0].is_cuda and not self._custom_ns and M[0].dtype == torch.float32
        sumsq = torch.zeros(Bp, dtype=torch.float32, device=X[0].device) if use_sumsq else None
        ops.muon_momentum(G, M, mu=mu, nesterov=nesterov, U=list(U[:B].unbind(0)), sumsq=sumsq)

        if distributed and shard_dim is not None:
            # shards of the matrices a rank owns travel to it: [W, per, *local] by source rank
            if sumsq is not None:
                work_n = dist.all_reduce(sumsq, group=pg, async_op=True)
            recv = torch.empty_like(U)
            _exchange(recv, U, pg)
            yield
            if sumsq is not None:
                work_n.wait()
            recv = recv.view(W, per, *local_shape)
            d = shard_dim + 2
            order = list(range(recv.dim()))
            order.remove(0)
            order.insert(d - 1, 0)          # source-rank axis moves right before the sharded dim
            whole = recv.permute(order).reshape(per, *params[0].shape)
            mine = sumsq[self._device_rank * per:(self._device_rank + 1) * per] if sumsq is not None else None
            ortho = self._orthogonalize(whole, mine, flatten, eps)
            # back: split along the sharded dim by destination rank
            parts = ortho.reshape(per, *params[0].shape[:shard_dim], W, local_shape[shard_dim],
                                  *params[0].shape[shard_dim + 1:])
            send = parts.movedim(shard_dim + 1, 0).contiguous().view(Bp, *local_shape)
            _exchange(U, send, pg)
            yield
        elif distributed:
            lo = self._device_rank * per
            mine = sumsq[lo:lo + per] if sumsq is not None else None
            ortho = self._orthogonalize(U[lo:lo + per], mine, flatten, eps)
            gather = self._symm_gather(ortho.device)
            if gather is not None:
                # all-gather kernel over symmetric memory (falls back to the group's own by itself)
                gather(U.view(-1), ortho.contiguous().view(-1), pg)
                yield
            else:
                work = dist.all_gather_into_tensor(U, ortho.contiguous(), group=pg, async_op=True)
                yield
                work.wait()
        else:
            U = self._orthogonalize(U, sumsq, flatten, eps)

        adjusted_lr = _ADJUST[adjust](lr, params[0].shape)
        shadows = [nn_ops.shadow_for_update(p) for p in params]
        shadow_arg = shadows if all(s is not None for s in shadows) and X[0].is_cuda else None
        ops.muon_apply(X, list(U[:B].unbind(0)), decay=1.0 - lr * wd, step=adjusted_lr, shadow=shadow_arg)
        for p in params:
            if shadow_arg is not None:
                nn_ops.mark_shadow_fresh(p)
            else:
                nn_ops.mark_shadow_stale(p)

    def _fused_exchange_ok(self, p: Tensor, x_local: Tensor, shard_dim: int) -> bool:
        if self._custom_ns or not x_local.is_cuda or x_local.dim() != 2 or x_local.dtype != torch.float32:
            return False
        arena = symm.arena_for(self._process_group)
        if arena is None:
            return False
        # column blocks must be whole 32-column chunks of the epilogue; pitches 16-byte aligned
        if shard_dim == 1 and x_local.shape[1] % 32 != 0:
            return False
        return (x_local.shape[1] * 2) % 16 == 0

    def _muon_update_class_fused(self, params, X, G, M, group, shard_dim: int, per: int, Bp: int) -> None:
        """Sharded Muon update whose two all-to-alls are peer stores issued by the kernels that
        produce the data (dion/muon.py:404-435 does them as NCCL all_to_all calls):
          1. the momentum kernel writes every bf16 shard directly into the receive buffer of the
             rank that owns the matrix;
          2. after a flag barrier the owner runs Newton-Schulz on its whole matrices;
          3. the epilogue of the last product stores each row/column block of the result into the
             update buffer of the rank that holds that shard;
          4. after a second barrier every rank applies its shards."""
        lr, mu, wd, eps = group["lr"], group["mu"], group["weight_decay"], group["epsilon"]
        W, rank, pg = self._world_size, self._device_rank, self._process_group
        arena = symm.arena_for(pg)
        B = len(params)
        local_shape = tuple(X[0].shape)
        full_shape = tuple(params[0].shape)
        dev = X[0].device
        recv = symm.empty(pg, (per, W, *local_shape), torch.bfloat16, dev)   # [owned matrix, source rank]
        upd = symm.empty(pg, (Bp, *local_shape), torch.bfloat16, dev)        # [matrix of the class]
        if arena.offset_of(recv) is None or arena.offset_of(upd) is None:
            raise _ArenaTooSmall()
        # 1. momentum + Nesterov + bf16 cast, stored into the owners' receive buffers
        peer_recv = [arena.peer_view(d, recv) for d in range(W)]
        U = [peer_recv[i // per][i % per, rank] for i in range(B)]
        ops.muon_momentum(G, M, mu=mu, nesterov=group["nesterov"], U=U, sumsq=None)
        arena.barrier()
        # 2./3. Newton-Schulz on the matrices this rank owns, result scattered to the shard holders
        cnt = max(0, min(per, B - rank * per))
        if cnt > 0:
            if shard_dim == 0:
                whole = recv[:cnt].reshape(cnt, *full_shape)                  # row blocks are already in place
                mode, block = 1, local_shape[0]
            else:
                whole = recv[:cnt].permute(0, 2, 1, 3).reshape(cnt, *full_shape)
                mode, block = 2, local_shape[1]
            shard_bytes = X[0].numel() * 2
            key = (arena.peers[0], arena.offset_of(upd), cnt, per, rank)
            cache = getattr(self, "_scatter_cache", None)
            if cache is None:
                cache = self._scatter_cache = {}
            ptrs = cache.get(key)
            if ptrs is None:
                addr = [[arena.peer_address(s, upd) + (rank * per + j) * shard_bytes for s in range(W)]
                        for j in range(cnt)]
                ptrs = cache[key] = torch.tensor(addr, dtype=torch.int64, device=dev).view(-1)
            newton_schulz(whole, eps, scatter=dict(ptrs=ptrs, mode=mode, block=block, dests=W, block_like=upd[0]))
        arena.barrier()
        # 4. apply
        adjusted_lr = _ADJUST[group["adjust_lr"]](lr, params[0].shape)
        shadows = [nn_ops.shadow_for_update(p) for p in params]
        shadow_arg = shadows if all(s is not None for s in shadows) else None
        ops.muon_apply(X, list(upd[:B].unbind(0)), decay=1.0 - lr * wd, step=adjusted_lr, shadow=shadow_arg)
        for p in params:
            if shadow_arg is not None:
                nn_ops.mark_shadow_fresh(p)
            else:
                nn_ops.mark_shadow_stale(p)

    def _symm_gather(self, device):
        """All-gather object for the unsharded path (updates computed by their owners are
        distributed to every rank), or None where symmetric memory does not apply."""
        if device.type != "cuda" or self._process_group is None:
            return None
        g = getattr(self, "_gather_obj", None)
        if g is None:
            from ..parallel.fsdp_comm import SymmAllGather, _usable

            if not _usable(self._process_group, device):
                return None
            g = self._gather_obj = SymmAllGather(self._process_group, device)
        return g

    # ------------------------------------------------------------------ scalar groups

    def _scalar_task(self, group: dict, algo: str) -> Generator[None, None, None]:
        params = [p for p in group["params"] if p.grad is not None]
        if not params:
            return
        states = [self._get_or_initialize_state(p, algo) for p in params]
        X = to_local(params)
        G = to_local([p.grad for p in params])
        Ms = to_local([s["momentum"] for s in states])
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
        return
        yield  # pragma: no cover - makes this a generator

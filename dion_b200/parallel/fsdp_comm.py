"""FSDP2 collectives as in-tree kernels over symmetric memory.

FSDP2 (``torch.distributed.fsdp.fully_shard``) lets a module replace the two collectives it
issues - the all-gather of parameter shards before a block runs and the reduce-scatter of
its gradients afterwards (the reference gets both from NCCL, models/gpt_model.py:336-376) -
through ``FSDPModule.set_custom_all_gather`` / ``set_custom_reduce_scatter``.  The objects
here plug into those hooks:

* :class:`SymmAllGather` - every rank copies its shard into a double-buffered symmetric
  staging slot and pulls the peers' slots over NVLink straight into the (ordinary)
  all-gather output, all in one kernel; no closing barrier, the slot parity protects reuse.
* :class:`SymmReduceScatter` - ``allocate`` hands FSDP a symmetric buffer for the
  reduce-scatter *input* (FSDP copies the unsharded gradients into it), and the kernel has
  every rank sum its slice over all peers (peer loads in rank order, or ``multimem.ld_reduce``
  in the switch) with the ``1/world`` factor fused, writing an ordinary output buffer that FSDP
  keeps as the sharded gradient.

Anything the kernels do not cover (CPU tensors, gloo, more than eight ranks, dtypes other
than fp32 / bf16, unaligned sizes, ``async_op=True``, exotic reduce ops) goes to the process
group's own collective, so the objects are safe to install unconditionally.

:func:`install` walks a model and installs one pair of objects per shard process group.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

try:  # the hooks exist from torch 2.8 on
    from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter
except Exception:  # pragma: no cover
    AllGather = ReduceScatter = object  # type: ignore[assignment,misc]

from ..ops import runtime
from . import symm

# channels of the arena's flag block used here (the optimizer's kernels use 0-3 of *their* arenas;
# these arenas are separate objects, the numbers only have to differ within one arena)
_CH_AG = 0
_CH_RS_START = 1
_CH_RS_END = 2
# A rank may reach a collective long after its peers (data loading, logging, a checkpoint);
# the wait stays bounded, but generously.
_WAIT_NS = int(float(os.environ.get("DION_B200_FSDP_WAIT_S", "30")) * 1e9)
_MIN_BYTES = 1 << 20


def _is_cuda(device) -> bool:
    return torch.device(device).type == "cuda"


def _kernel_dtype(dtype: torch.dtype) -> bool:
    return dtype in (torch.float32, torch.bfloat16)


class _Arena:
    """A symmetric arena with two equal slots, recreated (collectively) when a request outgrows it."""

    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        self.group, self.device = group, device
        self.arena: Optional[symm.SymmetricArena] = None
        self.slot_bytes = 0
        self.calls = 0
        self.declined = False

    def ensure(self, nbytes: int) -> bool:
        """True when a slot of `nbytes` is available.  `nbytes` is the size of a collective's
        per-rank input, which FSDP pads to the same value on every rank, so all ranks of the group
        take the same branch here; the creation itself agrees on size and success across the group
        (:func:`symm.create_arena`), and a group that could not create its arena stays on the
        library collectives on every rank."""
        if self.declined:
            return False
        if self.arena is not None and nbytes <= self.slot_bytes:
            return True
        if self.arena is not None:
            # kernels of every rank that still use the old arena must have retired
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        slot = max(_MIN_BYTES, int(nbytes * 1.25))
        slot = (slot + 255) // 256 * 256
        self.arena = symm.create_arena(self.group, 2 * slot, self.device)
        if self.arena is None:
            self.declined = True
            self.slot_bytes = 0
            if dist.get_rank() == 0:
                print("[dion_b200] symmetric memory unavailable for FSDP collectives; using the library's")
            return False
        self.slot_bytes = self.arena.capacity // 2 // 256 * 256
        self.calls = 0
        return True

    def slot_offset(self, index: int) -> int:
        """Byte offset of slot `index` from the arena base (flag block included)."""
        return symm._FLAG_BYTES + index * self.slot_bytes


def _usable(group: dist.ProcessGroup, device: torch.device) -> bool:
    return symm._usable(group, torch.device(device))


class SymmAllGather(AllGather):
    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        self.device = torch.device(device)
        self._slots = _Arena(group, self.device) if _usable(group, self.device) else None
        self.kernel_calls = 0
        self.fallback_calls = 0

    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.empty(tuple(size), dtype=dtype, device=device)

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup,
                 async_op: bool = False):
        a = self._slots
        nbytes = input_tensor.numel() * input_tensor.element_size()
        ok = (a is not None and not async_op and input_tensor.is_cuda and symm._key(group) == symm._key(a.group)
              and input_tensor.is_contiguous() and output_tensor.is_contiguous()
              and nbytes % 16 == 0 and input_tensor.data_ptr() % 16 == 0 and output_tensor.data_ptr() % 16 == 0
              and output_tensor.numel() == input_tensor.numel() * dist.get_world_size(group)
              and nbytes > 0 and a.ensure(nbytes))
        if not ok:
            self.fallback_calls += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)
        ar = a.arena
        ar.epoch += 1
        torch.ops.dion_b200.symm_all_gather(input_tensor, output_tensor, ar.peers, 0, a.slot_offset(ar.epoch & 1),
                                            ar.rank, ar.epoch, _CH_AG, ar.counter,
                                            runtime.status_tensor(self.device), _WAIT_NS)
        self.kernel_calls += 1
        return None


class SymmReduceScatter(ReduceScatter):
    def __init__(self, group: dist.ProcessGroup, device: torch.device):
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self._slots = _Arena(group, self.device) if _usable(group, self.device) else None
        self._next = 0
        self._events: List[Optional[torch.cuda.Event]] = [None, None]
        self._live: Dict[int, Tuple[int, int]] = {}  # data_ptr -> (slot index, arena generation)
        self._pending_numel: Optional[int] = None
        self._generation = 0
        self.kernel_calls = 0
        self.fallback_calls = 0

    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        n = 1
        for s in size:
            n *= int(s)
        a = self._slots
        # FSDP asks for the input (world * n elements) and then for the output (n elements) of each
        # reduce-scatter; only the input has to be symmetric, the output becomes the sharded gradient
        # and must outlive the call.
        if self._pending_numel is not None and n * self.world == self._pending_numel:
            self._pending_numel = None
            return torch.empty(tuple(size), dtype=dtype, device=device)
        self._pending_numel = None
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if (a is None or not _kernel_dtype(dtype) or not _is_cuda(device) or n == 0
                or n % self.world != 0 or (nbytes // self.world) % 16 != 0):
            return torch.empty(tuple(size), dtype=dtype, device=device)
        had = a.arena
        if not a.ensure(nbytes):
            return torch.empty(tuple(size), dtype=dtype, device=device)
        if a.arena is not had:
            self._generation += 1
            self._events = [None, None]
            self._live.clear()
        idx = self._next
        self._next ^= 1
        ev = self._events[idx]
        if ev is not None:
            # the kernel that last read this slot (on the reduce-scatter stream) must have retired
            torch.cuda.current_stream(self.device).wait_event(ev)
        off = a.slot_offset(idx)
        t = a.arena.buf[off:off + nbytes].view(dtype).view(tuple(size))
        self._live[t.data_ptr()] = (idx, self._generation)
        self._pending_numel = n
        return t

    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: dist.ProcessGroup,
                 op, async_op: bool = False):
        a = self._slots
        slot = self._live.get(input_tensor.data_ptr()) if a is not None else None
        scale = None
        if op == dist.ReduceOp.SUM:
            scale = 1.0
        elif op == dist.ReduceOp.AVG:
            scale = 1.0 / self.world
        ok = (slot is not None and slot[1] == self._generation and scale is not None and not async_op
              and symm._key(group) == symm._key(a.group) and input_tensor.is_contiguous() and output_tensor.is_contiguous()
              and output_tensor.dtype == input_tensor.dtype and output_tensor.data_ptr() % 16 == 0
              and input_tensor.numel() == output_tensor.numel() * self.world)
        if not ok:
            self.fallback_calls += 1
            return dist.reduce_scatter_tensor(output_tensor, input_tensor, op=op, group=group, async_op=async_op)
        ar = a.arena
        ar.epoch += 1
        torch.ops.dion_b200.symm_reduce_scatter(input_tensor, output_tensor, ar.peers, 0, a.slot_offset(slot[0]),
                                                ar.mc_base, scale, ar.rank, ar.epoch, _CH_RS_START, _CH_RS_END,
                                                ar.counter, runtime.status_tensor(self.device), _WAIT_NS)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._events[slot[0]] = ev
        self.kernel_calls += 1
        return None


_installed: Dict[str, Tuple[SymmAllGather, SymmReduceScatter]] = {}


def install(model: torch.nn.Module) -> int:
    """Give every FSDP2-wrapped module of `model` the collectives above (one pair of objects per
    shard process group, shared by all modules that use the group).  Returns how many modules
    were switched.  ``DION_B200_FSDP_COMM=0`` leaves FSDP on the library collectives."""
    if os.environ.get("DION_B200_FSDP_COMM", "1") == "0":
        return 0
    try:
        from torch.distributed.fsdp import FSDPModule
    except Exception:  # pragma: no cover
        return 0
    n = 0
    for m in model.modules():
        if not isinstance(m, FSDPModule) or not hasattr(m, "set_custom_all_gather"):
            continue
        pg_state = m._get_fsdp_state()._fsdp_param_group
        if pg_state is None:
            continue
        group = pg_state.mesh_info.shard_process_group
        device = pg_state.device
        if not _usable(group, device):
            continue
        key = symm._key(group)
        if key not in _installed:
            _installed[key] = (SymmAllGather(group, device), SymmReduceScatter(group, device))
        ag, rs = _installed[key]
        m.set_custom_all_gather(ag)
        m.set_custom_reduce_scatter(rs)
        n += 1
    return n

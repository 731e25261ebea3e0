"""Helpers shared by the optimizers: local/DTensor conversion, process-group access for
DeviceMesh or ProcessGroup arguments, averaged all-reduce of tensor lists, batching of
same-shape parameters, and a small cooperative scheduler for overlapping collectives.

Behavioural reference: dion/opt_utils.py:8-145 and dion/dion.py:1165-1197.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Dict, Generator, Iterable, Iterator, List, Optional, Sequence, Union

import torch
import torch.distributed as dist
from torch import Tensor
from torch.distributed import ProcessGroup
from torch.distributed.tensor import DeviceMesh, DTensor

MeshOrGroup = Union[DeviceMesh, ProcessGroup, None]


def to_local(t):
    """Local shard of a DTensor (or of every DTensor in a list); plain tensors pass through."""
    if isinstance(t, Tensor):
        return t.to_local() if isinstance(t, DTensor) else t
    return [x.to_local() if isinstance(x, DTensor) else x for x in t]


def like_dtensor(local, ref: Tensor):
    """Wrap local tensor(s) as DTensor(s) with the mesh and placements of `ref`; a plain
    `ref` returns the input unchanged."""
    if not isinstance(ref, DTensor):
        return local
    if isinstance(local, Tensor):
        return DTensor.from_local(local, device_mesh=ref.device_mesh, placements=ref.placements, run_check=False)
    return [DTensor.from_local(x, device_mesh=ref.device_mesh, placements=ref.placements, run_check=False)
            for x in local]


def group_of(mesh: MeshOrGroup) -> Optional[ProcessGroup]:
    """The process group behind a 1-D DeviceMesh / ProcessGroup / None."""
    if mesh is None:
        return None
    if isinstance(mesh, DeviceMesh):
        if mesh.ndim != 1:
            raise ValueError(f"expected a 1-D DeviceMesh, got {mesh.ndim}-D")
        return mesh.get_group()
    if isinstance(mesh, ProcessGroup):
        return mesh
    raise TypeError(f"expected DeviceMesh, ProcessGroup or None, got {type(mesh)}")


def group_size(mesh: MeshOrGroup) -> int:
    if mesh is None:
        return 1
    if isinstance(mesh, DeviceMesh):
        return mesh.size()
    return dist.get_world_size(mesh)


def group_rank(mesh: MeshOrGroup) -> int:
    if mesh is None:
        return 0
    if isinstance(mesh, DeviceMesh):
        return mesh.get_local_rank() if mesh.ndim == 1 else mesh.get_rank()
    return dist.get_rank(mesh)


def _supports_avg(group: ProcessGroup) -> bool:
    try:
        return dist.get_backend(group) == "nccl"
    except Exception:  # pragma: no cover
        return False


def all_reduce_(tensors: Union[Tensor, Sequence[Tensor]], group: Optional[ProcessGroup], average: bool,
                async_op: bool = False):
    """In-place all-reduce (sum or mean) of one tensor or a list of tensors over `group`.

    Lists are reduced with as few collectives as possible: same-dtype tensors are
    flattened into one bucket.  With `async_op` a zero-argument `wait()` callable is
    returned that finishes the operation (copies back / divides)."""
    if group is None or dist.get_world_size(group) == 1:
        return (lambda: None) if async_op else None
    single = isinstance(tensors, Tensor)
    ts: List[Tensor] = [tensors] if single else [t for t in tensors]
    ts = [to_local(t) for t in ts]
    world = dist.get_world_size(group)
    op = dist.ReduceOp.AVG if (average and _supports_avg(group)) else dist.ReduceOp.SUM
    post_div = average and op == dist.ReduceOp.SUM

    by_dtype: Dict[torch.dtype, List[Tensor]] = OrderedDict()
    for t in ts:
        by_dtype.setdefault(t.dtype, []).append(t)
    pending = []
    for dtype, lst in by_dtype.items():
        if len(lst) == 1 and lst[0].is_contiguous():
            work = dist.all_reduce(lst[0], op=op, group=group, async_op=True)
            pending.append((work, None, lst))
        else:
            flat = torch.cat([t.reshape(-1) for t in lst])
            work = dist.all_reduce(flat, op=op, group=group, async_op=True)
            pending.append((work, flat, lst))

    def wait():
        for work, flat, lst in pending:
            work.wait()
            if flat is not None:
                if post_div:
                    flat.div_(world)
                off = 0
                for t in lst:
                    n = t.numel()
                    t.copy_(flat[off:off + n].view_as(t))
                    off += n
            elif post_div:
                lst[0].div_(world)

    if async_op:
        return wait
    wait()
    return None


def batches_by_shape(params: Iterable[Tensor], max_batch: Optional[int] = None) -> Iterator[List[Tensor]]:
    """Group parameters that share (shape, placements, dtype) - the unit one batched kernel
    sequence works on - optionally chunked to at most `max_batch` members
    (dion/opt_utils.py:48-65)."""
    groups: Dict[tuple, List[Tensor]] = OrderedDict()
    for p in params:
        placements = tuple(p.placements) if isinstance(p, DTensor) else None
        groups.setdefault((tuple(p.shape), placements, p.dtype), []).append(p)
    for members in groups.values():
        if max_batch is None:
            yield members
        else:
            for i in range(0, len(members), max_batch):
                yield members[i:i + max_batch]


class Task:
    """A generator-based unit of work that yields whenever it has launched an asynchronous
    collective and has nothing else to do until it finishes."""

    def __init__(self, gen: Generator[None, None, None]):
        self._gen = gen
        self.done = False
        self.advance()

    def advance(self) -> bool:
        if self.done:
            return False
        try:
            next(self._gen)
            return True
        except StopIteration:
            self.done = True
            return False

    run = advance  # the reference's name for the same step (AsyncTask.run, dion/opt_utils.py:89-98)


class Scheduler:
    """Round-robin scheduler over lazily created tasks: at most `max_in_flight` tasks are
    alive; each turn admits one new task and advances every live one by one step, so the
    collectives of one batch overlap the math of the others (dion/opt_utils.py:100-145)."""

    def __init__(self, tasks: Iterable[Union["Task", Callable[[], Generator[None, None, None]]]], max_in_flight: int = 3):
        if max_in_flight <= 0:
            raise ValueError(f"max_in_flight={max_in_flight} must be positive")
        self._source = iter(tasks)
        self._max = max_in_flight

    def run(self) -> None:
        live: List[Task] = []
        exhausted = False
        while live or not exhausted:
            nxt: List[Task] = []
            if not exhausted and len(live) < self._max:
                try:
                    make = next(self._source)
                    t = make if isinstance(make, Task) else Task(make())  # a started task or a factory of one
                    if not t.done:
                        nxt.append(t)
                except StopIteration:
                    exhausted = True
            for t in live:
                if t.advance():
                    nxt.append(t)
            live = nxt

"""The reference's ``dion.opt_utils`` under its own names (dion/opt_utils.py:8-145): DTensor <-> local
conversion, batching of same-shape parameters and the cooperative task runtime.  The implementations live in
:mod:`dion_b200.optim.common`; this module is the import path a user of the reference expects."""

from __future__ import annotations

from typing import Generator, Iterable, List

import torch
from torch import Tensor

from .optim.common import Scheduler, Task, batches_by_shape, like_dtensor, to_local  # noqa: F401

dtensor_from_local = like_dtensor
AsyncTask = Task


def create_param_batches(params: Iterable[Tensor], batch_size: int) -> Generator[List[Tensor], None, None]:
    """Lists of at most ``batch_size`` parameters that share shape, sharding and dtype
    (dion/opt_utils.py:48-65)."""
    yield from batches_by_shape(params, batch_size)


def pad_batch(batch: List[Tensor], batch_size: int) -> List[Tensor]:
    """Append uninitialised tensors shaped like the first member until the batch has ``batch_size`` members
    (dion/opt_utils.py:68-76); modifies and returns ``batch``."""
    if not 0 < len(batch) <= batch_size:
        raise ValueError(f"a batch of {len(batch)} cannot be padded to {batch_size}")
    while len(batch) < batch_size:
        batch.append(torch.empty_like(batch[0]))
    return batch


class AsyncRuntime(Scheduler):
    """Event loop over a generator of started :class:`AsyncTask` objects with at most
    ``max_concurrent_tasks`` alive: every turn admits one new task and advances each live one to its next
    ``yield`` (dion/opt_utils.py:100-145)."""

    def __init__(self, task_gen: Iterable[Task], max_concurrent_tasks: int):
        if max_concurrent_tasks <= 0:
            raise ValueError(f"{max_concurrent_tasks=} cannot be <= 0")
        super().__init__(task_gen, max_in_flight=max_concurrent_tasks)

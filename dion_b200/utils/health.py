"""Host-side liveness of the ranks of a job, through the process group's key-value store.

A collective (NCCL's or an in-tree kernel's) that a peer never joins can only end in a timeout.
The cheap way to avoid launching it is to know, on the host and between steps, that the peer is
gone: every rank publishes the last step it finished (and says so when it leaves on purpose), and
checks the others before it launches the next step.  Nothing here touches a GPU; the reference
has no counterpart (a rank that disappears hangs its job, train.py:246-282 only checks the
environment at start-up).

    hb = StepHeartbeat.from_default_group()
    for step in ...:
        hb.check(step)          # raises RankFailure before anything is launched
        train_step()
        hb.beat(step)
    hb.leave()
"""

from __future__ import annotations

import time
from typing import List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    """Some ranks left or stopped making progress; `.ranks` lists them."""

    def __init__(self, message: str, ranks: List[int]):
        super().__init__(message)
        self.ranks = ranks


class StepHeartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "dion_b200/heartbeat", max_lag: int = 50,
                 stale_after_s: float = 300.0, check_every: int = 1):
        """`max_lag`: how many steps a peer may trail before it is looked at; `stale_after_s`: how old
        its last beat must be before a trailing peer counts as failed; `check_every`: look at the peers
        only every so many steps (one store read per peer)."""
        self.store, self.rank, self.world = store, rank, world
        self.prefix, self.max_lag, self.stale_after_s, self.check_every = prefix, max_lag, stale_after_s, check_every
        self._key = lambda r: f"{self.prefix}/{r}"
        self.beat(-1)

    @classmethod
    def from_default_group(cls, **kw) -> Optional["StepHeartbeat"]:
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return None
        from torch.distributed.distributed_c10d import _get_default_store

        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), **kw)

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def leave(self) -> None:
        """Announce an orderly departure (between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), "left")

    def _read(self, r: int):
        try:
            if not self.store.check([self._key(r)]):
                return None
            raw = self.store.get(self._key(r)).decode()
        except Exception:
            return None
        if raw == "left":
            return "left"
        step, stamp = raw.split(":")
        return int(step), float(stamp)

    def check(self, step: int) -> None:
        """Raise RankFailure if a peer has left, or trails by more than `max_lag` steps with a beat
        older than `stale_after_s`."""
        if self.check_every > 1 and step % self.check_every != 0:
            return
        gone, now = [], time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == "left":
                gone.append(r)
            elif v is not None:
                peer_step, stamp = v
                if step - peer_step > self.max_lag and now - stamp > self.stale_after_s:
                    gone.append(r)
        if gone:
            raise RankFailure(f"rank {self.rank}: ranks {gone} left or stopped before step {step}; "
                              "not launching the step", gone)

"""CUDA-event phase timers (the reference times its loop with ``time.time()`` around a device
synchronisation, train.py:825-841).  Phases are bracketed by events recorded on the current
stream, so measuring adds no synchronisation; `summary()` synchronises once, and
`max_over_ranks()` reduces with MAX so that multi-GPU numbers are the slowest rank's."""

from __future__ import annotations

from collections import defaultdict
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


class PhaseTimers:
    def __init__(self, enabled: bool = True, nvtx: bool = False):
        self.enabled = enabled and torch.cuda.is_available()
        # NVTX ranges around the same phases, for timeline tools; off by default
        self.nvtx = nvtx and torch.cuda.is_available()
        self._open: Dict[str, torch.cuda.Event] = {}
        self._pairs: Dict[str, List[Tuple[torch.cuda.Event, torch.cuda.Event]]] = defaultdict(list)

    def start(self, name: str) -> None:
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if not self.enabled:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[name] = ev

    def stop(self, name: str) -> None:
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        if not self.enabled:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._pairs[name].append((self._open.pop(name), ev))

    def reset(self) -> None:
        self._open.clear()
        self._pairs.clear()

    def summary(self) -> Dict[str, float]:
        """Mean milliseconds per occurrence of every phase."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in self._pairs.items()}

    def max_over_ranks(self) -> Dict[str, float]:
        s = self.summary()
        if not s or not dist.is_initialized() or dist.get_world_size() == 1:
            return s
        keys = sorted(s)
        t = torch.tensor([s[k] for k in keys], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return dict(zip(keys, t.tolist()))


def cuda_time_ms(fn, iters: int = 10, warmup: int = 3, flush_l2: bool = False) -> float:
    """Mean device time of `fn()` over `iters` calls, events on the current stream."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters

"""Symmetric-memory arenas and the collectives that run on them (the transport under the averaged
all-reduces of the reference's optimizers: ``all_reduce_replicate_mesh``, dion/dion.py:1165-1197, and
the funcol / DTensor redistributions around the power iteration, dion/dion.py:806-844, 925-960).

One arena per process group: a symmetric allocation (same size on every rank, peers mapped
over NVLink, optionally bound to an NVSwitch multicast object) with a flag block in front.
Buffers handed out by :func:`empty` are views into the arena; :func:`all_reduce` on such a
view runs the in-tree all-reduce kernel (peer loads / stores or ``multimem`` instructions
issued by the kernel itself), anything else falls back to the process group's own
collective (NCCL on GPUs, gloo on CPUs), so call sites do not care which path is taken.

Sizing is lazy and symmetric: a step that needs more than the arena holds is served from
ordinary memory (library collectives) and the arena grows at the next :func:`begin_step`,
which every rank reaches with the same request history.

Environment: ``DION_B200_SYMM=0`` disables the arenas, ``DION_B200_MULTICAST=0`` keeps the
kernels on plain peer loads and stores.
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import runtime

_FLAG_BYTES = 4096
_WANT_OFF = 2048  # inside the flag block, far behind the flag words: one fp32 per rank, see post_want()
_ALIGN = 256
_MIN_ARENA = 8 << 20
_RS_WAIT_NS = int(1.5e9)  # bound of the reduce-scatter kernel's waits for its peers
# Debug mode (DION_B200_DEBUG=1, which also selects the kernels' debug build): every buffer handed out by an
# arena is followed by a guard of _CANARY_BYTES filled with a pattern; begin_step() checks all guards of the
# step that just ended (a host synchronisation, hence debug only).  A damaged guard means that some kernel -
# of this rank or, since peers store into this memory, of another one - wrote past the end of a buffer.
_DEBUG = os.environ.get("DION_B200_DEBUG", "0") == "1"
_CANARY_BYTES = 256
_CANARY = 0xA5
_CH_SLOT = 4               # flag channel of the push exchanges (0-3: all-reduce, reduce-into, reduce-scatter)
_SLOT_WAIT_NS = int(1.5e9)

# How often each kind of collective ran as an in-tree kernel and how often it went to the process group's
# own implementation since the last reset_stats(); benchmarks report it next to their timings.
stats: Dict[str, int] = {}


def count(kind: str, kernel: bool) -> None:
    k = f"{kind}.{'kernel' if kernel else 'library'}"
    stats[k] = stats.get(k, 0) + 1


def reset_stats() -> None:
    stats.clear()


def _enabled() -> bool:
    return os.environ.get("DION_B200_SYMM", "1") != "0"


class SymmetricArena:
    """Creating one is collective over `group` (rendezvous + barrier) and must be given the same
    `nbytes` on every rank: use :func:`create_arena`, which agrees on both the size and on whether
    every rank could allocate, unless the caller has that agreement by other means."""

    def __init__(self, group: dist.ProcessGroup, nbytes: int, device: torch.device, buf: Optional[torch.Tensor] = None):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import _ext

        _ext.load(required=True)
        self.group = group
        self.device = device
        self.capacity = int(nbytes)
        self.buf = buf if buf is not None else symm_mem.empty(self.capacity + _FLAG_BYTES, dtype=torch.uint8,
                                                              device=device)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.rank = int(self.hdl.rank)
        self.world = int(self.hdl.world_size)
        self.peers = [int(p) for p in self.hdl.buffer_ptrs]
        mc = 0
        if os.environ.get("DION_B200_MULTICAST", "1") != "0":
            try:
                mc = int(self.hdl.multicast_ptr or 0)
            except Exception:  # pragma: no cover - depends on driver / fabric
                mc = 0
        self.mc_base = mc
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        self.cursor = 0
        self.high_water = 0
        self._views: Dict[int, int] = {}  # data_ptr -> byte offset inside the arena (flag block included)
        self._guards = []                 # debug mode: (start, nbytes) of every buffer of the current step
        # the group's agreement on how much memory a step needs (post_want / agreed_want)
        self._want_view = self.buf[_WANT_OFF:_WANT_OFF + 4 * self.world].view(torch.float32)
        self._want_src = torch.zeros(self.world, dtype=torch.float32, pin_memory=True)
        self._want_host = torch.zeros(self.world, dtype=torch.float32, pin_memory=True)
        self._want_event: Optional[torch.cuda.Event] = None
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flag block is zero before anyone signals

    # -- allocation
    def reset(self) -> None:
        if _DEBUG:
            self.check_canaries()
        self.cursor = 0
        self._views.clear()
        self._guards.clear()

    def check_canaries(self) -> None:
        """Debug mode: raise if the guard behind any buffer of the current step was overwritten."""
        if not self._guards:
            return
        torch.cuda.synchronize(self.device)
        for index, (start, nbytes) in enumerate(self._guards):
            guard = self.buf[_FLAG_BYTES + start + nbytes:_FLAG_BYTES + start + nbytes + _CANARY_BYTES]
            if not bool((guard == _CANARY).all()):
                bad = int((guard != _CANARY).nonzero()[0])
                raise runtime.DionKernelError(
                    f"symmetric arena of rank {self.rank}: the guard behind buffer {index} of this step (offset {start}, "
                    f"{nbytes} bytes) was overwritten from its byte {bad} on")

    def alloc(self, shape, dtype) -> Optional[torch.Tensor]:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = (self.cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        # The cursor also advances for a request that does not fit (every later request of the step
        # then fails too): the high-water mark is the total need of one step, so that the arena
        # created at the next step boundary is large enough at once instead of growing by one
        # buffer per step.
        self.cursor = start + nbytes + (_CANARY_BYTES if _DEBUG else 0)
        self.high_water = max(self.high_water, self.cursor)
        if self.cursor > self.capacity:
            return None
        off = _FLAG_BYTES + start
        t = self.buf[off:off + nbytes].view(dtype).view(*shape)
        self._views[t.data_ptr()] = off
        if _DEBUG:
            self.buf[off + nbytes:off + nbytes + _CANARY_BYTES].fill_(_CANARY)
            self._guards.append((start, nbytes))
        return t

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        return self._views.get(t.data_ptr())

    def peer_view(self, rank: int, t: torch.Tensor) -> torch.Tensor:
        """The buffer of `rank` that sits where `t` sits in this rank's arena (same shape and
        dtype); writing to it stores into that GPU's memory over NVLink."""
        off = self._views[t.data_ptr()]
        return self.hdl.get_buffer(rank, tuple(t.shape), t.dtype, off // t.element_size())

    def peer_address(self, rank: int, t: torch.Tensor) -> int:
        return self.peers[rank] + self._views[t.data_ptr()]

    # -- agreement on the size of the next arena
    def post_want(self, nbytes: int) -> None:
        """Tell the group how many bytes this rank's last step asked for.  Every rank puts its figure
        (in MiB, exact in fp32) into its own element of a vector that the all-reduce kernel sums, and the
        result travels to pinned host memory asynchronously; :meth:`agreed_want` reads it a step later, by
        which time the copy has long finished, so the host never waits for the GPU."""
        self._want_src.zero_()
        self._want_src[self.rank] = float((int(nbytes) + (1 << 20) - 1) >> 20)
        self._want_view.copy_(self._want_src, non_blocking=True)
        self.all_reduce(self._want_view, _WANT_OFF, average=False)
        self._want_host.copy_(self._want_view, non_blocking=True)
        if self._want_event is None:
            self._want_event = torch.cuda.Event()
        self._want_event.record()

    def agreed_want(self) -> Optional[int]:
        """Largest request over the ranks of the group as of the last :meth:`post_want` (bytes), the same
        number on every rank; None before the first one."""
        if self._want_event is None:
            return None
        self._want_event.synchronize()
        return int(self._want_host.max().item()) << 20

    # -- collectives (stream ordered on the current stream)
    def all_reduce(self, t: torch.Tensor, off: int, average: bool) -> None:
        self.epoch += 1
        torch.ops.dion_b200.symm_all_reduce(t, self.peers, 0, off, self.mc_base,
                                            (1.0 / self.world) if average else 1.0, self.rank, self.epoch,
                                            self.counter, runtime.status_tensor(self.device))

    def reduce_scatter(self, t: torch.Tensor, off: int, out: torch.Tensor, average: bool) -> None:
        """out = slice `rank` of the sum (mean) of `t` over the group: every rank reads its slice from all
        peers (or lets the switch add them up, `multimem.ld_reduce`); the kernel retires once every peer
        has finished reading this rank's `t`."""
        self.epoch += 1
        torch.ops.dion_b200.symm_reduce_scatter(t.view(-1), out.view(-1), self.peers, 0, off, self.mc_base,
                                                (1.0 / self.world) if average else 1.0, self.rank, self.epoch, 0, 1,
                                                self.counter, runtime.status_tensor(self.device), _RS_WAIT_NS)

    def reduce_into(self, src: torch.Tensor, off: int, dst: torch.Tensor, scale: float = 1.0, beta: float = 0.0) -> None:
        self.epoch += 1
        torch.ops.dion_b200.symm_reduce_into(src, dst, self.peers, 0, off, scale, beta, self.rank, self.epoch,
                                             self.counter, runtime.status_tensor(self.device))

    # -- push exchanges: producers store their contribution into slot `rank` of a buffer on the consuming
    #    ranks, the consumer kernel waits for everybody's announcement and adds the slots up in rank order
    def alloc_slots(self, shape) -> Optional[torch.Tensor]:
        """fp32 buffer [world, *shape] in this rank's arena (None when it does not fit): slot s is written
        by rank s of the group."""
        return self.alloc((self.world, *shape), torch.float32)

    def slot_address(self, rank: int, slots: torch.Tensor, slot: int, elem: int = 0) -> int:
        """Address, in the memory of `rank`, of element `elem` of slot `slot` of the buffer that sits where
        `slots` sits in this rank's arena."""
        per = slots.numel() // slots.shape[0]
        return self.peers[rank] + self._views[slots.data_ptr()] + (slot * per + elem) * 4

    def wait_args(self):
        """Arguments of the flag exchange for the next consumer kernel on this arena (advances the epoch):
        (peers, flag_off, channel, rank, epoch, budget_ns)."""
        self.epoch += 1
        return (self.peers, 0, _CH_SLOT, self.rank, self.epoch, _SLOT_WAIT_NS)

    def barrier(self, channel: int = 0) -> None:
        self.epoch += 1
        torch.ops.dion_b200.symm_barrier(self.counter, self.peers, 0, channel, self.rank, self.epoch,
                                         runtime.status_tensor(self.device))


_arenas: Dict[str, SymmetricArena] = {}
_wanted: Dict[str, int] = {}
_idle: Dict[str, int] = {}
_declined: set = set()  # groups whose arena could not be created on some rank: library collectives for good
_failed = False


def _key(group: dist.ProcessGroup) -> str:
    return getattr(group, "group_name", None) or str(id(group))


def _usable(group: Optional[dist.ProcessGroup], device: torch.device) -> bool:
    if group is None or _failed or not _enabled() or device.type != "cuda":
        return False
    try:
        if dist.get_backend(group) != "nccl":
            return False
    except Exception:
        return False
    w = dist.get_world_size(group)
    return 1 < w <= 8


def create_arena(group: dist.ProcessGroup, nbytes: int, device: torch.device) -> Optional[SymmetricArena]:
    """Collective creation of an arena of at least `nbytes`.  The ranks first agree on the size (the
    largest request wins), then each allocates, then they agree on whether every allocation succeeded;
    only then do they enter the rendezvous.  Every rank therefore gets an arena of the same size or
    None, never a mixture - a rank that ran out of memory does not leave its peers waiting in the
    rendezvous, and no rank ends up on the in-tree kernels while another uses the library."""
    import torch.distributed._symmetric_memory as symm_mem

    size = torch.tensor([int(nbytes)], dtype=torch.int64, device=device)
    dist.all_reduce(size, op=dist.ReduceOp.MAX, group=group)
    nbytes = int(size.item())
    buf, err = None, None
    try:
        buf = symm_mem.empty(nbytes + _FLAG_BYTES, dtype=torch.uint8, device=device)
    except Exception as e:  # pragma: no cover - machine dependent
        err = e
    ok = torch.tensor([0 if buf is None else 1], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        if err is not None:
            print(f"[dion_b200] rank {dist.get_rank()}: symmetric allocation of {nbytes} bytes failed "
                  f"({type(err).__name__}: {err})")
        return None
    return SymmetricArena(group, nbytes, device, buf=buf)


def begin_step(groups, device: torch.device) -> None:
    """Reset (and if necessary create or grow) the arenas of `groups`.  Collective: every rank
    calls it at the same point of every optimizer step with the same groups in the same order.

    Whether an arena is created or replaced is decided from figures the whole group shares, never from
    this rank's own bookkeeping: a group without an arena agrees on its first size with a (blocking)
    all-reduce, which happens once or twice in the life of a group; a group with an arena exchanges the
    ranks' needs through the arena itself every step (:meth:`SymmetricArena.post_want`) and acts on the
    figure of the previous step, which every rank reads as the same number.  Requests are expected to be
    the same on every rank of a group (uniform shards): a step that outgrows the arena then overflows to
    ordinary memory - and the library collectives - on every rank alike."""
    for g in groups:
        if not _usable(g, device):
            continue
        k = _key(g)
        if k in _declined:
            continue
        arena = _arenas.get(k)
        local = max(_wanted.get(k, 0), arena.high_water if arena else 0)
        if arena is None:
            want = torch.tensor([local], dtype=torch.int64, device=device)
            dist.all_reduce(want, op=dist.ReduceOp.MAX, group=g)
            agreed = int(want.item())
            if agreed == 0:
                # nobody has asked for a buffer of this group yet; a group that stays unused stops asking
                _idle[k] = _idle.get(k, 0) + 1
                if _idle[k] >= 3:
                    _declined.add(k)
                continue
        else:
            agreed = arena.agreed_want()
            if agreed is None or agreed <= arena.capacity:
                arena.reset()
                arena.post_want(local)
                continue
            # every kernel that uses the old arena has to retire on every rank before it is dropped
            torch.cuda.synchronize(device)
        new = create_arena(g, max(_MIN_ARENA, int(agreed * 1.25)), device)
        if new is None:
            _declined.add(k)
            _arenas.pop(k, None)
            if dist.get_rank() == 0:
                print("[dion_b200] symmetric memory unavailable on some rank of a group; "
                      "that group uses the library collectives")
            continue
        _arenas[k] = new
        new.post_want(local)


def empty(group: Optional[dist.ProcessGroup], shape, dtype, device) -> torch.Tensor:
    """Buffer that will be reduced over `group`: from the group's arena when it has room."""
    device = torch.device(device)
    if _usable(group, device) and _key(group) not in _declined:
        arena = _arenas.get(_key(group))
        if arena is not None:
            t = arena.alloc(shape, dtype)
            if t is not None:
                return t
            _wanted[_key(group)] = arena.high_water
        else:
            n = 1
            for s in shape:
                n *= int(s)
            _wanted[_key(group)] = _wanted.get(_key(group), 0) + n * 4 + _ALIGN
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def request(group: Optional[dist.ProcessGroup], nbytes: int, device) -> None:
    """Note that `nbytes` of arena memory of `group` would have been used in this step, so that the next
    step boundary creates (or grows) the arena: for buffers that are only ever taken from an arena that
    exists, and would otherwise never cause one to be created."""
    if _usable(group, torch.device(device)) and _key(group) not in _declined and _key(group) not in _arenas:
        _wanted[_key(group)] = _wanted.get(_key(group), 0) + int(nbytes) + _ALIGN


def all_reduce(t: torch.Tensor, group: Optional[dist.ProcessGroup], average: bool = False) -> None:
    """In-place all-reduce (sum or mean) of `t` over `group`, blocking in stream order."""
    if group is None or dist.get_world_size(group) == 1:
        return
    arena = _arenas.get(_key(group)) if t.is_cuda else None
    if arena is not None:
        off = arena.offset_of(t)
        if off is not None and t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16):
            arena.all_reduce(t, off, average)
            count("all_reduce", True)
            return
    count("all_reduce", False)
    world = dist.get_world_size(group)
    nccl = t.is_cuda and dist.get_backend(group) == "nccl"
    if average and nccl:
        dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
    else:
        dist.all_reduce(t, group=group)
        if average:
            t.div_(world)


def reduce_scatter(t: torch.Tensor, group: dist.ProcessGroup, average: bool = False,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Slice `rank` of the sum (or mean) of the flat `t` over `group`, blocking in stream order;
    ``t.numel()`` must be a multiple of the group size.  Buffers in the group's arena go through the
    in-tree kernel, anything else through the process group."""
    world = dist.get_world_size(group)
    n = t.numel() // world
    if out is None:
        out = torch.empty(n, dtype=t.dtype, device=t.device)
    arena = _arenas.get(_key(group)) if t.is_cuda else None
    if arena is not None:
        off = arena.offset_of(t)
        if (off is not None and t.is_contiguous() and out.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16)
                and (n * t.element_size()) % 16 == 0 and out.data_ptr() % 16 == 0):
            arena.reduce_scatter(t, off, out, average)
            count("reduce_scatter", True)
            return out
    count("reduce_scatter", False)
    flat = t.reshape(-1)
    if average and t.is_cuda and dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out.view(-1), flat, op=dist.ReduceOp.AVG, group=group)
    else:
        dist.reduce_scatter_tensor(out.view(-1), flat, group=group)
        if average:
            out.div_(world)
    return out


def arena_for(group: Optional[dist.ProcessGroup]) -> Optional[SymmetricArena]:
    return _arenas.get(_key(group)) if group is not None else None

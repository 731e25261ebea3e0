"""Exhaustive interleaving check of the flag protocols that have no closing barrier: the push exchanges
(csrc/dion_fused.cu, csrc/symm_flags.cuh, parallel/symm.py: ``alloc_slots`` / ``wait_args``) and the all-gather
kernel's alternating staging slots (csrc/comm_kernels.cu).

The protocol: every rank's GEMM epilogue stores its partial product into slot ``rank`` of a buffer in the
memory of each consuming rank; the consumer kernel that follows on the same stream announces "my stores are
complete" by writing the exchange's epoch into every peer's flag word, waits until every peer's flag word in its
own memory has reached that epoch, and then reads all slots of its buffer.  Nothing tells a producer that a
consumer has *finished reading*, so a buffer may only be written again when the order of operations on every
rank's stream already implies that - which is a property of how many distinct buffers a cycle of exchanges
goes through, not of any single kernel.

This module states that argument as a model and checks it by enumerating every interleaving of the ranks'
actions (depth-first over the reachable states, each visited once):

* a rank executes its actions strictly in order (one CUDA stream);
* stores to a peer's slot, the flag writes to each peer, and the reads of each slot are separate atomic
  actions, so a peer's later store can fall between two reads of one consumer kernel;
* a wait is enabled once all flag words it polls have reached its epoch (flags only grow);
* a read of slot ``q`` during exchange ``x`` must see the value rank ``q`` stored for ``x`` - an older value
  means the wait let the consumer through too early, a newer one that a producer reused the buffer while it was
  still being read.

``check(world, cycles, buffers)`` returns None when no interleaving violates this, or a witness schedule.
Run as a script it prints the verdict for the configurations the package uses and for the one it must avoid.
The model is about ordering only; it says nothing about memory-model fences (the kernels use release stores /
acquire loads at system scope and a system fence before the announcement) or about timeouts.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

Action = Tuple[str, int, int]  # (kind, peer or -1, exchange index)


def program(rank: int, world: int, exchanges: Sequence[int]) -> List[Action]:
    """Actions of one rank for a sequence of exchanges; ``exchanges[x]`` is the buffer exchange x uses."""
    acts: List[Action] = []
    for x, _ in enumerate(exchanges):
        for d in range(world):
            acts.append(("push", d, x))        # producer: store my contribution into slot `rank` on rank d
        for d in range(world):
            acts.append(("announce", d, x))    # consumer kernel, first CTA: flag[d][rank] = epoch(x)
        acts.append(("wait", -1, x))           # consumer kernel: all flag[rank][*] >= epoch(x)
        for q in range(world):
            acts.append(("read", q, x))        # consumer kernel: read slot q of my buffer
    return acts


def program_pull(rank: int, world: int, exchanges: Sequence[int]) -> List[Action]:
    """Actions of one rank for the all-gather kernel's protocol (csrc/comm_kernels.cu, ``all_gather_kernel``):
    copy the own shard into the own staging slot, announce it, then pull every peer's slot as soon as that peer
    has announced.  There is no closing barrier; the slots alternate instead."""
    acts: List[Action] = []
    for x, _ in enumerate(exchanges):
        acts.append(("stage", rank, x))        # write my staging slot (local memory)
        for d in range(world):
            acts.append(("announce", d, x))
        for q in range(world):
            acts.append(("wait1", q, x))       # flag[rank][q] >= epoch(x)
            acts.append(("pull", q, x))        # read rank q's staging slot over NVLink
    return acts


def check_pull(world: int, cycles: int, buffers: Sequence[int]) -> Optional[List[Tuple[int, Action]]]:
    """As :func:`check` for the pull protocol: ``slots[q][b]`` is rank q's staging slot b, written only by q and
    read by everybody."""
    exchanges = list(buffers) * cycles
    nbuf = max(exchanges) + 1
    progs = [program_pull(r, world, exchanges) for r in range(world)]
    start = (tuple(0 for _ in range(world)), tuple(-1 for _ in range(world * nbuf)), tuple(0 for _ in range(world * world)))
    seen = {start}
    stack = [(start, [])]
    while stack:
        (pcs, slots, flags), trail = stack.pop()
        for r in range(world):
            if pcs[r] == len(progs[r]):
                continue
            kind, peer, x = progs[r][pcs[r]]
            b = exchanges[x]
            nslots, nflags = slots, flags
            if kind == "stage":
                i = r * nbuf + b
                nslots = slots[:i] + (x,) + slots[i + 1:]
            elif kind == "announce":
                i = peer * world + r
                nflags = flags[:i] + (x + 1,) + flags[i + 1:]
            elif kind == "wait1":
                if flags[r * world + peer] < x + 1:
                    continue
            elif slots[peer * nbuf + b] != x:  # pull
                return trail + [(r, progs[r][pcs[r]])]
            state = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], nslots, nflags)
            if state not in seen:
                seen.add(state)
                stack.append((state, trail + [(r, progs[r][pcs[r]])]))
    return None


def check(world: int, cycles: int, buffers: Sequence[int]) -> Optional[List[Tuple[int, Action]]]:
    """``buffers``: the buffer index used by each exchange of one cycle (an optimizer step, or a run of
    tensor-parallel products); the cycle repeats ``cycles`` times with the same buffers.  Returns a violating
    schedule ``[(rank, action), ...]`` or None."""
    exchanges = list(buffers) * cycles
    nbuf = max(exchanges) + 1
    progs = [program(r, world, exchanges) for r in range(world)]
    # shared state: slots[d][b][q] = index of the exchange whose value sits there (-1: nothing yet);
    #               flags[d][q]    = last epoch rank q announced to rank d (epoch of exchange x is x + 1)
    slots0 = tuple(-1 for _ in range(world * nbuf * world))
    flags0 = tuple(0 for _ in range(world * world))
    start = (tuple(0 for _ in range(world)), slots0, flags0)
    seen = {start}
    stack = [(start, [])]
    while stack:
        (pcs, slots, flags), trail = stack.pop()
        for r in range(world):
            if pcs[r] == len(progs[r]):
                continue
            kind, peer, x = progs[r][pcs[r]]
            b = exchanges[x]
            nslots, nflags = slots, flags
            if kind == "push":
                i = (peer * nbuf + b) * world + r
                nslots = slots[:i] + (x,) + slots[i + 1:]
            elif kind == "announce":
                i = peer * world + r
                nflags = flags[:i] + (x + 1,) + flags[i + 1:]
            elif kind == "wait":
                if any(flags[r * world + q] < x + 1 for q in range(world)):
                    continue  # not enabled yet
            else:  # read
                if slots[(r * nbuf + b) * world + peer] != x:
                    return trail + [(r, progs[r][pcs[r]])]
            state = (pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:], nslots, nflags)
            if state not in seen:
                seen.add(state)
                stack.append((state, trail + [(r, progs[r][pcs[r]])]))
    return None


# The configurations of the package and the one it has to avoid (world, cycles, buffers of one cycle).
DION_STEP = dict(world=2, cycles=3, buffers=(0, 1))        # P and R exchanges of a step: two buffers, reused every step
TP_PRODUCTS = dict(world=2, cycles=2, buffers=(0, 1))      # row-parallel products alternate between two receive buffers
LONE_BUFFER = dict(world=2, cycles=2, buffers=(0,))        # one buffer reused by consecutive exchanges: unsafe


def main() -> None:
    for name, cfg in (("Dion step (P, R)", DION_STEP), ("three ranks", dict(world=3, cycles=2, buffers=(0, 1))),
                      ("lone buffer", LONE_BUFFER)):
        witness = check(**cfg)
        report(name, witness)
    report("all-gather, two alternating staging slots", check_pull(world=3, cycles=2, buffers=(0, 1)))
    report("all-gather, one staging slot", check_pull(world=2, cycles=2, buffers=(0,)))


def report(name: str, witness) -> None:
    if witness is None:
        print(f"{name}: no interleaving reads a wrong slot")
    else:
        print(f"{name}: violated after {len(witness)} actions; last: rank {witness[-1][0]} {witness[-1][1]}")


if __name__ == "__main__":
    main()

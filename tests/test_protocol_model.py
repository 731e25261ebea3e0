"""Exhaustive interleaving check of the push-exchange protocol (dion_b200/utils/protocol_check.py): the buffer
schedules the package uses are safe under every interleaving of the ranks' streams, and the schedule it avoids -
one buffer reused by consecutive exchanges with nothing in between - is caught with a witness."""
from dion_b200.utils import protocol_check as pc


def test_two_buffers_per_cycle_are_safe_for_two_and_three_ranks():
    assert pc.check(**pc.DION_STEP) is None
    assert pc.check(**pc.TP_PRODUCTS) is None
    assert pc.check(world=3, cycles=2, buffers=(0, 1)) is None
    # more exchanges per step (several parameter classes) only add ordering
    assert pc.check(world=2, cycles=2, buffers=(0, 1, 2, 3)) is None


def test_a_lone_reused_buffer_is_caught():
    witness = pc.check(**pc.LONE_BUFFER)
    assert witness is not None
    rank, (kind, slot, exchange) = witness[-1]
    assert kind == "read" and exchange == 0
    # the reader of exchange 0 was overtaken by the other rank's store for exchange 1 into the same buffer
    overtaking = [(r, a) for r, a in witness if a[0] == "push" and a[2] == 1 and a[1] == rank]
    assert overtaking and overtaking[0][0] == slot


def test_the_model_blocks_a_wait_until_every_peer_announced():
    prog = pc.program(0, 2, [0])
    kinds = [a[0] for a in prog]
    assert kinds == ["push", "push", "announce", "announce", "wait", "read", "read"]
    # a single exchange can never read before both pushes happened: no violation in any interleaving
    assert pc.check(world=2, cycles=1, buffers=(0,)) is None


def test_all_gather_staging_slots_must_alternate():
    """The all-gather kernel has no closing barrier: with two alternating staging slots no interleaving lets a
    rank overwrite a slot that a peer still pulls; with a single slot one does."""
    assert pc.check_pull(world=2, cycles=3, buffers=(0, 1)) is None
    assert pc.check_pull(world=3, cycles=2, buffers=(0, 1)) is None
    witness = pc.check_pull(world=2, cycles=2, buffers=(0,))
    assert witness is not None and witness[-1][1][0] == "pull"


def test_the_rule_is_a_reuse_distance_of_two():
    """A buffer may be rewritten once one other exchange has passed since it was read: schedules whose every
    reuse is at least two exchanges apart are safe, a back-to-back reuse anywhere in the cycle is not."""
    for buffers, safe in (((0, 1, 0, 2), True), ((0, 1, 2), True), ((0, 1, 1), False), ((0, 0, 1), False)):
        assert (pc.check(world=2, cycles=2, buffers=buffers) is None) == safe, buffers

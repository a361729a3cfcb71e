"""The arithmetic of the kernel's one-word grid barrier, replayed on the CPU.

`tk::grid_barrier` (trainkernel_b200/csrc/tk_device.cuh) keeps ONE 32-bit word per launch slot: bit 31
is the barrier's phase, bits 0..30 count arrivals.  Block 0 adds 2^31 - (arrivals - 1), every other block
adds 1; a waiting block polls until the phase differs from the one its own atomic returned, and the last
arriver recognises itself from the count it was handed and does not poll.  This file checks those rules
with the same unsigned arithmetic for every arrival order that matters: they are what lets the word be
reused by any number of barriers, launches and graph replays without a reset.
"""
import itertools
import random

MASK = 0xFFFFFFFF
PHASE = 0x80000000
COUNT = 0x7FFFFFFF


def arrive(word: int, leader: bool, arrivals: int) -> tuple[int, int, bool]:
    """One block's atomic: returns (new word, value before, whether the block knows it was last)."""
    before = word
    word = (word + (PHASE - (arrivals - 1) if leader else 1)) & MASK
    counted = before & COUNT
    last = counted == arrivals - 1 if leader else counted == COUNT
    return word, before, last


def released(word: int, before: int) -> bool:
    """What a waiting block evaluates on every poll."""
    return ((word ^ before) & PHASE) != 0


def run_barrier(word: int, order: list[int], arrivals: int) -> int:
    """All blocks of `order` arrive (block 0 is the leader); checks the rules and returns the word afterwards."""
    seen = {}
    lasts = []
    for position, block in enumerate(order):
        word, before, last = arrive(word, block == 0, arrivals)
        seen[block] = before
        lasts.append(last)
        everyone = position == len(order) - 1
        # nobody is released before the last arrival, everybody right after it
        assert all(released(word, b) == everyone for b in seen.values())
    assert lasts == [False] * (len(order) - 1) + [True]      # exactly the last arriver knows it, whoever it is
    return word


def test_every_order_of_a_small_grid_releases_exactly_at_the_last_arrival():
    for arrivals in (2, 3, 4, 5):
        for order in itertools.permutations(range(arrivals)):
            word = 0
            for _ in range(3):                                 # consecutive barriers reuse the word
                word = run_barrier(word, list(order), arrivals)
                assert word & COUNT == 0                       # the count is back at zero: nothing to reset


def test_a_full_grid_over_many_barriers_and_launches():
    rng = random.Random(0)
    word = 0
    for barrier in range(2000):                                # the phase bit flips 2000 times: wrap-around is the normal case
        order = list(range(148))
        rng.shuffle(order)
        word = run_barrier(word, order, 148)
        assert word == (PHASE if barrier % 2 == 0 else 0)


def test_an_expected_count_above_the_grid_never_releases():
    # what the timeout test on the GPU provokes: one arrival more is expected than blocks exist
    word, befores = 0, []
    for block in range(8):
        word, before, last = arrive(word, block == 0, 9)
        befores.append(before)
        assert not last
    assert not any(released(word, before) for before in befores)

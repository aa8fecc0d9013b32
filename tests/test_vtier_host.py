"""Residency logic of the V tier (pure host code, no GPU): CLOCK victims, copy
runs, map updates, the invariants of the reference's tier (no aliasing, owners
agree with the map: ``tier/__init__.py:11-17``)."""
from __future__ import annotations

import numpy as np

from locks.attention.vtier import SlotClock


def _apply(dev_map, updates):
    for b, s in updates:
        dev_map[b] = s


def test_runs_of_contiguous_blocks_land_in_contiguous_slots():
    c = SlotClock(num_blocks=100, n_slots=16)
    runs, upd = c.plan([7, 5, 6, 20, 21, 40], np.zeros(16, np.uint8), 1 << 30)
    assert runs == [(5, 0, 3), (20, 3, 2), (40, 5, 1)]
    assert dict(upd) == {5: 0, 6: 1, 7: 2, 20: 3, 21: 4, 40: 5}
    c.check()


def test_clock_passes_over_slots_read_in_the_last_step():
    c = SlotClock(num_blocks=64, n_slots=4)
    c.plan([10, 11, 12, 13], np.zeros(4, np.uint8), 1 << 30)      # fills slots 0-3
    ref = np.array([1, 1, 0, 1], np.uint8)                        # slot 2 was idle
    runs, upd = c.plan([30], ref, 1 << 30)
    assert runs == [(30, 2, 1)]
    assert dict(upd) == {12: -1, 30: 2}
    c.check()
    # everything was read: the hand gives each slot its second chance, then evicts
    runs, upd = c.plan([31], np.ones(4, np.uint8), 1 << 30)
    assert len(runs) == 1 and runs[0][2] == 1
    c.check()


def test_mirror_and_device_map_stay_equal_under_random_traffic():
    rng = np.random.default_rng(0)
    NB, S = 300, 24
    c = SlotClock(NB, S)
    dev_map = np.full(NB, -1, np.int32)
    for step in range(200):
        want = rng.choice(NB, size=rng.integers(1, 40), replace=False)
        ref = np.zeros(S, np.uint8)
        missed = []
        for b in want:                       # what the decode kernel notes
            if dev_map[b] >= 0:
                ref[dev_map[b]] = 1
            else:
                missed.append(int(b))
        runs, upd = c.plan(missed, ref, max_blocks=16)
        _apply(dev_map, upd)
        assert (dev_map == c.slot_of).all()
        c.check()
        assert sum(n for _, _, n in runs) <= 16
        if step % 17 == 0:                   # a block changes owner
            gone = rng.choice(NB, size=5, replace=False).tolist()
            _apply(dev_map, c.drop(gone))
            assert (dev_map == c.slot_of).all()
            c.check()


def test_a_listed_block_the_mirror_still_holds_is_refilled_in_place():
    c = SlotClock(50, 8)
    c.plan([3, 4], np.zeros(8, np.uint8), 1 << 30)
    # device side dropped block 3 (reuse) without telling the mirror
    runs, upd = c.plan([3], np.zeros(8, np.uint8), 1 << 30)
    assert runs == [(3, 0, 1)] and dict(upd) == {3: 0}
    c.check()

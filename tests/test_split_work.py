"""The planner that cuts decode items into shares of about equal length (host side only)."""
import random

import numpy as np

from llm_steadyinfer_b200.csrc.ops import split_work


def _shares(work):
    live = work[work[:, 0] >= 0]
    return {int(i): int(live[live[:, 0] == i][0, 2]) for i in set(live[:, 0].tolist())}, live


def test_every_share_is_listed_once_and_slots_do_not_overlap():
    rng = random.Random(3)
    for _ in range(300):
        n = rng.randint(1, 70)
        tiles = [rng.choice([0, 1, 2, 3, 5, 17, 64, 128, 500]) for _ in range(n)]
        budget = rng.choice([1, 5, 37, 148])
        entries = budget + n
        work = split_work(tiles, budget, entries, 32, rng.choice([1, 2, 4]))
        assert work.shape == (entries, 4) and work.dtype == np.int32
        sp, live = _shares(work)
        assert set(sp) == {i for i, t in enumerate(tiles) if t > 0}
        taken = set()
        for i, k in sp.items():
            mine = live[live[:, 0] == i]
            assert sorted(mine[:, 1].tolist()) == list(range(k)) and (mine[:, 2] == k).all()
            first = int(mine[0, 3])
            assert (mine[:, 3] == first).all() and 1 <= k <= 32
            slots = set(range(first, first + k))
            assert not slots & taken and max(slots) < entries
            taken |= slots
        rest = work[len(live):]
        assert (rest[:, 0] == -1).all(), "live entries come first"


def test_equal_items_get_equal_shares_within_the_budget():
    sp, live = _shares(split_work([128] * 8, 37, 45, 32, 2))
    assert set(sp.values()) == {4} and len(live) == 32          # 5 each would need 40 > 37
    sp, _ = _shares(split_work([128] * 5, 37, 42, 32, 2))
    assert set(sp.values()) == {7}


def test_a_long_item_among_short_ones_is_cut_most():
    sp, live = _shares(split_work([128] + [8] * 7, 37, 45, 32, 2))
    assert sp[0] >= 20 and all(sp[i] <= 2 for i in range(1, 8)) and len(live) <= 37
    # more items than shares that run at once: the long one is still cut, to the mean load of a share
    sp, live = _shares(split_work([128] + [4] * 63, 37, 37 + 64, 32, 2))
    assert sp[0] >= 10 and all(sp[i] == 1 for i in range(1, 64))


def test_no_share_is_shorter_than_the_least_and_no_item_has_more_than_the_most():
    sp, _ = _shares(split_work([3, 1, 1000], 200, 203, 32, 2))
    assert sp[0] <= 2 and sp[1] == 1 and sp[2] == 32


def test_more_items_than_slots():
    # many equal sequences stay whole: HBM is busy either way, and every share has its cost
    sp, live = _shares(split_work([128] * 64, 37, 37 + 256, 32, 2))
    assert set(sp.values()) == {1}
    sp, _ = _shares(split_work([16] * 100, 37, 37 + 400, 32, 2))
    assert set(sp.values()) == {1}
    # a few more sequences than slots: whole, the last three blocks of each head would run alone for as long
    # as all the others took; cut, the chains on the slots are about equal
    sp, live = _shares(split_work([128] * 40, 37, 37 + 160, 32, 2))
    assert len(set(sp.values())) == 1 and 3 <= sp[0] <= 5 and len(live) <= 37 + 160
    # with no room for finer cuts the items stay whole
    sp, _ = _shares(split_work([128] * 40, 37, 37 + 40, 32, 2))
    assert set(sp.values()) == {1}

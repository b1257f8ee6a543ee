"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from ziglm_b200.cache import (CacheError, CacheFull, FreeList, GroupPages, NoFreeSlot, SequenceTooLong, SlotTable)


def test_free_list_hands_out_lowest_first_and_takes_back():
    f = FreeList(4, "slot")
    assert [f.take() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(NoFreeSlot):
        f.take()
    f.give_back(2); f.give_back(0)
    assert f.take() == 0 and f.take() == 2
    f.check()


def test_double_free_and_unknown_are_errors():
    f = FreeList(2, "page")
    a = f.take()
    f.give_back(a)
    with pytest.raises(CacheError, match="twice"):
        f.give_back(a)
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back(5)
    with pytest.raises(CacheError):
        f.give_back(1)            # never handed out


def _table(n_slots=3, n_pages=8, page=64, max_len=256, window=None):
    groups = [GroupPages(n_pages, page, None)]
    if window is not None:
        groups.append(GroupPages(n_pages, page, window))
    return SlotTable(n_slots, groups, max_len)


def test_pages_grow_with_the_sequence_and_come_back():
    t = _table()
    s = t.alloc()
    t.reserve({s: 5}); t.advance({s: 5})
    assert t.length_of(s) == 5 and t.groups[0].pages_of[s] == [0]
    t.reserve({s: 59}); t.advance({s: 59})
    assert t.groups[0].pages_of[s] == [0]                 # 64 positions still fit one page
    t.reserve({s: 1}); t.advance({s: 1})
    assert t.groups[0].pages_of[s] == [0, 1]
    u = t.alloc()
    t.reserve({u: 130}); t.advance({u: 130})
    assert t.groups[0].pages_of[u] == [2, 3, 4]
    t.check()
    t.free(s)
    assert t.groups[0].pool.n_free == 5
    v = t.alloc()
    assert v == s                                         # the slot is used again
    t.reserve({v: 1})
    assert t.groups[0].pages_of[v] == [0]                 # and so is its page
    with pytest.raises(CacheError):
        t.free(s) or t.free(s)
    t.check()


def test_reserve_is_all_or_nothing():
    t = _table(n_pages=3)
    a, b = t.alloc(), t.alloc()
    t.reserve({a: 64}); t.advance({a: 64})
    with pytest.raises(CacheFull):
        t.reserve({a: 64, b: 128})                        # needs 1 + 2 pages, 2 are free
    assert t.groups[0].pool.n_free == 2 and b not in t.groups[0].pages_of
    with pytest.raises(SequenceTooLong):
        t.reserve({a: 300})
    with pytest.raises(CacheError):
        t.reserve({7: 1})
    t.check()


def test_no_free_slot():
    t = _table(n_slots=1)
    t.alloc()
    with pytest.raises(NoFreeSlot):
        t.alloc()


def test_window_group_lets_go_of_pages_behind_the_window():
    t = _table(n_pages=8, max_len=512, window=70)
    s = t.alloc()
    t.reserve({s: 200}); t.advance({s: 200})
    full, win = t.groups
    assert full.pages_of[s] == [0, 1, 2, 3]
    # the next token sits at 200 and sees 131..200: pages 0 and 1 (positions 0..127) are behind it
    assert win.pages_of[s] == [-1, -1, 2, 3]
    assert win.pool.n_free == 6 and full.pool.n_free == 4
    t.check()
    t.free(s)
    assert win.pool.n_free == 8 and full.pool.n_free == 8
    t.check()


def test_random_traffic_keeps_every_slot_and_page_accounted_for():
    rng = random.Random(7)
    t = _table(n_slots=5, n_pages=24, max_len=400, window=100)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.25 and t.slots.n_free:
            s = t.alloc()
            assert s not in live
            live[s] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            t.free(s)
            del live[s]
        elif live:
            batch = rng.sample(list(live), rng.randint(1, len(live)))
            growth = {s: rng.randint(1, 90) for s in batch}
            try:
                t.reserve(growth)
            except (CacheFull, SequenceTooLong):
                t.check()
                continue
            t.advance(growth)
            for s, n in growth.items():
                live[s] += n
                assert t.length_of(s) == live[s]
        t.check()
        held = [p for g in t.groups[:1] for pages in g.pages_of.values() for p in pages if p >= 0]
        assert len(held) == len(set(held))                 # no page in two sequences
    for s in list(live):
        t.free(s)
    t.check()
    assert all(g.pool.n_free == g.pool.capacity for g in t.groups) and t.slots.n_free == 5


def test_the_array_of_block_tables_follows_the_lists():
    """The pages of a slot are also kept as a row of an int32 array (what a step copies to the device):
    after growth, release behind a window, freeing and reuse the two agree."""
    import numpy as np
    from ziglm_b200.cache.slots import GroupPages, SlotTable
    groups = [GroupPages(40, 4, None), GroupPages(40, 4, 6)]
    for g in groups:
        g.mirror(5, 10)
    table = SlotTable(5, groups, 40)

    def check():
        for g in groups:
            for slot in range(5):
                pages = g.pages_of.get(slot, [])
                want = np.full(10, -1, dtype=np.int32)
                want[:len(pages)] = pages
                assert (g.table[slot] == want).all()

    a, b = table.alloc(), table.alloc()
    for n_a, n_b in ((3, 9), (1, 1), (6, 2), (1, 1), (13, 5)):
        table.reserve({a: n_a, b: n_b})
        table.advance({a: n_a, b: n_b})
        check()
    assert (groups[1].table[a, :3] == -1).all()        # behind the window of 6 after 24 positions
    table.free(a)
    check()
    c = table.alloc()
    table.reserve({c: 7})
    table.advance({c: 7})
    check()
    table.check()

"""The cache's bookkeeping: no slot or page is lost, held twice or freed
twice; pages are used again; a step that does not fit changes nothing."""
import random

import pytest

from foundry_b200.cache import (PAGE, CacheFull, CacheMisuse, FreeList, GroupPages, SlotTable,
                                pages_for)


def test_free_list_hands_out_each_id_once():
    fl = FreeList(4, "page")
    got = fl.take(3)
    assert sorted(got) == [0, 1, 2] and fl.free == 1 and fl.held == 3
    with pytest.raises(CacheFull):
        fl.take(2)
    assert fl.free == 1  # a refused request takes nothing
    fl.give([got[1]])
    with pytest.raises(CacheMisuse):
        fl.give([got[1]])  # freed twice
    with pytest.raises(CacheMisuse):
        fl.give([3])  # never held
    with pytest.raises(CacheMisuse):
        fl.give([17])
    fl.check()
    assert sorted(fl.take(2)) == sorted([got[1], 3])


def test_pages_follow_the_length():
    table = SlotTable(4, [GroupPages(8)])
    s = table.open()
    table.grow(s, 1)
    assert len(table.groups[0].pages(s)) == 1
    table.grow(s, PAGE)
    assert len(table.groups[0].pages(s)) == 1
    table.grow(s, PAGE + 1)
    assert len(table.groups[0].pages(s)) == 2 and table.length[s] == PAGE + 1
    with pytest.raises(CacheMisuse):
        table.grow(s, 3)  # a sequence never shrinks
    table.close(s)
    assert table.groups[0].pool.free == 8 and table.slots.free == 4
    with pytest.raises(CacheMisuse):
        table.close(s)
    with pytest.raises(CacheMisuse):
        table.grow(s, 1)
    table.check()


def test_a_window_group_keeps_a_ring():
    group = GroupPages(16, window=100)  # 2 pages of window + 1
    assert group.ring_pages == 3
    table = SlotTable(2, [GroupPages(64), group])
    s = table.open()
    table.grow(s, 1000)
    assert len(table.groups[0].pages(s)) == pages_for(1000)
    assert len(group.pages(s)) == 3
    table.close(s)
    table.check()


def test_reservation_is_all_or_nothing():
    table = SlotTable(4, [GroupPages(4)])
    a, b = table.open(), table.open()
    assert table.can_grow({a: 2 * PAGE, b: 2 * PAGE})
    assert not table.can_grow({a: 3 * PAGE, b: 2 * PAGE})
    table.grow(a, 2 * PAGE)
    assert not table.can_grow({a: 2 * PAGE + 1, b: 2 * PAGE})
    assert table.can_grow({b: 2 * PAGE})


def test_no_slot_or_page_is_lost_under_random_traffic():
    rng = random.Random(0)
    table = SlotTable(6, [GroupPages(40), GroupPages(20, window=130)])
    live = {}
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and table.slots.free:
            live[table.open()] = 0
        elif action < 0.8 and live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 150)
            if table.can_grow({s: new}):
                table.grow(s, new)
                live[s] = new
            else:
                with pytest.raises(CacheFull):
                    table.grow(s, new)
                # a refused growth in a later group may leave earlier groups grown;
                # the engine asks can_grow first. Close the sequence to stay consistent.
                table.close(s)
                del live[s]
        elif live:
            s = rng.choice(list(live))
            table.close(s)
            del live[s]
        table.check()
        assert table.slots.held == len(live)
        for s, n in live.items():
            assert len(table.groups[0].pages(s)) == pages_for(n)
            assert len(table.groups[1].pages(s)) == min(pages_for(n), 4)
    for s in list(live):
        table.close(s)
    table.check()
    assert table.slots.free == 6
    assert [g.pool.free for g in table.groups] == [40, 20]


def test_given_back_pages_are_used_again():
    table = SlotTable(2, [GroupPages(3)])
    a = table.open()
    table.grow(a, 3 * PAGE)
    first = list(table.groups[0].pages(a))
    b = table.open()
    with pytest.raises(CacheFull):
        table.grow(b, 1)
    table.close(a)
    table.grow(b, 3 * PAGE)
    assert sorted(table.groups[0].pages(b)) == sorted(first)


def test_a_window_ring_limits_the_tokens_of_one_step():
    """A step writes all its keys before it reads any: with a ring of
    ceil(W / 64) + 1 pages, a step of c tokens from position s keeps the keys
    (s - W, s] of its first token only while c <= ring * 64 - W + 1. Checked by
    replaying the ring's overwrites."""
    import torch
    from foundry_b200.cache import KVRequest, SequenceCache
    for window in (1, 33, 64, 100, 128, 200):
        cache = SequenceCache({0: KVRequest(2, 16), 1: KVRequest(2, 16, window)}, 1024, 2,
                              torch.float32, torch.device("cpu"))
        limit = cache.step_token_limit()
        ring = pages_for(window) + 1
        assert limit == ring * PAGE - window + 1 >= PAGE
        for start in (0, 5, 63, 64, 300):
            for count, intact in ((limit, True), (limit + 1, False)):
                rows = {}  # ring row -> position held after the step's writes
                for p in range(max(0, start - ring * PAGE), start + count):
                    rows[p % (ring * PAGE)] = p
                needed = range(max(0, start - window + 1), start + 1)
                ok = all(rows.get(p % (ring * PAGE)) == p for p in needed)
                assert ok or not intact
                if not intact and start >= window:
                    assert not ok
    no_window = SequenceCache({0: KVRequest(2, 16)}, 1024, 2, torch.float32, torch.device("cpu"))
    assert no_window.step_token_limit() is None


def test_a_step_can_be_taken_back():
    """`forget_from` gives up a slot's last tokens and keeps its pages; it cannot
    grow a slot, touch a free one, or take back state of fixed size."""
    from foundry_b200.cache.pages import CacheMisuse, GroupPages, SlotTable
    table = SlotTable(2, [GroupPages(4)])
    slot = table.open()
    table.grow(slot, 64)
    table.grow(slot, 65)
    pages = list(table.groups[0].pages(slot))
    table.forget_from(slot, 64)
    assert table.length[slot] == 64 and table.groups[0].pages(slot) == pages
    table.grow(slot, 65)  # the same page serves again
    assert table.groups[0].pages(slot) == pages
    with pytest.raises(CacheMisuse):
        table.forget_from(slot, 66)
    with pytest.raises(CacheMisuse):
        table.forget_from(slot, -1)
    table.close(slot)
    with pytest.raises(CacheMisuse):
        table.forget_from(slot, 0)
    table.check()

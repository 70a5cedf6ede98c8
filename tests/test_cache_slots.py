"""Slots and pages: nothing lost, held twice or freed twice; what ended is used again (no device)."""
import random

import pytest

from transformer_b200.cache import PAGE, CacheError, FreeList, SequenceTable


def test_free_list_hands_out_each_once():
    fl = FreeList(5, "slot")
    got = [fl.take() for _ in range(5)]
    assert sorted(got) == list(range(5)) and got[0] == 0
    with pytest.raises(CacheError, match="no free slot"):
        fl.take()
    fl.give_back(3)
    with pytest.raises(CacheError, match="not held"):
        fl.give_back(3)
    with pytest.raises(CacheError, match="not held"):
        fl.give_back(17)
    assert fl.take() == 3
    fl.check()


def test_pages_follow_the_length():
    t = SequenceTable(max_slots=4, n_pages=6, max_context=300)
    s = t.open()
    assert t.extend(s, 1) == 0 and len(t.page_list[s]) == 1
    assert t.extend(s, 63) == 1 and len(t.page_list[s]) == 1
    assert t.extend(s, 1) == 64 and len(t.page_list[s]) == 2
    assert t.extend(s, 200) == 65 and len(t.page_list[s]) == 5
    with pytest.raises(CacheError, match="context"):
        t.extend(s, 100)
    s2 = t.open()
    t.extend(s2, 64)
    with pytest.raises(CacheError, match="cache full"):
        t.extend(s2, 1)
    assert t.length[s2] == 64, "a refused extension changes nothing"
    t.check()
    t.close(s)
    assert t.pages.free == 5
    t.extend(s2, 1)
    t.check()


def test_close_twice_and_unknown_slot():
    t = SequenceTable(2, 4, 128)
    s = t.open()
    t.close(s)
    with pytest.raises(CacheError, match="not open"):
        t.close(s)
    with pytest.raises(CacheError, match="not open"):
        t.extend(s, 1)


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    t = SequenceTable(max_slots=8, n_pages=12, max_context=640)
    live = []
    seen_pages = set()
    for _ in range(3000):
        op = rng.random()
        if op < 0.3 and len(live) < 8:
            live.append(t.open())
        elif op < 0.8 and live:
            s = rng.choice(live)
            try:
                t.extend(s, rng.choice([1, 1, 1, 7, 64, 100]))
            except CacheError:
                pass
            seen_pages.update(t.page_list[s])
        elif live:
            s = live.pop(rng.randrange(len(live)))
            t.close(s)
        t.check()
    for s in live:
        t.close(s)
    t.check()
    assert t.pages.free == 12 and t.slots.free == 8
    assert seen_pages == set(range(12)), "every page came into use again"
    assert PAGE == 64

"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice."""
import random

import pytest
import torch

from alpacca_b200.cache import CacheFull, IdPool, SequenceCache
from alpacca_b200.parts import KVSpec, StateSpec


def test_id_pool():
    p = IdPool(4, "thing")
    got = [p.alloc() for _ in range(4)]
    assert got == [0, 1, 2, 3] and p.n_free == 0
    with pytest.raises(CacheFull):
        p.alloc()
    p.free(2)
    p.free(0)
    with pytest.raises(ValueError, match="freed twice"):
        p.free(2)
    with pytest.raises(ValueError, match="does not exist"):
        p.free(9)
    assert p.alloc() == 0 and p.alloc() == 2      # the lowest free id first: freed ids are used again
    p.check()
    with pytest.raises(CacheFull):
        p.alloc_many(1)


def make_cache(max_tokens=64 * 10, max_slots=4, max_positions=300, specs=None):
    specs = specs or [KVSpec(2, 16), KVSpec(2, 16), KVSpec(2, 16)]
    return SequenceCache(specs, max_tokens, max_slots, max_positions, torch.float32, "cpu")


def test_groups_by_needs():
    c = make_cache(specs=[KVSpec(2, 16), KVSpec(2, 16, window=70), None, StateSpec((3, 5)), KVSpec(2, 16)])
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert c.kv_groups[0].k.shape == (2, 10, 2, 64, 16) and c.kv_groups[1].k.shape == (1, 10, 2, 64, 16)
    assert c.state_groups[0].state.shape == (1, 4, 3, 5)
    assert c.entry_place[2] is None and c.entry_place[0][:2] == ("kv", 0) and c.entry_place[4] == ("kv", 0, 1)
    v = c.entry_view(4, [torch.zeros(1, 1, dtype=torch.int32)] * 2)
    assert v.k.data_ptr() == c.kv_groups[0].k[1].data_ptr()


def test_slots_and_pages_grow_and_come_back():
    c = make_cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 5), (b, 130)])
    c.commit([(a, 5), (b, 130)])
    g = c.kv_groups[0]
    assert len(g.page_lists[a]) == 1 and len(g.page_lists[b]) == 3 and g.pages.n_held == 4
    c.reserve([(a, 59)])          # 64 tokens still fit the first page
    c.commit([(a, 59)])
    assert len(g.page_lists[a]) == 1
    c.reserve([(a, 1)])
    c.commit([(a, 1)])
    assert len(g.page_lists[a]) == 2 and c.length(a) == 65
    c.check()
    c.free_slot(b)
    assert g.pages.n_held == 2 and c.slots.n_held == 1
    with pytest.raises(ValueError, match="freed twice"):
        c.free_slot(b)
    b2 = c.alloc_slot()
    assert b2 == b and c.length(b2) == 0 and g.page_lists[b2] == []     # the slot is used again, empty
    c.check()


def test_full_cache_raises_and_changes_nothing():
    c = make_cache(max_tokens=64 * 3)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 100)])
    c.commit([(a, 100)])
    before = [list(pl) for pl in c.kv_groups[0].page_lists.values()]
    with pytest.raises(CacheFull, match="cache full"):
        c.reserve([(a, 1), (b, 65)])
    assert [list(pl) for pl in c.kv_groups[0].page_lists.values()] == before
    short = make_cache(max_positions=50)
    with pytest.raises(CacheFull, match="context window full"):
        short.reserve([(short.alloc_slot(), 51)])
    for _ in range(2):
        c.alloc_slot()
    with pytest.raises(CacheFull, match="no free slot"):
        c.alloc_slot()


def test_window_group_gives_pages_back_early():
    c = make_cache(specs=[KVSpec(2, 16, window=70)], max_tokens=64 * 4, max_positions=10_000)
    s = c.alloc_slot()
    g = c.kv_groups[0]
    for _ in range(40):                    # 40 steps of 50 tokens: far more than the 4 pages hold at once
        c.reserve([(s, 50)])
        c.commit([(s, 50)])
        live = [p for p in g.page_lists[s] if p >= 0]
        assert len(live) <= 4 and len(live) == g.pages.n_held
        first_needed = c.length(s) - 50 - 70 + 1
        for i, p in enumerate(g.page_lists[s]):
            if (i + 1) * 64 > max(first_needed, 0):
                assert p >= 0, "a page inside the window was given back"
    c.free_slot(s)
    assert g.pages.n_held == 0


def test_state_is_zero_for_a_new_sequence():
    c = make_cache(specs=[StateSpec((4,))])
    s = c.alloc_slot()
    c.state_groups[0].state[0, s] = 7.0
    c.free_slot(s)
    assert c.alloc_slot() == s and c.state_groups[0].state[0, s].abs().sum() == 0


def test_block_table():
    c = make_cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 70), (b, 3)])
    width = c.table_width(0, [b, a])
    out = torch.empty(2, width, dtype=torch.int32)
    c.fill_block_table(0, [b, a], out, width)
    assert width == 2 and out[1].tolist() == c.kv_groups[0].page_lists[a] and out[0, 0].item() == c.kv_groups[0].page_lists[b][0]


def test_random_walk_keeps_the_books():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 12, max_slots=5, max_positions=400)
    live = []
    for _ in range(600):
        r = rng.random()
        try:
            if r < 0.25 and len(live) < 5:
                live.append(c.alloc_slot())
            elif r < 0.4 and live:
                c.free_slot(live.pop(rng.randrange(len(live))))
            elif live:
                reqs = [(s, rng.choice([1, 1, 1, 17, 64, 90])) for s in rng.sample(live, rng.randint(1, len(live)))]
                c.reserve(reqs)
                c.commit(reqs)
        except CacheFull:
            pass
        c.check()
        g = c.kv_groups[0]
        assert all(len(g.page_lists[s]) >= -(-c.length(s) // 64) for s in live)
    for s in live:
        c.free_slot(s)
    c.check()
    assert c.kv_groups[0].pages.n_held == 0 and c.slots.n_held == 0


def test_truncate_gives_back_the_pages_behind_the_new_length():
    c = make_cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 200), (b, 70)])
    c.commit([(a, 200), (b, 70)])
    g = c.kv_groups[0]
    kept = list(g.page_lists[a][:2])
    assert g.pages.n_held == 4 + 2
    c.truncate(a, 200)                       # nothing to do
    assert g.pages.n_held == 6
    c.truncate(a, 65)                        # positions 0..64: two pages stay, two come back
    assert c.length(a) == 65 and g.page_lists[a] == kept and g.pages.n_held == 2 + 2
    c.check()
    c.truncate(a, 64)                        # a page boundary: the second page holds nothing any more
    assert g.page_lists[a] == kept[:1] and g.pages.n_held == 1 + 2
    c.reserve([(a, 10)])                     # and the sequence grows again from there
    c.commit([(a, 10)])
    assert c.length(a) == 74 and len(g.page_lists[a]) == 2
    c.truncate(a, 0)
    assert c.length(a) == 0 and g.page_lists[a] == [] and g.pages.n_held == 2
    c.check()
    with pytest.raises(ValueError, match="cannot be truncated to"):
        c.truncate(b, 71)
    with pytest.raises(ValueError, match="cannot be truncated to"):
        c.truncate(b, -1)
    with pytest.raises(ValueError, match="not in use"):
        c.truncate(3, 0)
    c.free_slot(a)
    c.free_slot(b)
    assert g.pages.n_held == 0
    c.check()


def test_truncate_is_refused_where_it_cannot_be_undone():
    # a state of fixed size has no earlier value
    c = make_cache(specs=[KVSpec(2, 16), StateSpec((4,))])
    s = c.alloc_slot()
    c.reserve([(s, 100)])
    c.commit([(s, 100)])
    with pytest.raises(ValueError, match="state of fixed size"):
        c.truncate(s, 50)
    c.truncate(s, 100)
    assert c.length(s) == 100
    # a window that has given pages back: the shorter sequence would read them
    c = make_cache(specs=[KVSpec(2, 16, window=70)])
    s = c.alloc_slot()
    c.reserve([(s, 250)])
    c.commit([(s, 250)])
    c.reserve([(s, 1)])                      # positions before 250 - 70 + 1 = 181 are not needed: pages 0 and 1 go
    c.commit([(s, 1)])
    g = c.kv_groups[0]
    assert g.page_lists[s][:2] == [-1, -1]
    with pytest.raises(ValueError, match="already given back"):
        c.truncate(s, 150)                   # would read from position 81, page 1
    assert c.length(s) == 251
    c.truncate(s, 200)                       # reads from position 131, page 2: held
    assert c.length(s) == 200 and len(g.page_lists[s]) == 4
    c.check()

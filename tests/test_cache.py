"""The cache's bookkeeping: no page or slot lost, held twice or freed twice (no GPU)."""
import random

import pytest

from odin_infer_b200.cache import CacheError, CacheManager, KVRequest, PAGE, PagePool


def test_page_pool():
    p = PagePool(5)
    a = p.take(3)
    assert len(set(a)) == 3 and p.n_free == 2 and p.n_held == 3
    with pytest.raises(CacheError, match="full"):
        p.take(3)
    p.give_back(a[:1])
    with pytest.raises(CacheError, match="twice"):
        p.give_back(a[:1])
    with pytest.raises(CacheError, match="does not belong"):
        p.give_back([7])
    p.check()
    b = p.take(3)
    assert a[0] in b  # a freed page is used again
    p.give_back(b + a[1:])
    p.check()
    assert p.n_free == 5


def manager(n_tokens=64 * 10, ctx=64 * 6, window=0):
    m = CacheManager(n_tokens, ctx)
    m.add_entry(KVRequest(2, 16), 0)
    m.add_entry(KVRequest(2, 16), 0)
    if window:
        m.add_entry(KVRequest(2, 16, window), 0)
    m.add_entry(None, 100)
    m.entry_writes = [True] * len(m.line_of)
    return m


def test_groups_and_lines():
    m = manager(window=128)
    assert len(m.groups) == 2  # all keys; a window of them: storage of their own
    full, win = m.groups[KVRequest(2, 16).key], m.groups[KVRequest(2, 16, 128).key]
    assert full.n_lines == 2 and win.n_lines == 1 and full is not win
    assert m.line_of[0] == (KVRequest(2, 16).key, 0) and m.line_of[1] == (KVRequest(2, 16).key, 1)
    assert m.line_of[3] is None and m.state_bytes_per_slot == 256 and m.state_offset_of[3] == 0
    # an entry that reads another entry's cache gets its line, and no line of its own
    i = m.add_entry(KVRequest(2, 16), 0, shares_line_of=1)
    assert m.line_of[i] == m.line_of[1] and full.n_lines == 2
    with pytest.raises(CacheError, match="keeps none"):
        m.add_entry(KVRequest(2, 16), 0, shares_line_of=3)
    with pytest.raises(CacheError, match="cannot read"):
        m.add_entry(KVRequest(4, 16), 0, shares_line_of=0)


def test_slots_and_growth():
    m = manager()
    s0, s1 = m.take_slot(), m.take_slot()
    assert m.extend(s0, 70) == 0 and m.lengths[s0] == 70
    assert m.extend(s1, 1) == 0
    g = next(iter(m.groups.values()))
    assert g.pool.n_held == 3
    assert m.extend(s0, 58) == 70 and g.pool.n_held == 3   # 128 tokens: still two pages
    assert m.extend(s0, 1) == 128 and g.pool.n_held == 4
    m.check()
    with pytest.raises(CacheError, match="context limit"):
        m.extend(s1, 64 * 6)
    m.give_back_slot(s0)
    with pytest.raises(CacheError, match="not held"):
        m.give_back_slot(s0)
    with pytest.raises(CacheError, match="not held"):
        m.extend(s0, 1)
    assert g.pool.n_held == 1
    s2 = m.take_slot()
    assert s2 == s0 and m.lengths[s2] == 0  # the slot is used again, empty
    m.check()


def test_full_cache_fails_cleanly_and_leaves_nothing_held():
    m = manager(n_tokens=64 * 4, ctx=64 * 4)
    a, b = m.take_slot(), m.take_slot()
    m.extend(a, 64 * 3)
    with pytest.raises(CacheError, match="full"):
        m.extend(b, 65)
    m.check()
    assert m.lengths[b] == 0 and all(g.pool.n_held == 3 for g in m.groups.values())
    m.extend(b, 64)
    m.check()


def test_window_group_gives_pages_back():
    m = manager(window=100)
    win = m.groups[KVRequest(2, 16, 100).key]
    full = m.groups[KVRequest(2, 16).key]
    s = m.take_slot()
    m.extend(s, 300)
    m.after_step(s)
    # the next query, at 300, sees keys >= 201: pages 0..2 are dead
    assert win.pool.n_held == 2 and full.pool.n_held == 5
    assert list(win.block_table[s, :3]) == [-1, -1, -1]
    m.extend(s, 1)
    m.after_step(s)
    m.check()
    m.give_back_slot(s)
    m.check()
    assert win.pool.n_held == 0 and full.pool.n_held == 0


def test_random_walk_keeps_invariants():
    rnd = random.Random(0)
    m = manager(n_tokens=64 * 40, ctx=64 * 8, window=90)
    live = []
    for _ in range(600):
        op = rnd.random()
        try:
            if op < 0.25 and m.n_free_slots:
                live.append(m.take_slot())
            elif op < 0.8 and live:
                s = rnd.choice(live)
                m.extend(s, rnd.choice([1, 1, 1, 17, 64, 130]))
                m.after_step(s)
            elif live:
                s = live.pop(rnd.randrange(len(live)))
                m.give_back_slot(s)
        except CacheError as e:
            assert "full" in str(e) or "context limit" in str(e)
        m.check()
    for s in live:
        m.give_back_slot(s)
    m.check()
    assert all(g.pool.n_held == 0 for g in m.groups.values()) and m.n_free_slots == m.max_slots


def test_sizing_from_max_tokens():
    m = CacheManager(1000, 10 ** 6)
    assert m.n_pages == 16 and m.max_seq_len == 16 * PAGE and m.max_slots == 16

"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; shared prefixes are counted; slots come back."""
import random

import pytest

from tensorline_b200.cache import CacheError, CacheManager, PagedKV, PagePool, SlotState, page_hash


def test_pool_refcount_lru_and_eviction():
    """The scenario of tzar-beep/Tensorline's tests/test_prefix_cache.py:8-22."""
    a = PagePool(4)
    x = a.take(2)
    h0 = page_hash(None, [1, 2])
    a.publish(x[0], h0, None, [1, 2])
    a.drop(x)
    assert a.num_free == 4 and a.num_cached == 1            # freed but still published
    assert a.adopt(h0, None, [1, 2]) == x[0] and a.num_free == 3
    assert a.adopt(h0) == x[0]                             # shared: count 2
    a.drop([x[0]])
    assert a.num_free == 3
    a.drop([x[0]])
    assert a.num_free == 4
    a.take(4)                                           # pressure evicts it
    assert a.num_cached == 0 and a.adopt(h0) is None
    a.check()


def test_hash_chains_over_the_whole_prefix_and_hits_are_verified():
    assert page_hash(page_hash(None, [1]), [2]) != page_hash(page_hash(None, [9]), [2])
    a = PagePool(2)
    (p,) = a.take(1)
    h = page_hash(None, [4, 5])
    a.publish(p, h, None, [4, 5])
    assert a.adopt(h, None, [4, 6]) is None                # same hash claimed, other tokens: a miss


def test_double_free_and_foreign_pages_raise():
    a = PagePool(3)
    x = a.take(1)
    a.drop(x)
    with pytest.raises(CacheError, match="double free"):
        a.drop(x)
    with pytest.raises(CacheError, match="outside"):
        a.drop([7])
    assert a.take(4) is None and a.num_free == 3        # all or nothing


def _manager(window=None, pages=12, page=4, seqs=4, sharing=True, state=False):
    needs = {0: PagedKV(2, 16, None), 1: PagedKV(2, 16, window), 2: PagedKV(1, 8, window)}
    if state:
        needs[3] = SlotState((5,), "float32")
    return CacheManager(needs, page_size=page, num_pages=pages, max_num_seqs=seqs, max_model_len=4 * pages * page,
                        prefix_caching=sharing)


def test_groups_by_need_and_table_rows():
    m = _manager(window=6)
    assert len(m.groups) == 2 and m.groups[0].window is None and m.groups[1].window == 6
    assert m.group_of == {0: 0, 1: 1, 2: 1}
    assert m.prefix_caching                                 # window groups share prefixes too
    assert m.admit("r") == 0 and m.grow("r", 0, 9)
    assert len(m.pages("r", 0)) == 3 and len(m.pages("r", 1)) == 3
    slot = m.slot("r")
    assert list(m.groups[0].table[slot, :3]) == m.pages("r", 0)
    assert m.groups[0].table[slot, 3] == m.groups[0].scratch_page
    m.check()


def test_window_gives_pages_back_and_they_are_used_again():
    m = _manager(window=6, pages=5)
    m.admit("a")
    assert m.grow("a", 0, 8)
    m.advance("a", 8, None)               # next query at 8 reads keys >= 3: page 0 (keys 0..3) is still needed
    assert m.pages("a", 1)[0] >= 0
    assert m.grow("a", 8, 12)
    m.advance("a", 12, None)              # next query at 12 reads keys >= 7: page 0 is behind the window
    assert m.pages("a", 1)[0] == -1 and m.pages("a", 0)[0] >= 0
    assert m.num_free_pages(1) == 5 - 2 and m.num_free_pages(0) == 5 - 3
    m.check()
    for upto in range(13, 21):            # the full group runs out at 20 tokens, the window group never does
        ok = m.grow("a", upto - 1, upto)
        m.advance("a", upto, None) if ok else None
    assert ok and not m.grow("a", 20, 21)
    assert m.num_free_pages(1) >= 2
    m.release("a")
    assert m.num_free_pages(0) == 5 and m.num_free_pages(1) == 5 and m.num_free_slots == 4
    with pytest.raises(CacheError, match="double release"):
        m.release("a")


def test_prefix_sharing_counts_and_fully_cached_prompt():
    m = CacheManager({0: PagedKV(1, 16)}, page_size=4, num_pages=8, max_num_seqs=3, max_model_len=32)
    toks = list(range(100, 112))
    assert m.admit("a", toks) == 0 and m.grow("a", 0, 12)
    m.advance("a", 12, toks)                                 # three full pages published
    assert m.admit("b", toks + [1, 2]) == 12                 # shares all three
    assert m.pages("b") == m.pages("a")
    assert m.admit("c", toks) == 8                           # fully cached: the last page is recomputed
    m.check()
    m.release("a")
    m.check()
    assert m.num_free_pages() == 5                           # still held by b (3 pages) and c (2 of them)
    m.release("b"); m.release("c")
    assert m.num_free_pages() == 8
    assert m.admit("d", toks[:8] + [7, 7, 7, 7]) == 8        # freed pages stay matchable until evicted
    m.check()


def test_window_group_shares_the_pages_its_window_still_reaches():
    """Two groups, all keys and a window of 6 keys, pages of 4.  A request whose first 12 tokens are
    published takes, in the window group, only the pages a query at position 12 can read (keys 7..11:
    pages 1 and 2); if one of those has been used up meanwhile the hit shrinks to what both groups serve."""
    needs = {0: PagedKV(1, 16, None), 1: PagedKV(1, 16, 6)}
    m = CacheManager(needs, page_size=4, num_pages={None: 8, 6: 4}, max_num_seqs=3, max_model_len=32)
    assert m.groups[0].pool.num_pages == 8 and m.groups[1].pool.num_pages == 4
    toks = list(range(50, 64))
    assert m.admit("a", toks) == 0 and m.grow("a", 0, 14)
    m.advance("a", 14, toks)                                # three full pages offered in both groups
    wa = m.pages("a", 1)                                    # a's next query (14) reads keys 9..: pages 0, 1 are passed
    assert wa[:2] == [-1, -1] and wa[2] >= 0
    assert m.admit("b", toks[:12] + [1, 2, 3]) == 12
    assert m.pages("b", 0) == m.pages("a", 0)[:3]
    wb = m.pages("b", 1)                                    # page 1 is revived from the idle ones, page 2 is shared with a
    assert wb[0] == -1 and wb[1] >= 0 and wb[2] == wa[2] and m.groups[1].pool.refcount(wb[2]) == 2
    slot = m.slot("b")
    assert m.groups[1].table[slot, 0] == m.groups[1].scratch_page
    m.check()
    m.release("a"); m.release("b")
    assert m.num_free_pages(0) == 8 and m.num_free_pages(1) == 4
    # the window group's pool is used up by someone else: its published pages are gone, the full group's are not
    assert m.admit("c") == 0 and m.grow("c", 0, 4)
    m.release("c")                                          # took the window group's longest-idle page: page 0 of a
    assert m.admit("d", toks[:12] + [9]) == 12              # page 0 is not needed at position 12
    m.release("d")
    assert m.admit("e") == 0 and m.grow("e", 0, 16)          # now every page of the window group is rewritten
    m.release("e")
    assert m.admit("f", toks[:12] + [9]) == 0               # the full group alone cannot restore the prefix
    m.check()


@pytest.mark.parametrize("window,sharing,state,seed", [(None, True, True, 0), (None, False, True, 1), (7, True, False, 2),
                                                        (3, False, True, 3), (None, True, False, 4), (5, True, False, 5)])
def test_random_orders_never_lose_a_page(window, sharing, state, seed):
    rng = random.Random(seed)
    m = _manager(window=window, pages=10, page=4, seqs=3, sharing=sharing, state=state)
    assert m.prefix_caching == (sharing and not state)
    live = {}                                                # rid -> [tokens, computed]
    prompts = [[rng.randrange(5) for _ in range(rng.randrange(1, 30))] for _ in range(6)]
    nxt = 0
    for it in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 3:
            rid = f"r{nxt}"; nxt += 1
            toks = list(rng.choice(prompts))
            cached = m.admit(rid, toks)
            assert cached is not None and cached % 4 == 0 and cached < len(toks)
            live[rid] = [toks, cached]
        elif op < 0.8 and live:
            rid = rng.choice(sorted(live))
            toks, done = live[rid]
            if done == len(toks):
                toks.append(rng.randrange(5))
            n = rng.randrange(1, len(toks) - done + 1)
            if done + n <= 40 and m.grow(rid, done, done + n):
                live[rid][1] = done + n
                m.advance(rid, done + n, toks)
            # a refusal must leave everything as it was
        elif live:
            rid = rng.choice(sorted(live))
            m.release(rid)
            del live[rid]
        m.check()
        for g in m.groups:
            held = sum(1 for rid in live for p in m.pages(rid, g.index) if p >= 0)
            assert held >= g.pool.num_pages - g.pool.num_free      # shared pages are counted once in the pool
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups) and m.num_free_slots == 3


def test_slots_are_exclusive_and_return():
    m = _manager(seqs=2)
    assert m.admit("a") == 0 and m.admit("b") == 0
    assert m.slot("a") != m.slot("b") and m.admit("c") is None
    with pytest.raises(CacheError, match="already admitted"):
        m.admit("a")
    m.release("a")
    assert m.admit("c") == 0 and m.slot("c") != m.slot("b")
    assert 3 not in m.group_of and m.padding_slot == 2

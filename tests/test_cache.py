"""The cache's bookkeeping (CPU): no page or slot lost, held twice or freed twice."""
import random

import pytest
import torch

from turboquant_cpp_b200.cache import CacheBook, CacheFull, CacheMisuse, IndexPool, PagedCache
from turboquant_cpp_b200.parts import KVNeed, StateNeed


def test_pool_gives_each_index_once_and_takes_it_back_once():
    p = IndexPool(4, "page")
    got = [p.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        p.take()
    p.give_back(got[1])
    with pytest.raises(CacheMisuse):
        p.give_back(got[1])                      # freed twice
    with pytest.raises(CacheMisuse):
        p.give_back(17)
    assert p.take() == got[1]                    # used again


def test_sequences_reserve_commit_close():
    book = CacheBook([8, 8], [0, 0], page_size=64, max_slots=3)
    a, b = book.open(), book.open()
    assert a.slot != b.slot
    book.reserve_all([a, b], [70, 1])
    assert [len(x) for x in a.pages] == [2, 2] and [len(x) for x in b.pages] == [1, 1]
    book.commit(a, 70)
    book.commit(b, 1)
    book.reserve(a, 58)                          # 70 + 58 = 128: still two pages
    assert len(a.pages[0]) == 2
    book.commit(a, 58)
    book.reserve(a, 1)
    assert len(a.pages[0]) == 3
    book.check_invariants()
    book.close(a)
    with pytest.raises(CacheMisuse):
        book.close(a)                            # closed twice
    with pytest.raises(CacheMisuse):
        book.reserve(a, 1)
    book.close(b)
    book.check_invariants()
    assert all(p.n_free == 8 for p in book.pools) and book.slots.n_free == 3


def test_reserve_all_is_all_or_nothing():
    book = CacheBook([3], [0], page_size=64, max_slots=4)
    a, b = book.open(), book.open()
    with pytest.raises(CacheFull):
        book.reserve_all([a, b], [128, 128])     # 4 pages wanted, 3 there
    assert book.pools[0].n_free == 3 and not a.pages[0] and not b.pages[0]
    book.reserve_all([a, b], [128, 64])
    assert book.pools[0].n_free == 0
    c = book.open()
    with pytest.raises(CacheFull):
        book.reserve(c, 1)
    with pytest.raises(CacheFull):
        [book.open() for _ in range(2)]          # slots run out too
    book.check_invariants()


def test_windowed_group_gives_old_pages_back():
    book = CacheBook([10, 10], [0, 32], page_size=64, max_slots=2)
    s = book.open()
    book.reserve(s, 200)
    book.commit(s, 200)                          # later queries see positions >= 201 - 32 = 169: pages 0, 1 go
    assert [p is None for p in s.pages[1]] == [True, True, False, False]
    assert all(p is not None for p in s.pages[0])
    assert book.pools[1].n_free == 8 and book.pools[0].n_free == 6
    book.reserve(s, 100)
    book.commit(s, 100)                          # 300 tokens: positions >= 269: pages 0..3 gone
    assert [p is None for p in s.pages[1]] == [True] * 4 + [False]
    book.check_invariants()
    book.close(s)
    assert book.pools[1].n_free == 10


def test_random_walk_keeps_the_books():
    rng = random.Random(0)
    book = CacheBook([40, 40], [0, 100], page_size=64, max_slots=6)
    live = []
    for _ in range(2000):
        r = rng.random()
        try:
            if r < 0.2 and len(live) < 6:
                live.append(book.open())
            elif r < 0.8 and live:
                s = rng.choice(live)
                n = rng.choice([1, 1, 1, 5, 64, 130])
                book.reserve(s, n)
                book.commit(s, n)
            elif live:
                book.close(live.pop(rng.randrange(len(live))))
        except CacheFull:
            if live:
                book.close(live.pop(0))
        book.check_invariants()
    for s in live:
        book.close(s)
    assert all(p.n_free == p.n for p in book.pools) and book.slots.n_free == 6


def test_paged_cache_groups_state_and_tables():
    full, win = KVNeed(2, 16, 0), KVNeed(2, 16, 32)
    needs = [full, win, None, win, full]          # entry 2 keeps no keys; entry 4 reads entry 0's cache
    state = [None, None, StateNeed((3, 4)), None, None]
    cache = PagedCache(needs, state, [None, None, None, None, 0], max_tokens=640, dtype=torch.float32, device="cpu",
                       max_slots=4)
    assert cache.groups == [full, win] and cache.entry_group == [0, 1, None, 1, 0]
    assert cache.kv[4] is cache.kv[0] and cache.kv[2] is None
    assert cache.kv[0].shape == (10, 2, 2, 64, 16) and cache.kv[1] is not cache.kv[3]
    assert cache.state[2].shape == (4, 3, 4)
    a = cache.open()
    cache.state[2][a.slot] += 1.0
    cache.reserve([a], [130])
    cache.commit([a], [130])
    t = cache.page_tables([a])
    assert t[0].shape == (1, 3) and (t[0] >= 0).all()
    assert t[1].tolist()[0][0] == -1 and t[1].tolist()[0][2] >= 0      # window 32: page 0 was given back
    lc = cache.layer_caches([torch.from_numpy(x) for x in t])
    assert lc[4].writes is False and lc[0].writes is True and lc[2].kv is None and lc[2].state is cache.state[2]
    slot = a.slot
    cache.close(a)
    b = cache.open()
    assert b.slot == slot and float(cache.state[2][slot].abs().sum()) == 0.0     # the slot is used again, zeroed
    assert cache.bytes_per_token() == 3 * 2 * 2 * 16 * 4      # three entries keep keys and values

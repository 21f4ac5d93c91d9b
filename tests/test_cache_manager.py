"""The cache manager on its own: pages, block tables, groups, slots."""
import random

import pytest
import torch

from ferrox_b200.cache.manager import CacheError, CacheManager
from ferrox_b200.cache.specs import CacheSpec, KvCacheSpec, StateSpec


def manager(n_pages=8, page_size=4, window=6, max_slots=3, with_state=True):
    specs = [
        CacheSpec(paged=KvCacheSpec(2, 8, None)),
        CacheSpec(paged=KvCacheSpec(1, 16, window), state=StateSpec((5,)) if with_state else None),
        CacheSpec(paged=KvCacheSpec(2, 8, None)),
        None,
    ]
    return CacheManager(specs, page_size=page_size, n_pages=n_pages, max_slots=max_slots, max_positions=64,
                        device="cpu", dtype=torch.float32)


def test_pool_is_all_or_nothing_and_lifo():
    m = manager(n_pages=4, page_size=4, window=64, max_slots=3)
    a, b = m.open_request(), m.open_request()
    assert m.reserve(a, 12) and m.held_pages(a)[None] == [0, 1, 2] and m.free_pages()[None] == 1
    assert m.reserve(b, 8) is False and m.free_pages()[None] == 1  # nothing taken on failure
    m.close_request(a)
    assert m.reserve(b, 4) and m.held_pages(b)[None] == [2]  # most recently freed first (a's pages went back 0, 1, 2)
    with pytest.raises(CacheError):
        m.close_request(a)  # freed twice
    with pytest.raises(CacheError):
        m.reserve(7, 4)  # never opened
    m.check_invariants()


def test_groups_by_need_and_shapes():
    m = manager()
    assert set(m.groups) == {None, 6}
    assert m.groups[None].caches == [0, 2] and m.groups[6].caches == [1]
    assert m.layer_cache(0).k.shape == (8, 2, 4, 8) and m.layer_cache(1).v.shape == (8, 1, 4, 16)
    assert m.layer_cache(1).state.shape == (3, 5) and m.layer_cache(0).state is None
    assert m.layer_cache(3).k is None and m.layer_cache(3).block_table is None
    assert m.layer_cache(0).block_table is m.layer_cache(2).block_table  # one table per group


def test_reserve_commit_release_and_window():
    m = manager(n_pages=8, page_size=4, window=6)
    s = m.open_request()
    assert m.reserve(s, 10)  # 3 pages in both groups
    assert m.held_pages(s) == {None: [0, 1, 2], 6: [0, 1, 2]}
    m.commit(s, 10)  # next query at 10 reads from 5 on: page 0 (0..3) is out, page 1 (4..7) still needed
    assert m.held_pages(s) == {None: [0, 1, 2], 6: [1, 2]}
    assert m.groups[6].table[s, 0] == -1
    m.check_invariants()
    assert m.reserve(s, 17) and m.held_pages(s)[6] == [1, 2, 0, 3]  # the freed page is used again
    m.commit(s, 17)  # reads from 12 on: pages 0..2 out
    assert m.held_pages(s)[6] == [0, 3] and m.held_pages(s)[None] == [0, 1, 2, 3, 4]
    m.check_invariants()
    m.close_request(s)
    assert m.free_pages() == {None: 8, 6: 8}
    m.check_invariants()
    with pytest.raises(CacheError):
        m.close_request(s)


def test_exhaustion_changes_nothing():
    m = manager(n_pages=4, page_size=4)
    a, b = m.open_request(), m.open_request()
    assert m.reserve(a, 12)
    before = (m.free_pages(), m.held_pages(b), m.groups[None].table.copy())
    assert m.reserve(b, 8) is False
    assert (m.free_pages(), m.held_pages(b)) == before[:2] and (m.groups[None].table == before[2]).all()
    assert m.reserve(b, 4)
    m.check_invariants()
    with pytest.raises(CacheError):
        m.reserve(a, 65)  # beyond max_positions


def test_slots_and_state():
    m = manager(max_slots=2)
    a, b = m.open_request(), m.open_request()
    assert m.open_request() is None
    m.layer_cache(1).state[a] += 3.0
    m.close_request(a)
    c = m.open_request()
    assert c == a and float(m.layer_cache(1).state[c].abs().sum()) == 0.0  # slot reused, state zeroed
    assert b != c


def test_tables_reach_the_device_copy():
    m = manager()
    s = m.open_request()
    m.reserve(s, 9)
    m.sync_tables()
    assert m.layer_cache(0).block_table[s, :3].tolist() == [0, 1, 2]
    m.commit(s, 9)
    m.sync_tables()
    assert m.layer_cache(1).block_table[s, 0].item() == -1
    m.close_request(s)
    m.sync_tables()
    assert (m.layer_cache(0).block_table[s] == -1).all()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(n_pages=rng.choice([6, 9, 16]), page_size=rng.choice([1, 2, 4, 8]), window=rng.choice([3, 6, 17]),
                max_slots=4)
    live = {}
    for _ in range(400):
        op = rng.random()
        if op < 0.2 and m.n_free_slots:
            live[m.open_request()] = 0
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            new_len = min(64, live[s] + rng.randint(1, 9))
            if new_len > live[s] and m.reserve(s, new_len):
                m.commit(s, new_len)
                live[s] = new_len
                # every position the next query may read is mapped
                for key, g in m.groups.items():
                    lo = 0 if key is None else max(0, new_len - key + 1)
                    for pos in range(lo, new_len):
                        assert g.table[s, pos // m.page_size] >= 0
        elif live:
            s = rng.choice(list(live))
            m.close_request(s)
            del live[s]
        m.check_invariants()
    for s in list(live):
        m.close_request(s)
    m.check_invariants()
    assert all(n == m.groups[k].pool.n_pages for k, n in m.free_pages().items())


def test_a_whole_step_is_reserved_for_all_requests_or_for_none():
    """The step function's one call: several requests grow together; if the pages do not suffice for all of them,
    none gets any; the lengths advance only at commit, and a windowed group then lets go of what fell out."""
    m = manager(n_pages=6, page_size=4, window=6, max_slots=3)
    a, b, c = m.open_request(), m.open_request(), m.open_request()
    assert m.reserve_step([a, b], [9, 4]) == [0, 0]          # 3 + 1 pages in both groups
    assert m.free_pages() == {None: 2, 6: 2} and m.seq_len[a] == 0
    m.commit_step([a, b], [9, 4])
    assert (m.seq_len[a], m.seq_len[b]) == (9, 4)
    assert m.held_pages(a) == {None: [0, 1, 2], 6: [1, 2]}   # the next query at 9 reads from 4 on
    before = (m.free_pages(), m.held_pages(a), m.held_pages(b), m.held_pages(c))
    # a needs 1 page more, b 1, c 2: four pages where the full group has two free
    assert m.reserve_step([a, b, c], [4, 4, 5]) is None
    assert before == (m.free_pages(), m.held_pages(a), m.held_pages(b), m.held_pages(c))
    assert m.reserve_step([a, b], [4, 4]) == [9, 4]
    m.commit_step([a, b], [4, 4])
    assert (m.seq_len[a], m.seq_len[b]) == (13, 8) and m.free_pages()[None] == 0
    with pytest.raises(CacheError):
        m.reserve_step([a, 7], [1, 1])                        # a slot no request holds
    m.check_invariants()
    for s in (a, b, c):
        m.close_request(s)
    assert m.free_pages() == {None: 6, 6: 6}
    m.check_invariants()

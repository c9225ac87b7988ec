import random

import numpy as np
import pytest
import torch

from rosellm_b200.cache import CacheManager, DoubleFree, IdAllocator
from rosellm_b200.parts import KVCacheSpec, StateSpec


def test_allocator_all_or_nothing_and_lifo():
    a = IdAllocator(4)
    got = a.alloc(3)
    assert got == [0, 1, 2] and a.num_free == 1
    assert a.alloc(2) is None and a.num_free == 1  # nothing taken on failure
    a.free([1])
    assert a.alloc(1) == [1]  # freed last, handed out next
    with pytest.raises(DoubleFree):
        a.free([3])
    a.free([0, 1, 2])
    with pytest.raises(DoubleFree):
        a.free([2])
    a.check()
    assert a.num_free == 4


def manager(window=None, pages=12, page=4, slots=4, seq=64, two_groups=False, state=False):
    kv = {0: KVCacheSpec(2, 16, None), 1: KVCacheSpec(2, 16, window if two_groups else None)}
    if not two_groups and window is not None:
        kv = {0: KVCacheSpec(2, 16, window), 1: KVCacheSpec(2, 16, window)}
    st = {1: StateSpec((3,), torch.float32)} if state else {}
    return CacheManager(kv, st, page_size=page, num_pages=pages, max_slots=slots, max_seq_len=seq, device="cpu")


def test_reserve_commit_release_and_reuse():
    m = manager()
    assert len(m.groups) == 1 and m.groups[0].layers == [0, 1]
    s = m.new_request()
    assert m.reserve(s, 9) and m.pages_of(s) == [0, 1, 2]
    m.commit(s, 9)
    assert m.reserve(s, 3) and m.pages_of(s) == [0, 1, 2]  # 12 tokens still fit three pages
    m.commit(s, 3)
    assert m.reserve(s, 1) and len(m.pages_of(s)) == 4
    m.commit(s, 1)
    s2 = m.new_request()
    assert not m.reserve(s2, 40) and m.pages_of(s2) == [] and m.num_free_pages == 8
    m.check()
    m.release(s)
    assert m.num_free_pages == 12
    assert m.reserve(s2, 4) and m.pages_of(s2) == [3]  # the page given back last
    with pytest.raises(ValueError):
        m.release(s)
    with pytest.raises(ValueError):
        m.reserve(s2, 1000)
    m.check()


def test_window_group_gives_pages_back_while_the_request_lives():
    m = manager(window=6, two_groups=True, pages=40)
    assert len(m.groups) == 2
    full, win = (0, 1) if m.groups[0].spec.window is None else (1, 0)
    s = m.new_request()
    for n in (5, 1, 1, 7, 2, 1, 1, 1, 9, 1):
        assert m.reserve(s, n)
        m.commit(s, n)
        m.check()
        cur = int(m.num_tokens[s])
        assert len(m.pages_of(s, full)) == -(-cur // 4)
        first_needed = max(0, cur - 6 + 1) // 4
        assert m.pages_of(s, win) == [int(p) for p in m.groups[win].table[s, first_needed:-(-cur // 4)]]
        assert all(p < 0 for p in m.groups[win].table[s, :first_needed])
    assert len(m.pages_of(s, win)) <= 3
    m.release(s)
    assert all(g.allocator.num_free == 40 for g in m.groups)


def test_state_slots_are_reset_for_a_new_request():
    m = manager(state=True)
    s = m.new_request()
    m.sync_to_device()
    m.state(1)[s] = 7.0
    m.release(s)
    s2 = m.new_request()
    assert s2 == s
    m.sync_to_device()
    assert float(m.state(1)[s2].abs().sum()) == 0.0
    assert m.state(1).shape == (4, 3)


def test_block_table_reaches_the_device_copy():
    m = manager()
    s = m.new_request()
    m.reserve(s, 10)
    m.sync_to_device()
    assert m.block_table(0)[s, :3].tolist() == m.pages_of(s)
    m.commit(s, 10)
    m.release(s)
    m.sync_to_device()
    assert (m.block_table(0)[s] == -1).all()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_lose_and_double_nothing(seed, window):
    rng = random.Random(seed)
    m = manager(window=window, pages=24, page=4, slots=5, seq=80, two_groups=window is not None)
    live: dict[int, int] = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 5:
            s = m.new_request()
            assert s is not None and s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 16])
            if live[s] + n > 80:
                continue
            before = [g.allocator.num_free for g in m.groups]
            if m.reserve(s, n):
                m.commit(s, n)
                live[s] += n
            else:
                assert [g.allocator.num_free for g in m.groups] == before  # all or nothing
        elif live:
            s = rng.choice(list(live))
            m.release(s)
            del live[s]
        m.check()
        assert all(int(m.num_tokens[s]) == n for s, n in live.items())
    for s in list(live):
        m.release(s)
    m.check()
    assert all(g.allocator.num_free == 24 for g in m.groups) and m.num_free_slots == 5
    assert m.new_request() is not None

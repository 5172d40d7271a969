"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""
import random

import pytest

from cuca_b200.cache.pages import (NO_BLOCK, BlockPool, CacheBookkeepingError, GroupLayout, KvPools, PoolExhausted,
                                   StateSlots)


def pools(n_full=12, n_win=6, window=20, bs=16):
    groups = [GroupLayout(2, 16, None, (0, 2), n_full), GroupLayout(2, 16, window, (1,), n_win)]
    return KvPools(groups, bs)


def test_reserve_is_all_or_nothing_and_release_returns_everything():
    kv = pools(n_full=4, n_win=4)
    a, b = kv.new_seq(), kv.new_seq()
    kv.reserve(a, 33)  # 3 pages in each group
    assert [len(t) for t in a.tables] == [3, 3] and kv.owed(a, 48) == [0, 0] and kv.owed(a, 49) == [1, 1]
    with pytest.raises(PoolExhausted):
        kv.reserve(b, 17)  # needs 2, only 1 left: nothing may be taken
    assert [len(t) for t in b.tables] == [0, 0] and [p.free for p in kv.pools] == [1, 1]
    kv.check()
    kv.release(a)
    kv.reserve(b, 64)
    kv.check()
    kv.release(b)
    assert [p.free for p in kv.pools] == [4, 4]
    with pytest.raises(CacheBookkeepingError):
        kv.release(b)


def test_double_free_is_caught():
    p = BlockPool(3)
    b = p.alloc()
    p.release(b)
    with pytest.raises(CacheBookkeepingError):
        p.release(b)
    with pytest.raises(CacheBookkeepingError):
        p.release(7)


def test_pages_are_used_again_last_freed_first():
    kv = pools()
    a = kv.new_seq()
    kv.reserve(a, 16)
    first = a.tables[0][0]
    kv.release(a)
    b = kv.new_seq()
    kv.reserve(b, 16)
    assert b.tables[0][0] == first


def test_window_gives_pages_back_as_it_passes_them():
    kv = pools(n_full=12, n_win=6, window=20, bs=16)
    s = kv.new_seq()
    kv.reserve(s, 64)
    s.length = 64
    freed = kv.release_window(s)
    # next query at 64 sees keys >= 45: pages 0 and 1 (positions 0..31) are behind the window
    assert freed == 2 and s.tables[1][:2] == [NO_BLOCK, NO_BLOCK] and s.tables[1][2] != NO_BLOCK
    assert all(b != NO_BLOCK for b in s.tables[0])  # the full group keeps everything
    assert kv.release_window(s) == 0
    kv.check()
    kv.reserve(s, 96)
    s.length = 96
    assert kv.release_window(s) == 2
    kv.check()
    kv.release(s)
    assert [p.free for p in kv.pools] == [12, 6]


def test_truncate_rolls_back_and_marks_tables_dirty():
    kv = pools()
    s = kv.new_seq()
    kv.reserve(s, 50)
    s.length = 50
    s.dirty_from = [4, 4]
    kv.truncate(s, 20)
    assert [len(t) for t in s.tables] == [2, 2] and s.length == 20 and s.dirty_from == [2, 2]
    kv.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_a_page(seed):
    rng = random.Random(seed)
    kv = pools(n_full=40, n_win=14, window=rng.choice([5, 20, 47]), bs=rng.choice([8, 16]))
    slots = StateSlots(6)
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and slots.free:
            live.append((kv.new_seq(), slots.alloc()))
        elif op < 0.75 and live:
            seq, _ = rng.choice(live)
            grow = rng.choice([1, 1, 1, 2, 7, 33])
            try:
                kv.reserve(seq, seq.length + grow)
                seq.length += grow
                kv.release_window(seq)
            except PoolExhausted:
                victim = live.pop(rng.randrange(len(live)))
                kv.release(victim[0])
                slots.release(victim[1])
        elif op < 0.85 and live:
            seq, _ = rng.choice(live)
            kv.truncate(seq, rng.randint(0, seq.length))
        elif live:
            seq, slot = live.pop(rng.randrange(len(live)))
            kv.release(seq)
            slots.release(slot)
        kv.check()
        held = sum(1 for s, _ in live for b in s.tables[0] if b != NO_BLOCK)
        assert kv.pools[0].used == held
    for seq, slot in live:
        kv.release(seq)
        slots.release(slot)
    kv.check()
    assert [p.free for p in kv.pools] == [40, 14] and slots.free == 6


def test_reset_frees_everything():
    kv = pools(n_full=12, n_win=12)
    for n in (10, 40, 70):
        s = kv.new_seq()
        kv.reserve(s, n)
    kv.reset()
    kv.check()
    assert [p.free for p in kv.pools] == [12, 12]


def test_state_slots_are_handed_out_once():
    s = StateSlots(3)
    got = [s.alloc(), s.alloc(), s.alloc()]
    assert sorted(got) == [0, 1, 2] and s.alloc() is None
    s.release(got[1])
    assert s.alloc() == got[1]
    with pytest.raises(CacheBookkeepingError):
        s.release(5)
    s.release(got[0])
    with pytest.raises(CacheBookkeepingError):
        s.release(got[0])

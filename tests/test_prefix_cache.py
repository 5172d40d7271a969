"""The prefix store of the cache manager and the scheduler's use of it, without a GPU
(behaviour of src/provider/local/model/paged.rs:18-35,344-480,831-928 and engine/scheduler.rs:793-896)."""
import random

import pytest

from cuca_b200.cache.pages import NO_BLOCK, GroupLayout, KvPools, PoolExhausted, StateSlots
from cuca_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from tests.test_scheduler import FakeBackend


def pools(n_blocks=8, bs=4, window=None):
    groups = [GroupLayout(2, 16, None, (0,), n_blocks)]
    if window:
        groups.append(GroupLayout(1, 16, window, (1,), n_blocks))
    return KvPools(groups, bs)


def test_finished_pages_are_found_by_the_next_prompt_with_the_same_head():
    kv = pools()
    ids = list(range(100, 114))                  # 14 tokens: three full pages of 4 and two more positions
    a = kv.new_seq()
    kv.reserve(a, 14)
    a.length = 14
    pages = a.tables[0]
    kv.finish(a, ids)
    assert a.released and kv.pools[0].cached == 3 and kv.pools[0].free == 8    # cached pages can still be taken
    # same first 9 tokens: two whole pages are shared (9 - 1 = 8 positions)
    b = kv.new_seq_with_prefix(ids[:9])
    assert b.length == 8 and b.tables[0] == pages[:2] and kv.pools[0].cached == 1
    # the whole prompt again: at most len - 1 positions, in whole pages
    c = kv.new_seq_with_prefix(ids[:12])
    assert c.length == 8 and c.tables[0] == pages[:2]                           # page 2 would end at the last token
    d = kv.new_seq_with_prefix(ids[:13])
    assert d.length == 12 and d.tables[0] == pages[:3] and kv.pools[0].cached == 0
    # another head: nothing is shared; a different token inside the first page breaks the chain at once
    e = kv.new_seq_with_prefix([100, 101, 999, 103] + ids[4:12])
    assert e.length == 0 and e.tables[0] == []
    kv.check()
    for s in (b, c, d, e):
        kv.release(s)
    kv.check()
    assert kv.pools[0].cached == 3 and kv.stats()["live_requests"] == 0


def test_shared_pages_are_not_written_and_survive_their_first_owner():
    kv = pools()
    ids = list(range(40, 52))
    a = kv.new_seq()
    kv.reserve(a, 12)
    a.length = 12
    kv.publish(a, ids)                           # a keeps running: its full pages are named already
    b = kv.new_seq_with_prefix(ids[:9] + [7, 7, 7])
    assert b.length == 8 and b.tables[0] == a.tables[0][:2]
    kv.reserve(b, 12)
    assert b.tables[0][2] not in a.tables[0]     # b appends in a page of its own
    kv.release(a)
    kv.check()
    assert kv.pools[0].cached == 1               # a's third page: named, unreferenced; the shared two are b's now
    kv.truncate(b, 6)                            # the end falls into a named page: only whole pages are kept
    assert b.length == 4 and len(b.tables[0]) == 1
    kv.release(b)
    kv.check()


def test_allocation_evicts_the_least_recently_used_cached_page_and_forgets_its_name():
    kv = pools(n_blocks=4)
    first, second = list(range(8)), list(range(50, 58))
    for ids in (first, second):
        s = kv.new_seq()
        kv.reserve(s, 8)
        s.length = 8
        kv.finish(s, ids)
    assert kv.pools[0].cached == 4 and kv.pools[0].free == 4
    big = kv.new_seq()
    kv.reserve(big, 9)                           # three pages: the two of `first` and the older one of `second` go
    assert kv.pools[0].cached == 1
    assert kv.new_seq_with_prefix(first + [1]).length == 0
    hit = kv.new_seq_with_prefix(second + [1])
    assert hit.length == 0                       # its first page is gone, so the chain cannot start
    with pytest.raises(PoolExhausted):
        kv.reserve(big, 4 * 4 + 1)
    kv.check()


def test_windowed_group_needs_only_the_pages_of_its_window():
    kv = pools(n_blocks=16, window=6)
    ids = list(range(200, 220))
    a = kv.new_seq()
    kv.reserve(a, 20)
    a.length = 20
    kv.release_window(a)                         # the next query (position 20) sees keys >= 15: pages 0..2 are passed
    assert a.tables[1][:3] == [NO_BLOCK] * 3 and a.tables[1][3] != NO_BLOCK
    kv.finish(a, ids)
    b = kv.new_seq_with_prefix(ids + [9])        # 20 positions = 5 pages; the windowed group has pages 3 and 4 of them
    assert b.length == 20 and len(b.tables[0]) == 5
    assert b.tables[1][:3] == [NO_BLOCK] * 3 and b.tables[1][3] != NO_BLOCK and len(b.tables[1]) == 5
    kv.reserve(b, 24)
    kv.check()
    # a shorter prefix would need window pages that are gone (13 tokens: 12 positions, window from 7 on = page 1):
    # it is shortened until every group has what it needs, here to nothing
    c = kv.new_seq_with_prefix(ids[:13])
    assert c.length == 0
    kv.check()


def test_random_orders_keep_the_books_straight():
    rng = random.Random(5)
    kv = pools(n_blocks=24, bs=4)
    heads = [[rng.randrange(50) for _ in range(16)] for _ in range(3)]
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.4:
            prompt = rng.choice(heads)[:rng.randrange(1, 17)] + [rng.randrange(50) for _ in range(rng.randrange(0, 6))]
            s = kv.new_seq_with_prefix(prompt)
            try:
                kv.reserve(s, len(prompt))
            except PoolExhausted:
                kv.release(s)
                continue
            s.length = len(prompt)
            live.append((s, prompt))
        elif live:
            s, prompt = live.pop(rng.randrange(len(live)))
            if op < 0.8:
                kv.finish(s, prompt)
            else:
                kv.release(s)
        kv.check()
    for s, prompt in live:
        kv.finish(s, prompt)
    kv.check()
    assert kv.pools[0].free == 24


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_hits_bring_the_right_tokens_through_heavy_eviction(seed):
    """Hundreds of different prompts through a pool of 32 pages: names are taken out of the pool's name table all
    the time (its probe runs are closed up on removal). The test remembers which tokens every page was last filled
    with: a prefix hit must hand out pages that hold exactly the prompt's tokens, a prompt that was just finished
    must be found whole, and a hit is never longer than what some finished prompt shares with it."""
    rng = random.Random(seed)
    bs, n_blocks = 4, 32
    kv = pools(n_blocks=n_blocks, bs=bs)
    content = {}                                 # page -> the tokens it was last filled with
    finished = []
    stems = [[rng.randrange(9) for _ in range(24)] for _ in range(6)]

    def run(prompt, finish=True):
        s = kv.new_seq_with_prefix(prompt)
        shared = s.length // bs
        assert s.length % bs == 0 and s.length <= len(prompt) - 1
        for i in range(shared):
            assert content[s.tables[0][i]] == tuple(prompt[i * bs:(i + 1) * bs]), "a hit handed out another prompt's page"
        longest = max((next((k for k in range(min(len(f), len(prompt))) if f[k] != prompt[k]), min(len(f), len(prompt)))
                       for f in finished), default=0)
        assert s.length <= longest // bs * bs, "a hit is longer than any finished prompt shares"
        try:
            kv.reserve(s, len(prompt))
        except PoolExhausted:
            kv.release(s)
            return None
        s.length = len(prompt)
        for i in range(shared, len(s.tables[0])):
            content[s.tables[0][i]] = tuple(prompt[i * bs:(i + 1) * bs])
        if finish:
            kv.finish(s, prompt)
            finished.append(list(prompt))
            return None
        return s

    held = []
    for step in range(1500):
        stem = rng.choice(stems)
        prompt = stem[:rng.randrange(1, 25)] + [rng.randrange(9) for _ in range(rng.randrange(0, 9))]
        if rng.random() < 0.15 and len(held) < 3:
            s = run(prompt, finish=False)
            if s is not None:
                held.append((s, prompt))
        else:
            run(prompt)
            if rng.random() < 0.5 and len(prompt) > bs:   # just finished: found whole (below its last token)
                again = kv.new_seq_with_prefix(prompt)
                assert again.length == (len(prompt) - 1) // bs * bs
                kv.release(again)
        if held and rng.random() < 0.3:
            s, prompt = held.pop(rng.randrange(len(held)))
            kv.finish(s, prompt)
            finished.append(list(prompt))
        if step % 50 == 0:
            kv.check()
    for s, prompt in held:
        kv.finish(s, prompt)
    kv.check()
    assert kv.pools[0].free == n_blocks


# ------------------------------------------------------------------ the scheduler's use of it
def make(n_blocks=16, prefix_cache=True):
    kv = KvPools([GroupLayout(2, 16, None, (0,), n_blocks)], 4)
    slots = StateSlots(4)
    be = FakeBackend(kv)
    sch = Scheduler(kv, slots, be, SchedulerConfig(4, 8, 8, 256, (7,), prefix_cache=prefix_cache), seed_source=lambda: 1)
    return sch, be, kv


def test_the_second_request_prefills_only_what_the_first_did_not_leave():
    sch, be, kv = make()
    prompt = list(range(300, 318))               # 18 tokens
    first = sch.submit(Request(prompt, max_tokens=3, temperature=0.0))
    sch.run_until_done()
    rows_first = sum(len(t) for step in be.steps for (_, _, t, _) in step)
    assert rows_first == 18 + 2 and kv.pools[0].cached == 5          # 20 positions cached: five full pages
    be.steps.clear()
    second = sch.submit(Request(prompt, max_tokens=3, temperature=0.0))
    sch.run_until_done()
    # 16 of the 18 prompt tokens were found (whole pages below the last token); two are prefilled
    assert be.steps[0] == [(second.id, 16, prompt[16:], True)]
    assert sch.stats.prefix_hit_tokens == 16 and second.finish_reason == "length" and len(second.completion) == 3
    # a prompt that shares the head and then differs
    be.steps.clear()
    third = sch.submit(Request(prompt[:10] + [1, 2, 3], max_tokens=1, temperature=0.0))
    sch.run_until_done()
    assert be.steps[0] == [(third.id, 8, prompt[8:10] + [1, 2, 3], True)]
    kv.check()
    assert first.finish_reason == "length"


def test_without_the_flag_nothing_is_shared():
    sch, be, kv = make(prefix_cache=False)
    prompt = list(range(300, 318))
    for _ in range(2):
        sch.submit(Request(prompt, max_tokens=2, temperature=0.0))
        sch.run_until_done()
    assert kv.pools[0].cached == 0 and sch.stats.prefix_hit_tokens == 0
    firsts = [step[0] for step in be.steps if step[0][2] == prompt[:8]]
    assert len(firsts) == 2 and all(f[1] == 0 for f in firsts)   # both requests prefill from position 0


def test_a_preempted_request_finds_its_own_pages_again():
    # 6 pages of 4: two requests of 9 prompt tokens decode until the pool runs out; the younger is preempted,
    # its pages stay named, and when it comes back it prefills only the tail
    sch, be, kv = make(n_blocks=6)
    a = sch.submit(Request(list(range(9)), max_tokens=8, temperature=0.0))
    b = sch.submit(Request(list(range(50, 59)), max_tokens=8, temperature=0.0))
    sch.run_until_done()
    assert b.preemptions >= 1 and a.preemptions == 0
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert len(a.completion) == 8 and len(b.completion) == 8
    assert sch.stats.prefix_hit_tokens > 0
    kv.check()

"""The scheduler's decisions, with a scripted backend instead of a device."""
import pytest

from cuca_b200.cache.pages import GroupLayout, KvPools, StateSlots
from cuca_b200.engine.scheduler import (DECODE, Request, RequestError, Scheduler, SchedulerConfig,
                                        prefill_chunk_for)


class FakeBackend:
    """Records every step; 'samples' prompt-independent tokens: 1000 + request id * 100 + count."""

    def __init__(self, pools, eos_after=None):
        self.pools = pools
        self.steps = []
        self.started = []
        self.eos_after = eos_after or {}
        self.counts = {}

    def start(self, seq):
        self.started.append((seq.id, seq.slot, seq.rng_state()))

    def run(self, plans):
        self.steps.append([(p.seq.id, p.seq.blocks.length, list(p.tokens), p.want_last) for p in plans])
        out = []
        for p in plans:
            # what the real step function does to the bookkeeping
            assert len(p.seq.blocks.tables[0]) * self.pools.block_size >= p.seq.blocks.length + len(p.tokens)
            p.seq.blocks.length += len(p.tokens)
            if p.want_last:
                n = self.counts.get(p.seq.id, 0)
                self.counts[p.seq.id] = n + 1
                out.append(7 if self.eos_after.get(p.seq.id) == n else 1000 + p.seq.id * 100 + n)
        self.pools.check()
        return out


def make(n_blocks=64, max_sequences=4, max_step_tokens=8, prefill_chunk=8, ctx=256, bs=16, eos=(7,), eos_after=None):
    pools = KvPools([GroupLayout(2, 16, None, (0, 1), n_blocks)], bs)
    slots = StateSlots(max_sequences)
    be = FakeBackend(pools, eos_after)
    sch = Scheduler(pools, slots, be, SchedulerConfig(max_sequences, max_step_tokens, prefill_chunk, ctx, tuple(eos)),
                    seed_source=lambda: 42)
    return sch, be, pools, slots


def test_prefill_chunk_rule():
    assert prefill_chunk_for(8192) == 256 and prefill_chunk_for(1 << 20) == 16 and prefill_chunk_for(128) == 256


def test_submit_rejects_empty_and_overlong():
    sch, *_ = make(ctx=32)
    with pytest.raises(RequestError):
        sch.submit(Request([]))
    with pytest.raises(RequestError):
        sch.submit(Request(list(range(32))))
    with pytest.raises(RequestError):
        sch.submit(Request([1], top_p=0.0))
    with pytest.raises(RequestError):
        sch.submit(Request([1], temperature=-1.0))


def test_exact_usage_max_tokens_and_context_cap():
    sch, be, pools, slots = make(ctx=32, max_step_tokens=64, prefill_chunk=64)
    a = sch.submit(Request(list(range(10)), max_tokens=5))
    b = sch.submit(Request(list(range(30))))  # only 2 positions of context left
    sch.run_until_done()
    assert len(a.completion) == 5 and a.finish_reason == "length"
    assert len(b.completion) == 2 and b.finish_reason == "length"
    assert a.completion == [1000, 1001, 1002, 1003, 1004]
    # the last token is emitted but never forwarded: a cached 10 + 4 positions
    assert all(p.free == p.n_blocks for p in pools.pools) and slots.free == 4


def test_end_of_generation_id_stops_uncounted():
    sch, be, pools, slots = make(eos_after={0: 3})
    a = sch.submit(Request([5, 6, 8], max_tokens=50))
    sch.run_until_done()
    assert a.finish_reason == "stop" and a.completion == [1000, 1001, 1002]
    b = sch.submit(Request([5, 6, 8], max_tokens=50, stop_token_ids=[1101]))
    sch.run_until_done()
    assert b.finish_reason == "stop" and b.completion == [1100]


def test_prompts_are_cut_under_the_token_budget_and_interleave_with_decode():
    sch, be, pools, _ = make(max_step_tokens=8, prefill_chunk=8)
    a = sch.submit(Request(list(range(3)), max_tokens=20))
    sch.turn()  # a: whole prompt
    assert be.steps[-1] == [(0, 0, [0, 1, 2], True)] and a.phase == DECODE
    b = sch.submit(Request(list(range(100, 120)), max_tokens=4))
    sch.turn()  # a decodes 1 row, b gets the 7 rows left
    assert be.steps[-1][0] == (0, 3, [1000], True)
    assert be.steps[-1][1] == (1, 0, list(range(100, 107)), False)
    sch.turn()
    assert be.steps[-1][1] == (1, 7, list(range(107, 114)), False)
    sch.turn()  # the last portion of b asks for logits
    assert be.steps[-1][1] == (1, 14, list(range(114, 120)), True) and b.phase == DECODE
    sch.turn()  # both decode: oldest first
    assert [s[0] for s in be.steps[-1]] == [0, 1] and all(len(s[2]) == 1 for s in be.steps[-1])
    sch.run_until_done()
    assert len(a.completion) == 20 and len(b.completion) == 4
    assert sch.stats.generated_tokens == 24 and sch.stats.admissions == 2


def test_two_prompts_share_one_step():
    sch, be, *_ = make(max_step_tokens=16, prefill_chunk=16)
    sch.submit(Request(list(range(5)), max_tokens=2))
    sch.submit(Request(list(range(50, 58)), max_tokens=2))
    sch.turn()
    assert [(s[0], len(s[2]), s[3]) for s in be.steps[-1]] == [(0, 5, True), (1, 8, True)]


def test_admission_is_fifo_and_waits_for_pages_and_slots():
    # 4 pages of 16: the first prompt (40 + 1 positions) needs 3, the second (20 + 1) needs 2 -> must wait
    sch, be, pools, _ = make(n_blocks=4, max_step_tokens=64, prefill_chunk=64)
    a = sch.submit(Request(list(range(40)), max_tokens=3))
    b = sch.submit(Request(list(range(20)), max_tokens=3))
    c = sch.submit(Request([1], max_tokens=1))  # would fit, but may not overtake b (head-of-line blocking)
    sch.turn()
    assert [s.id for s in sch.running] == [0] and [s.id for s in sch.waiting] == [1, 2]
    sch.run_until_done()
    assert [len(s.completion) for s in (a, b, c)] == [3, 3, 1]
    order = [i for i, _, _ in be.started]
    assert order == [0, 1, 2]
    sch2, be2, *_ = make(max_sequences=2)
    for i in range(5):
        sch2.submit(Request([i + 1], max_tokens=2))
    sch2.turn()
    assert len(sch2.running) == 2 and len(sch2.waiting) == 3
    sch2.run_until_done()
    assert sch2.stats.admissions == 5


def test_pages_run_out_the_youngest_is_preempted_and_resumes():
    # 7 pages of 16 (as the reference's preemption test): two requests that both grow past what fits
    sch, be, pools, slots = make(n_blocks=7, max_step_tokens=64, prefill_chunk=64, ctx=256)
    a = sch.submit(Request(list(range(30)), max_tokens=40, seed=1, temperature=1.0))
    b = sch.submit(Request(list(range(100, 130)), max_tokens=40, seed=2, temperature=1.0))
    sch.run_until_done()
    assert sch.stats.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0  # the oldest is never preempted
    assert len(a.completion) == 40 and len(b.completion) == 40 and a.finish_reason == b.finish_reason == "length"
    # b came back with prompt + generated as its new prompt and went on where it was
    resumed = [s for s in be.started if s[0] == 1]
    assert len(resumed) >= 2
    assert b.completion == [1100 + i for i in range(40)]  # no token lost or repeated
    # the generator state after k draws is seed + k * golden: a resumed request continues its sequence
    golden, m64 = 0x9E3779B97F4A7C15, (1 << 64) - 1
    assert resumed[0][2] == 2 and resumed[1][2] in {(2 + k * golden) & m64 for k in range(1, 41)}
    assert all(p.free == p.n_blocks for p in pools.pools) and slots.free == 4
    pools.check()


def test_a_prompt_portion_that_finds_no_page_waits_instead_of_failing():
    """Admission counts the prompts being prefilled, not what decoding requests will grow by: a prompt cut into
    portions can find the pool empty half-way. It goes back to the queue (it is the youngest) and finishes later."""
    sch, be, pools, slots = make(n_blocks=4, max_step_tokens=9, prefill_chunk=8, ctx=256)
    a = sch.submit(Request(list(range(30)), max_tokens=20))            # two pages, a third from position 32 on
    while a.phase != DECODE:
        sch.turn()
    b = sch.submit(Request(list(range(100, 130)), max_tokens=3))       # admitted: two pages are free
    sch.run_until_done()
    assert a.finish_reason == b.finish_reason == "length" and a.error is None and b.error is None
    assert len(a.completion) == 20 and b.completion == [1100, 1101, 1102]
    assert b.preemptions >= 1 and a.preemptions == 0
    starts_of_b = [st for st in be.started if st[0] == 1]
    assert len(starts_of_b) >= 2  # admitted, sent back while still in its prompt, admitted again
    assert all(p.free == p.n_blocks for p in pools.pools) and slots.free == 4
    pools.check()


def test_a_single_request_that_exhausts_the_pool_fails_cleanly():
    sch, be, pools, slots = make(n_blocks=2, max_step_tokens=64, prefill_chunk=64)
    a = sch.submit(Request(list(range(20)), max_tokens=100))
    sch.run_until_done()
    assert a.finish_reason == "error" and "exhausted" in a.error and len(a.completion) == 13  # 20 + 12 cached positions fill both pages; the 13th token has nowhere to go
    assert all(p.free == p.n_blocks for p in pools.pools) and slots.free == 4
    big = sch.submit(Request(list(range(100)), max_tokens=1))  # can never fit: fails instead of blocking the queue
    ok = sch.submit(Request([1, 2], max_tokens=1))
    sch.run_until_done()
    assert big.finish_reason == "error" and ok.finish_reason == "length"


def test_a_failed_step_fails_the_running_requests_and_resets_the_cache():
    sch, be, pools, slots = make()
    a = sch.submit(Request([1, 2, 3], max_tokens=5))
    sch.turn()

    def boom(plans):
        raise RuntimeError("injected")

    be.run = boom
    with pytest.raises(RuntimeError, match="injected"):
        sch.turn()
    assert a.finish_reason == "error" and not sch.running
    assert all(p.free == p.n_blocks for p in pools.pools) and slots.free == 4
    be.run = FakeBackend(pools).run
    b = sch.submit(Request([4], max_tokens=2))
    sch.run_until_done()
    assert len(b.completion) == 2  # the engine keeps serving


def test_seeded_requests_restart_their_generator():
    sch, be, *_ = make()
    a = sch.submit(Request([1], max_tokens=1, seed=123))
    b = sch.submit(Request([2], max_tokens=1, seed=123))
    c = sch.submit(Request([3], max_tokens=1))
    sch.run_until_done()
    states = {i: st for i, _, st in be.started}
    assert states[0] == states[1] == 123 and states[2] == 42


def test_prefix_cache_is_refused_when_a_mixer_keeps_state():
    """Pools whose model also keeps per-request state cannot serve requests from cached pages."""
    from cuca_b200.cache.pages import GroupLayout, KvPools, StateSlots, StatefulCacheError
    from cuca_b200.engine.scheduler import Scheduler, SchedulerConfig
    pools = KvPools([GroupLayout(1, 16, None, (0,), 8)], 4)
    pools.stateful = True
    with pytest.raises(StatefulCacheError, match="prefix_cache"):
        Scheduler(pools, StateSlots(2), None, SchedulerConfig(prefix_cache=True))
    Scheduler(pools, StateSlots(2), None, SchedulerConfig(prefix_cache=False))
    with pytest.raises(StatefulCacheError, match="rolled back"):
        pools.truncate(pools.new_seq(), 0)

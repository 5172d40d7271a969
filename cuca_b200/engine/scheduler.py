"""Continuous batching above the step function: admit, cut prompts into portions, decode, finish, free.

One `turn` is at most one step (src/provider/local/engine/scheduler.rs:515-535,
793-876,1032-1107 of the reference):

* admission is first-in first-out with head-of-line blocking; a request starts
  when fewer than `max_sequences` run, a state slot is free and the pools can
  give the pages its prompt (+1 position) needs on top of what the prompts
  already being prefilled still need;
* a step has at most `max_step_tokens` rows: every decoding request brings its
  one pending token (oldest first), then prefilling requests bring portions of
  `min(remaining, prefill_chunk, room)` tokens in admission order; only the last
  portion of a prompt asks for logits;
* a request finishes on an end-of-generation id (not counted, not forwarded),
  when its completion reaches `min(max_tokens, context - prompt)`, or when it
  fills the context; its pages and slot go back at once;
* when pages run out while decoding, the youngest running request is preempted:
  its pages are freed and it returns to the front of the queue with everything
  it had (prompt + generated) as its new prompt, to be prefilled again. The
  oldest request is never preempted; a request alone that exhausts the pool
  fails with an error (engine/scheduler.rs:970-1008).

This file decides; it touches no device. The `backend` runs a step and samples.
"""
from __future__ import annotations

import ctypes
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache.pages import KvPools, StateSlots, StatefulCacheError
from ..native import host

PREFILL, DECODE, ENDED = "prefill", "decode", "ended"
_GOLDEN = 0x9E3779B97F4A7C15
_M64 = (1 << 64) - 1


class RequestError(ValueError):
    """The request cannot run (empty or over-long prompt)."""


@dataclass
class Request:
    """What a caller asks for; field names follow the reference's request (src/request.rs:211-230)."""

    prompt: Sequence[int]
    max_tokens: Optional[int] = None
    temperature: float = 1.0
    top_k: int = 64
    top_p: float = 0.95
    seed: Optional[int] = None
    stop_token_ids: Sequence[int] = ()
    request_id: Optional[str] = None


@dataclass(eq=False)  # identity, not field-by-field equality: requests are looked up in lists every turn
class Sequence_:
    request: Request
    id: int
    prompt: list  # what must be prefilled (grows by the generated tokens after a preemption)
    prompt_tokens: int  # the caller's prompt length
    budget: int
    seed: int
    completion: list = field(default_factory=list)
    phase: str = PREFILL
    pos: int = 0  # prompt tokens already cached
    pending: Optional[int] = None  # sampled, not yet forwarded
    blocks: object = None
    slot: int = -1
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    draws: int = 0  # tokens drawn so far: the SplitMix64 state is seed + draws * golden
    queued_at: float = 0.0
    started_at: float = 0.0
    first_token_at: float = 0.0
    finished_at: float = 0.0
    preemptions: int = 0
    core_id: int = -1  # the request's record in the host core (reused after the request is forgotten)
    _forget: object = None  # set when the request has ended (see `_Forget`)

    def rng_state(self) -> int:
        return (self.seed + self.draws * _GOLDEN) & _M64

    @property
    def done(self) -> bool:
        return self.phase == ENDED


@dataclass(eq=False)
class Plan:
    """One request's share of the coming step."""

    seq: Sequence_
    tokens: list
    want_last: bool
    start: int = -1  # positions the request has cached before the step (-1: ask its block tables)


@dataclass
class SchedulerConfig:
    max_sequences: int = 4
    max_step_tokens: int = 256
    prefill_chunk: int = 256
    context_length: int = 8192
    eos_token_ids: tuple = ()
    prefix_cache: bool = False  # requests start from the longest cached prefix of their prompt


@dataclass
class ServingStats:
    """Counters in the manner of the reference's ServingStats (src/provider/local/mod.rs:2175-2226)."""

    running: int = 0
    waiting: int = 0
    max_sequences: int = 0
    free_blocks: int = 0
    used_blocks: int = 0
    total_blocks: int = 0
    preemptions: int = 0
    steps: int = 0
    batched_rows: int = 0
    prefill_rows: int = 0
    generated_tokens: int = 0
    admissions: int = 0
    prefix_hit_tokens: int = 0  # prompt tokens whose keys and values were found cached
    step_seconds: float = 0.0
    last_step_rows: int = 0


def prefill_chunk_for(context_length: int) -> int:
    """clamp(2^21 / context, 16, 256) (src/provider/local/model/mod.rs:387-389)."""
    return max(16, min(256, (1 << 21) // max(1, context_length)))


_PHASES = (PREFILL, DECODE, ENDED)
_REASONS = {1: "stop", 2: "length", 3: "error", 4: "cancelled"}
_EV_ADMITTED, _EV_TOKEN, _EV_FINISHED, _EV_PREEMPTED, _EV_PREFILLED, _EV_DECODING = 1, 2, 3, 4, 5, 6


class Scheduler:
    """The decisions are taken by the C++ host core (`csrc/host/scheduler.cpp`); this class hands requests over,
    runs the planned step through the `backend`, hands the sampled tokens back and keeps `Sequence_` objects in
    step with the events the core reports."""

    def __init__(self, pools: KvPools, slots: StateSlots, backend, config: SchedulerConfig,
                 seed_source: Optional[Callable[[], int]] = None):
        if config.prefix_cache and getattr(pools, "stateful", False):
            # a request that starts from cached pages skips the tokens they hold; a mixer with state of its own
            # would start with empty state in the middle of its sequence. The reference keeps snapshots of such
            # state beside the pages (src/provider/local/engine/scheduler.rs:813-830); this engine refuses.
            raise StatefulCacheError("prefix_cache cannot be used with this model: a mixer keeps per-request state "
                                     "besides its pages, and cached pages do not bring that state back")
        self.pools = pools
        self.slots = slots
        self.backend = backend
        self.cfg = config
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: list = []
        self._stats = ServingStats(max_sequences=config.max_sequences)
        self._next_id = 0
        self._seed_source = seed_source or _default_seed_source()
        self._lib = host.load()
        eos = [int(t) for t in config.eos_token_ids]
        self._h = self._lib.cuca_host_sched_new(pools._h, slots._h, config.max_sequences, config.max_step_tokens,
                                                config.prefill_chunk, config.context_length, host.ints(eos), len(eos),
                                                int(config.prefix_cache))
        self._seqs: dict = {}  # id in the core -> Sequence_, while the core still knows the request
        self._plan_buf = (ctypes.c_int * (8 * max(1, config.max_step_tokens)))()
        self._event_buf = (ctypes.c_int * 4096)()
        self._on_token = None

    def __del__(self):
        if getattr(self, "_h", None):
            h, self._h = self._h, None
            self._lib.cuca_host_sched_free(h)

    # ------------------------------------------------------------ submit
    def submit(self, request: Request) -> Sequence_:
        n = len(request.prompt)
        if n == 0:
            raise RequestError("the prompt is empty")
        if request.temperature < 0 or request.temperature != request.temperature:
            raise RequestError("temperature must be a finite number >= 0")
        if not 0.0 < request.top_p <= 1.0:
            raise RequestError("top_p must lie in (0, 1]")
        prompt = [int(t) for t in request.prompt]
        stops = [int(t) for t in request.stop_token_ids]
        sid = self._lib.cuca_host_sched_submit(self._h, host.ints(prompt), n,
                                               -1 if request.max_tokens is None else int(request.max_tokens),
                                               int(request.temperature > 0), host.ints(stops), len(stops))
        if sid < 0:
            # src/provider/local/mod.rs:3252, engine/scheduler.rs:471-482
            raise RequestError(host.last_error())
        seed = request.seed if request.seed is not None else self._seed_source()
        seq = Sequence_(request, self._next_id, prompt, n, int(self._lib.cuca_host_sched_seq_get(self._h, sid, 7)),
                        seed & _M64, queued_at=time.perf_counter(), core_id=sid)
        self._next_id += 1
        self._seqs[sid] = seq
        self.waiting.append(seq)
        self._events()  # a request without room for a single token has ended already
        return seq

    # ------------------------------------------------------------ one turn
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def turn(self) -> int:
        """Admit, plan, run one step, apply its results. Returns the rows of the step (0: nothing to do)."""
        lib = self._lib
        lib.cuca_host_sched_admit(self._h)
        self._events()
        n = lib.cuca_host_sched_plan(self._h, self._plan_buf, len(self._plan_buf) // 8)
        if n < 0:
            raise RuntimeError("the plan of a step has more requests than rows: the host core is confused")
        self._events()  # preemptions and failures found while planning
        if n == 0:
            return 0
        buf, plans = self._plan_buf, []
        for i in range(n):
            sid, offset, cnt, want_last, _slot, _blocks, start, token = buf[8 * i:8 * i + 8]
            seq = self._seqs[sid]
            plans.append(Plan(seq, [token] if token >= 0 else seq.prompt[offset:offset + cnt], bool(want_last), start))
        t0 = time.perf_counter()
        try:
            tokens = self.backend.run(plans)
        except Exception as e:  # a failed step fails every running request and resets the cache
            lib.cuca_host_sched_fail_running(self._h, f"step failed: {e}".encode())
            self._events()
            raise
        rows = sum(len(p.tokens) for p in plans)
        st = self._stats
        st.prefill_rows += sum(len(p.tokens) for p in plans if p.seq.phase == PREFILL)
        toks = [int(t) for t in tokens]
        if lib.cuca_host_sched_apply(self._h, host.ints(toks), len(toks)):
            raise RuntimeError(host.last_error())
        self._events()
        st.steps += 1
        st.batched_rows += rows
        st.step_seconds += time.perf_counter() - t0
        st.last_step_rows = rows
        return rows

    def cancel(self, seq: Sequence_) -> None:
        """The caller has no use for the request any more: its pages and slot go back, it ends as "cancelled"
        (src/provider/local/engine/scheduler.rs:663-678)."""
        if seq.phase != ENDED and self._seqs.get(seq.core_id) is seq:
            self._lib.cuca_host_sched_cancel(self._h, seq.core_id)
            self._events()

    def run_until_done(self, on_token: Optional[Callable] = None) -> None:
        self._on_token = on_token
        while self.has_work():
            if self.turn() == 0 and self.has_work():
                raise RuntimeError("the scheduler made no progress: the page pool is too small for the queue's head")

    # ------------------------------------------------------------ what the core reports
    def _events(self) -> None:
        lib, buf = self._lib, self._event_buf
        while True:
            n = lib.cuca_host_sched_events(self._h, buf, len(buf) // 4)
            if n < 0:
                self._event_buf = buf = (ctypes.c_int * (4 * -n))()
                continue
            break
        now = None
        for i in range(n):
            kind, sid, value, extra = buf[4 * i:4 * i + 4]
            seq = self._seqs[sid]
            if kind == _EV_TOKEN:
                if not seq.completion:
                    seq.first_token_at = time.perf_counter()
                seq.completion.append(value)
                seq.pending = value
                if seq.request.temperature > 0:
                    seq.draws += 1
                self._stats.generated_tokens += 1
                if self._on_token:
                    self._on_token(seq, value)
            elif kind == _EV_PREFILLED:
                seq.pos = value
            elif kind == _EV_DECODING:
                seq.phase = DECODE
            elif kind == _EV_ADMITTED:
                self.waiting.remove(seq)
                seq.slot, seq.blocks = value, self.pools.adopt(extra)
                seq.phase, seq.pos, seq.pending = PREFILL, 0, None
                seq.started_at = seq.started_at or time.perf_counter()
                self.backend.start(seq)
                self.running.append(seq)
                self._stats.admissions += 1
            elif kind == _EV_PREEMPTED:
                self.running.remove(seq)
                seq.prompt = list(seq.request.prompt) + list(seq.completion)
                seq.phase, seq.pos, seq.pending, seq.slot = PREFILL, 0, None, -1
                seq.preemptions += 1
                self._stats.preemptions += 1
                self.waiting.appendleft(seq)
            elif kind == _EV_FINISHED:
                if seq in self.running:
                    self.running.remove(seq)
                elif seq in self.waiting:
                    self.waiting.remove(seq)
                if value == 1 and seq.request.temperature > 0:
                    seq.draws += 1  # the end token was drawn too
                seq.phase, seq.slot, seq.pending = ENDED, -1, None
                seq.finish_reason = _REASONS[value]
                err = lib.cuca_host_sched_seq_error(self._h, sid)
                seq.error = err.decode(errors="replace") if err else None
                seq.finished_at = time.perf_counter()
                self.finished.append(seq)
                seq._forget = _Forget(self, sid)

    def _release_record(self, sid: int) -> None:
        """The last reference to an ended request is gone: the core may reuse its record."""
        if getattr(self, "_h", None) and self._seqs.get(sid) is None:
            self._lib.cuca_host_sched_forget(self._h, sid)

    @property
    def stats(self) -> ServingStats:
        """The counters, with the queue lengths and the pools' figures as they are now (asked of the host core when
        read, not at every turn)."""
        self._publish()
        return self._stats

    def _publish(self) -> None:
        st, ps = self._stats, self.pools.stats()
        st.running, st.waiting = len(self.running), len(self.waiting)
        st.prefix_hit_tokens = int(self._lib.cuca_host_sched_counter(self._h, 5))
        st.free_blocks, st.used_blocks, st.total_blocks = (min(ps["free_blocks"], default=0),
                                                           max(ps["used_blocks"], default=0),
                                                           min(ps["total_blocks"], default=0))


class _Forget:
    """Lives as long as an ended `Sequence_` does; when it goes, the host core may reuse the request's record."""

    def __init__(self, scheduler: Scheduler, sid: int):
        import weakref
        self._scheduler, self._sid = weakref.ref(scheduler), sid
        scheduler._seqs.pop(sid, None)

    def __del__(self):
        try:
            sch = self._scheduler()
            if sch is not None:
                sch._release_record(self._sid)
        except Exception:  # interpreter shutdown
            pass


def _default_seed_source():
    import random
    rng = random.Random(time.time_ns())
    return lambda: rng.getrandbits(64)

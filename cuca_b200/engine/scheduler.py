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

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache.pages import KvPools, PoolExhausted, StateSlots
from .step import StepEntry

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


@dataclass
class SchedulerConfig:
    max_sequences: int = 4
    max_step_tokens: int = 256
    prefill_chunk: int = 256
    context_length: int = 8192
    eos_token_ids: tuple = ()


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
    step_seconds: float = 0.0
    last_step_rows: int = 0


def prefill_chunk_for(context_length: int) -> int:
    """clamp(2^21 / context, 16, 256) (src/provider/local/model/mod.rs:387-389)."""
    return max(16, min(256, (1 << 21) // max(1, context_length)))


class Scheduler:
    def __init__(self, pools: KvPools, slots: StateSlots, backend, config: SchedulerConfig,
                 seed_source: Optional[Callable[[], int]] = None):
        self.pools = pools
        self.slots = slots
        self.backend = backend
        self.cfg = config
        self.waiting: deque = deque()
        self.running: list = []
        self.finished: list = []
        self.stats = ServingStats(max_sequences=config.max_sequences)
        self._next_id = 0
        self._seed_source = seed_source or _default_seed_source()

    # ------------------------------------------------------------ submit
    def submit(self, request: Request) -> Sequence_:
        n = len(request.prompt)
        if n == 0:
            raise RequestError("the prompt is empty")
        if n >= self.cfg.context_length:
            # src/provider/local/mod.rs:3252, engine/scheduler.rs:471-482
            raise RequestError(f"the prompt has {n} tokens; the context holds {self.cfg.context_length}")
        if request.temperature < 0 or request.temperature != request.temperature:
            raise RequestError("temperature must be a finite number >= 0")
        if not 0.0 < request.top_p <= 1.0:
            raise RequestError("top_p must lie in (0, 1]")
        room = self.cfg.context_length - n
        budget = room if request.max_tokens is None else min(int(request.max_tokens), room)
        seed = request.seed if request.seed is not None else self._seed_source()
        seq = Sequence_(request, self._next_id, list(request.prompt), n, budget, seed & _M64,
                        queued_at=time.perf_counter())
        self._next_id += 1
        if budget <= 0:
            self._finish(seq, "length")
            return seq
        self.waiting.append(seq)
        return seq

    # ------------------------------------------------------------ one turn
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def turn(self) -> int:
        """Admit, plan, run one step, apply its results. Returns the rows of the step (0: nothing to do)."""
        self._admit()
        plans = self._plan()
        if not plans:
            self._publish()
            return 0
        t0 = time.perf_counter()
        try:
            tokens = self.backend.run(plans)
        except Exception as e:  # a failed step fails every running request and resets the cache
            self._fail_running(f"step failed: {e}")
            raise
        rows = sum(len(p.tokens) for p in plans)
        st = self.stats
        st.prefill_rows += sum(len(p.tokens) for p in plans if p.seq.phase == PREFILL)
        self._apply(plans, tokens)
        st.steps += 1
        st.batched_rows += rows
        st.step_seconds += time.perf_counter() - t0
        st.last_step_rows = rows
        self._publish()
        return rows

    def run_until_done(self, on_token: Optional[Callable] = None) -> None:
        self._on_token = on_token
        while self.has_work():
            if self.turn() == 0 and self.has_work():
                raise RuntimeError("the scheduler made no progress: the page pool is too small for the queue's head")

    # ------------------------------------------------------------ admission
    def _committed(self) -> list:
        """Pages the prompts being prefilled still need (per group)."""
        total = [0] * len(self.pools.groups)
        for s in self.running:
            if s.phase == PREFILL:
                for i, o in enumerate(self.pools.owed(s.blocks, len(s.prompt) + 1)):
                    total[i] += o
        return total

    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.cfg.max_sequences and self.slots.free > 0:
            seq = self.waiting[0]
            owed = [c + o for c, o in zip(self._committed(), self.pools.owed(None, len(seq.prompt) + 1))]
            if not self.pools.can_give(owed):
                if not self.running and not self.pools.can_give(self.pools.owed(None, len(seq.prompt) + 1)):
                    # nothing runs and it still does not fit: it never will
                    self.waiting.popleft()
                    self._finish(seq, "error", f"the prompt needs more pages than the pool has")
                    continue
                break  # head-of-line blocking
            self.waiting.popleft()
            seq.slot = self.slots.alloc()
            seq.blocks = self.pools.new_seq()
            seq.phase, seq.pos, seq.pending = PREFILL, 0, None
            seq.started_at = seq.started_at or time.perf_counter()
            self.backend.start(seq)
            self.running.append(seq)
            self.stats.admissions += 1

    # ------------------------------------------------------------ planning
    def _plan(self) -> list:
        budget = self.cfg.max_step_tokens
        plans, used = [], 0
        # decoding requests, oldest first
        for seq in list(self.running):
            if seq.phase != DECODE or seq not in self.running:
                continue
            if used >= budget:
                break
            if not self._ensure_block(seq):
                continue
            plans.append(Plan(seq, [seq.pending], True))
            used += 1
        # the preemptions above may have removed planned requests
        plans = [p for p in plans if p.seq in self.running]
        used = len(plans)
        # prompts, in admission order
        for seq in list(self.running):
            if seq.phase != PREFILL:
                continue
            room = budget - used
            if room <= 0:
                break
            n = min(len(seq.prompt) - seq.pos, self.cfg.prefill_chunk, room)
            try:
                self.pools.reserve(seq.blocks, seq.pos + n)
            except PoolExhausted:
                # a prompt portion that cannot get its pages fails that request
                # (src/provider/local/engine/scheduler.rs:1260-1263)
                self._release(seq)
                self._finish(seq, "error", "the K/V page pool is exhausted")
                continue
            last = seq.pos + n == len(seq.prompt)
            plans.append(Plan(seq, seq.prompt[seq.pos:seq.pos + n], last))
            used += n
        return plans

    def _ensure_block(self, seq: Sequence_) -> bool:
        """Pages for the pending token's position; preempts the youngest on exhaustion."""
        while True:
            try:
                self.pools.reserve(seq.blocks, seq.blocks.length + 1)
                return True
            except PoolExhausted:
                if len(self.running) == 1:
                    self._release(seq)
                    self._finish(seq, "error", "the K/V page pool is exhausted by one request")
                    return False
                victim = self.running[-1]  # youngest
                if victim is self.running[0]:
                    victim = seq
                self._preempt(victim)
                if victim is seq:
                    return False

    def _preempt(self, seq: Sequence_) -> None:
        """Free the request's pages; it goes back to the front of the queue with all it had as its prompt."""
        self._release(seq)
        seq.prompt = list(seq.request.prompt) + list(seq.completion)
        # the pending token is the last of `completion`; it is part of the new prompt and its logits
        # will be asked for again at the end of the re-prefill
        seq.phase, seq.pos, seq.pending = PREFILL, 0, None
        seq.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(seq)

    # ------------------------------------------------------------ results
    def _apply(self, plans: list, tokens: list) -> None:
        it = iter(tokens)
        for p in plans:
            seq = p.seq
            if seq.phase == PREFILL:
                seq.pos += len(p.tokens)
                if not p.want_last:
                    continue
                # (a preempted request re-prefilled its own completion too: the logits just computed are those
                # that follow its last emitted token, so decoding simply goes on)
                seq.phase = DECODE
            self._take_token(seq, int(next(it)))

    def _take_token(self, seq: Sequence_, tok: int) -> None:
        """Rules of src/provider/local/engine/scheduler.rs:1287-1316."""
        seq.draws += 1 if seq.request.temperature > 0 else 0
        if tok in self.cfg.eos_token_ids or tok in seq.request.stop_token_ids:
            self._release(seq)
            self._finish(seq, "stop")
            return
        if not seq.completion:
            seq.first_token_at = time.perf_counter()
        seq.completion.append(tok)
        self.stats.generated_tokens += 1
        if getattr(self, "_on_token", None):
            self._on_token(seq, tok)
        total = seq.prompt_tokens + len(seq.completion)
        if len(seq.completion) >= seq.budget or total >= self.cfg.context_length:
            self._release(seq)
            self._finish(seq, "length")
            return
        seq.pending = tok

    def _release(self, seq: Sequence_) -> None:
        if seq in self.running:
            self.running.remove(seq)
        if seq.blocks is not None and not seq.blocks.released:
            self.pools.release(seq.blocks)
        if seq.slot >= 0:
            self.slots.release(seq.slot)
            seq.slot = -1

    def _finish(self, seq: Sequence_, reason: str, error: Optional[str] = None) -> None:
        seq.phase = ENDED
        seq.finish_reason = reason
        seq.error = error
        seq.finished_at = time.perf_counter()
        self.finished.append(seq)

    def _fail_running(self, why: str) -> None:
        """src/provider/local/engine/scheduler.rs:950-966: every running request fails, the pools start over."""
        for seq in list(self.running):
            self.running.remove(seq)
            seq.slot = -1
            self._finish(seq, "error", why)
        self.pools.reset()
        self.slots.reset()

    def _publish(self) -> None:
        st, ps = self.stats, self.pools.stats()
        st.running, st.waiting = len(self.running), len(self.waiting)
        st.free_blocks, st.used_blocks, st.total_blocks = (min(ps["free_blocks"], default=0),
                                                           max(ps["used_blocks"], default=0),
                                                           min(ps["total_blocks"], default=0))


def _default_seed_source():
    import random
    rng = random.Random(time.time_ns())
    return lambda: rng.getrandbits(64)

"""Decode steps captured as CUDA graphs.

A decode step of B single-token requests launches some three hundred small kernels; captured once per batch
bucket (1, 2, 4, ..., 64) and length bucket, it replays as one graph launch. Everything the step reads lives in
static device buffers: tokens, positions and slots of the rows (padding rows carry slot -1 and are skipped by
the kernels), the per-slot page tables and sampling constants. The graph ends with the sampling kernel and an
`advance` kernel that feeds each sampled token back as the row's next input, so several steps can also run
back to back without the host (`burst`), which is how the device-only decode rate is measured.
"""
from __future__ import annotations

import gc
from typing import Sequence

import torch

from ..kernels import ops
from .step import StepBatch

LEN_BUCKET = 512
MAX_HISTORY = 1024


_side_stream = None


def _capture_stream():
    """The stream captures run on (a capture cannot run on the default stream); one for the process."""
    global _side_stream
    if _side_stream is None:
        _side_stream = torch.cuda.Stream()
    return _side_stream


def batch_bucket(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class DecodeGraph:
    def __init__(self, core, backend, bucket: int, max_len: int, pool=None):
        self.core, self.backend = core, backend
        self.pool = pool  # the memory pool this graph's capture allocates from (shared by an engine's graphs)
        self.bucket, self.max_len = bucket, max_len
        dev = core.rt.device
        self.meta = torch.zeros(3 * bucket, dtype=torch.int32, device=dev)
        self.meta[2 * bucket:] = -1
        self.tokens = self.meta[:bucket]
        self.positions = self.meta[bucket:2 * bucket]
        self.slot_of_row = self.meta[2 * bucket:]
        self.logit_rows = torch.arange(bucket, dtype=torch.int32, device=dev)
        # the sampled token of every row, then the device error word as it stood at the end of the step
        self.sampled = torch.full((bucket + 1,), -1, dtype=torch.int32, device=dev)
        self.sampled[bucket] = 0
        self.history = torch.zeros(MAX_HISTORY, bucket, dtype=torch.int32, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.pinned = torch.zeros(3 * bucket, dtype=torch.int32).pin_memory()
        self.pinned_np = self.pinned.numpy()
        # the same description of a step that the step function builds, over static buffers; mixers plan from it
        self.batch = StepBatch.single_tokens(self.tokens, self.positions, self.slot_of_row, self.logit_rows, max_len)
        self.graph = None
        self.scratch = None
        # [bucket, vocab]: what this graph's last replay left, if DecodeGraphs.keep_logits was set when it was captured
        # (tests read it). Not held otherwise, so that the next capture can use its memory again.
        self.logits = None
        self.keep_logits = False
        self.launches = 0

    def _body(self):
        logits = self.core.model.forward(self.batch, self.core.cache)
        self.logits = logits if self.keep_logits else None
        be = self.backend
        if be.suppress is not None:
            ops.suppress_tokens(logits, be.suppress)
        ops.sample(logits, be.temperature, be.top_k, be.top_p, be.rng, self.slot_of_row, self.sampled, self.scratch,
                   be.sample_split)
        ops.decode_advance(self.tokens, self.positions, self.slot_of_row, self.sampled, self.history, self.counter,
                           MAX_HISTORY, self.core.rt.err, self.sampled[self.bucket:])

    def capture(self, needs_scratch: bool) -> None:
        if needs_scratch:
            self.scratch = torch.empty(self.bucket, ops.sample_scratch_words(self.core.spec.vocab_size),
                                       dtype=torch.int64, device=self.core.rt.device)
        # warm up (first launches configure kernels and build tensor maps), rows all padding; on the stream the engine
        # runs on, so that what the step allocates comes out of the allocator's cache for that stream and not
        # from the driver (a call that now and then took tens of milliseconds here)
        self.meta[2 * self.bucket:] = -1
        self._body()
        torch.cuda.synchronize()
        side = _capture_stream()
        from ..kernels import library
        before = library.launches
        self.graph = torch.cuda.CUDAGraph()
        # No collection of dead Python cycles while the stream captures: a cycle that holds a CUDA graph or device
        # tensors (an engine the caller dropped a moment ago) would be torn down in the middle of the capture, and
        # resetting a graph or recording an event then invalidates it.
        collecting = gc.isenabled()
        gc.disable()
        # Captured by hand rather than through `torch.cuda.graph`: that context manager empties the caching
        # allocator first, and handing back the gigabytes a prompt's step had cached took up to 0.8 s per capture
        # here (a stall in the middle of serving, each time a new batch size is met), after which the next prompt
        # step had to ask the driver for all of it again.
        current = torch.cuda.current_stream()
        side.wait_stream(current)
        try:
            with torch.cuda.stream(side):
                self.graph.capture_begin(pool=self.pool) if self.pool is not None else self.graph.capture_begin()
                try:
                    self._body()
                finally:
                    self.graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        current.wait_stream(side)
        self.launches = library.launches - before  # kernels one replay runs
        torch.cuda.synchronize()
        self.counter.zero_()

    def load_rows(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int]) -> None:
        n, b = len(tokens), self.bucket
        a = self.pinned_np
        a[:n] = tokens
        a[n:b] = 0
        a[b:b + n] = positions
        a[b + n:2 * b] = 0
        a[2 * b:2 * b + n] = slots
        a[2 * b + n:] = -1
        self.meta.copy_(self.pinned, non_blocking=True)

    def replay(self) -> None:
        self.graph.replay()


class DecodeGraphs:
    """Captured decode steps by (batch bucket, length bucket); built on first use. `prime` captures the largest one
    ahead of time: its intermediates size the shared memory pool, so that later captures, in the middle of serving,
    find their memory there."""

    keep_logits = False  # graphs captured while this is set keep their logits tensor (for tests)

    def __init__(self, core, backend):
        self.core, self.backend = core, backend
        self.graphs: dict = {}
        # One memory pool for all of them: only one replays at a time, so what one capture's intermediates used the
        # next one's may use again, and a later capture need not ask the driver for memory (which took 40 to 100 ms
        # now and then). What a graph must keep between replays (its logits) stays referenced and is never reused.
        self.pool = torch.cuda.graph_pool_handle()

    def get(self, n_rows: int, max_len: int, needs_scratch: bool) -> DecodeGraph:
        bucket = batch_bucket(n_rows)
        len_bucket = min(-(-max_len // LEN_BUCKET) * LEN_BUCKET, max(self.core.context_length, LEN_BUCKET))
        key = (bucket, len_bucket, needs_scratch)
        g = self.graphs.get(key)
        if g is None:
            g = DecodeGraph(self.core, self.backend, bucket, len_bucket, self.pool)
            g.keep_logits = self.keep_logits
            g.capture(needs_scratch)
            self.graphs[key] = g
        return g

    def prime(self, max_rows: int) -> None:
        self.get(max_rows, 1, False)

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


def batch_bucket(n: int) -> int:
    b = 1
    while b < n:
        b <<= 1
    return b


class DecodeGraph:
    def __init__(self, core, backend, bucket: int, max_len: int):
        self.core, self.backend = core, backend
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
        self.logits = None  # [bucket, vocab]: what the last replay's model pass left (valid until the next replay)
        self.launches = 0

    def _body(self):
        logits = self.logits = self.core.model.forward(self.batch, self.core.cache)
        be = self.backend
        if be.suppress is not None:
            ops.suppress_tokens(logits, be.suppress)
        ops.sample(logits, be.temperature, be.top_k, be.top_p, be.rng, self.slot_of_row, self.sampled, self.scratch)
        ops.decode_advance(self.tokens, self.positions, self.slot_of_row, self.sampled, self.history, self.counter,
                           MAX_HISTORY, self.core.rt.err, self.sampled[self.bucket:])

    def capture(self, needs_scratch: bool) -> None:
        if needs_scratch:
            self.scratch = torch.empty(self.bucket, ops.sample_scratch_words(self.core.spec.vocab_size),
                                       dtype=torch.int64, device=self.core.rt.device)
        # warm up on a side stream (first launches configure kernels and build tensor maps), rows all padding
        self.meta[2 * self.bucket:] = -1
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..kernels import library
        before = library.launches
        self.graph = torch.cuda.CUDAGraph()
        # No collection of dead Python cycles while the stream captures: a cycle that holds a CUDA graph or device
        # tensors (an engine the caller dropped a moment ago) would be torn down in the middle of the capture, and
        # resetting a graph or recording an event then invalidates it.
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self._body()
        finally:
            if collecting:
                gc.enable()
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
    """Captured decode steps by (batch bucket, length bucket); built on first use."""

    def __init__(self, core, backend):
        self.core, self.backend = core, backend
        self.graphs: dict = {}

    def get(self, n_rows: int, max_len: int, needs_scratch: bool) -> DecodeGraph:
        bucket = batch_bucket(n_rows)
        len_bucket = min(-(-max_len // LEN_BUCKET) * LEN_BUCKET, max(self.core.context_length, LEN_BUCKET))
        key = (bucket, len_bucket, needs_scratch)
        g = self.graphs.get(key)
        if g is None:
            g = DecodeGraph(self.core, self.backend, bucket, len_bucket)
            g.capture(needs_scratch)
            self.graphs[key] = g
        return g

"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step holds any mix of requests, each bringing `t >= 1` consecutive tokens
that continue what it has cached: portions of prompts beside single decoded
tokens, cut anywhere (src/provider/local/model/mod.rs:253-281,1037-1062 and
model/cpu.rs:1766-1874 of the reference). Only the given tokens run; keys and
values of earlier tokens come from the request's pages. Logits come back only
for the wanted places, as one `[wanted, vocab]` 32-bit tensor in the order of
the entries and of each entry's `want`. Everything is validated on the host
before a kernel runs, and a failed validation leaves the cache untouched
(model/cpu.rs:1822-1837,4154-4185).

Rows carry their request's slot; page tables live on the device per slot and a
step uploads only the entries that changed, together with tokens and positions,
in one copy from pinned memory.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.device import DeviceCache
from ..cache.pages import KvPools, SeqBlocks
from ..kernels import ops
from ..native import host


class StepError(ValueError):
    """The batch handed to the step function is not valid; nothing ran."""


@dataclass
class StepEntry:
    """One request's share of a step."""

    blocks: SeqBlocks  # its pages; `blocks.length` positions are cached already
    slot: int  # its state slot
    tokens: Sequence[int]  # its next tokens
    want: Sequence[int] = ()  # places among `tokens` whose logits are wanted


@dataclass
class AttentionPlan:
    """How the step's rows are handed to the attention kernels: single-token requests to the decode form,
    longer portions in tiles of up to 64 rows to the prefill form."""

    decode_rows: Optional[torch.Tensor]  # [n_decode] int32 row numbers; None: rows 0..n_decode-1
    n_decode: int
    max_len: int  # largest position + 1 among the decode rows (bounds the key chunks)
    tile_row0: Optional[torch.Tensor]
    tile_nrows: Optional[torch.Tensor]
    n_tiles: int
    fixed_chunking: Optional[tuple] = None  # (chunk, n_splits) frozen for a captured graph
    tile128_row0: Optional[torch.Tensor] = None  # the same portions cut into tiles of up to 128 rows (tcgen05 form)
    tile128_nrows: Optional[torch.Tensor] = None
    n_tiles128: int = 0

    def chunk(self, n_kv_heads: int, head_dim: int = 128):
        if self.fixed_chunking is not None:
            return self.fixed_chunking
        from ..kernels.ops import decode_chunking
        return decode_chunking(self.n_decode, n_kv_heads, self.max_len, head_dim)


@dataclass
class StepBatch:
    """The step as the parts see it (device tensors unless said otherwise)."""

    n_rows: int
    n_seqs: int
    tokens: torch.Tensor  # [rows] int32
    positions: torch.Tensor  # [rows] int32
    seq_of_row: torch.Tensor  # [rows] int32: the slot of the row's request (< 0: padding)
    slots: torch.Tensor  # [requests] int32
    logit_rows: Optional[torch.Tensor]  # [wanted] int32 row numbers
    n_logit_rows: int
    host: dict = field(default_factory=dict)  # the same lists on the host, for parts that plan there
    attention_plan: Optional[AttentionPlan] = None


class _Staging:
    """A ring of pinned buffers, so a step's upload never waits for the previous one."""

    def __init__(self, device, n: int = 8, ints: int = 1 << 16):
        self.device = device
        self.bufs = [torch.empty(ints, dtype=torch.int32).pin_memory() for _ in range(n)]
        self.events = [None] * n
        self.i = 0

    def take(self, ints: int = 0) -> torch.Tensor:
        """The next pinned buffer (at least `ints` long), free to be written."""
        i = self.i
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        if self.bufs[i].shape[0] < ints:
            self.bufs[i] = torch.empty(max(ints, 2 * self.bufs[i].shape[0]), dtype=torch.int32).pin_memory()
        return self.bufs[i]

    def send(self, n: int) -> torch.Tensor:
        """Copy the first `n` integers of the buffer `take` returned to the device."""
        i = self.i
        self.i = (self.i + 1) % len(self.bufs)
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        dev.copy_(self.bufs[i][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev

    def upload(self, arr: np.ndarray) -> torch.Tensor:
        n = arr.shape[0]
        self.take(n)[:n].numpy()[:] = arr
        return self.send(n)


class Stepper:
    """Owns the device cache and runs steps of one model."""

    def __init__(self, model, pools: KvPools, cache: DeviceCache, context_length: int):
        self.model = model
        self.rt = model.rt
        self.pools = pools
        self.cache = cache
        self.context_length = context_length
        self.vocab = model.spec.vocab_size
        self._staging = _Staging(self.rt.device)
        self.steps = 0

    # ------------------------------------------------------------ the step
    def build(self, entries: Sequence[StepEntry]) -> StepBatch:
        """Validate the batch and pack it (the host core does both, `csrc/host/step_pack.cpp`): empty batch, empty
        token list, context overflow, token id out of range, missing or returned pages, wanted places and duplicate
        slots are refused before anything changes. Then one copy from pinned memory brings tokens, positions,
        slots, wanted rows, the attention plan and the page-table entries that changed."""
        lib, pools = host.load(), self.pools
        n = len(entries)
        counts = [len(e.tokens) for e in entries]
        flat_tokens = [int(t) for e in entries for t in e.tokens]
        n_want = [len(e.want) for e in entries]
        flat_want = [int(w) for e in entries for w in e.want]
        seqs = host.ints(e.blocks.handle for e in entries)
        slots_c = host.ints(e.slot for e in entries)
        sizes = (ctypes.c_int * (10 + 2 * pools.n_groups))()
        meta = (ctypes.c_int * 9)()
        args = (pools._h, n, seqs, slots_c, host.ints(counts), host.ints(flat_tokens), host.ints(n_want),
                host.ints(flat_want), self.context_length, self.vocab, self.cache.max_sequences, self.cache.table_width)
        buf = self._staging.take()
        code = lib.cuca_host_step_pack(*args, buf.data_ptr(), buf.shape[0], sizes, meta)
        if code == host.TOO_SMALL:
            buf = self._staging.take(meta[8])
            code = lib.cuca_host_step_pack(*args, buf.data_ptr(), buf.shape[0], sizes, meta)
        if code:
            raise StepError(host.last_error())
        T, S, R, n_decode, max_len, identity, n_tiles, n_tiles128, total = list(meta)
        dev = self._staging.send(total)
        views, off = [], 0
        for k in sizes:
            views.append(dev[off:off + k])
            off += k
        for gi in range(pools.n_groups):
            idx, val = views[10 + 2 * gi], views[11 + 2 * gi]
            if idx.shape[0]:
                ops.scatter_int(self.cache.tables[gi], idx, val)
        starts, row = [], 0
        return StepBatch(n_rows=T, n_seqs=S, tokens=views[0], positions=views[1], seq_of_row=views[2],
                         slots=views[3], logit_rows=views[4] if R else None, n_logit_rows=R,
                         host={"counts": counts, "slots": [e.slot for e in entries], "tokens": flat_tokens},
                         attention_plan=AttentionPlan(None if identity else views[5], n_decode, max_len,
                                                      views[6] if n_tiles else None, views[7] if n_tiles else None,
                                                      n_tiles, tile128_row0=views[8] if n_tiles128 else None,
                                                      tile128_nrows=views[9] if n_tiles128 else None,
                                                      n_tiles128=n_tiles128))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; returns logits [wanted, vocab] (32-bit, on the device) or None if nothing is wanted."""
        if not entries:
            raise StepError("a step needs at least one request")
        batch = self.build(entries)
        logits = self.model.forward(batch, self.cache)
        # every request has its tokens cached now; pages behind windows go back
        if host.load().cuca_host_step_advance(self.pools._h, host.ints(e.blocks.handle for e in entries),
                                              host.ints(len(e.tokens) for e in entries), len(entries)):
            raise StepError(host.last_error())
        self.steps += 1
        return logits

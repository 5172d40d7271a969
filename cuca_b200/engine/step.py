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
step uploads only the entries that changed, together with tokens, positions and
the per-request description of the step, in one copy from pinned memory. The
step function does not plan for any kernel: mixers do that from `StepBatch`.
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


N_FIXED_SECTIONS = 8  # sections of the packed buffer before the per-group page-table updates


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
class StepBatch:
    """The step as the parts see it (device tensors unless said otherwise).

    Per row: `tokens`, `positions`, `seq_of_row` (the slot of the row's request; < 0: padding). Per request, in the
    order given: `slots`, `req_row0` (the row its tokens start at), `req_count` (how many tokens it brings),
    `req_start` (how many positions it had cached before). The same per-request lists stand in `host` as Python
    lists (`slots`, `counts`, `starts`, `tokens`) for parts that plan on the host. How rows are handed to kernels
    (tiles, lists of single-token rows, scans over whole portions) is each mixer's own business: it derives what it
    needs from these arrays, once per step, and keeps it in `plans` under a key of its own for the other layers of
    its kind."""

    n_rows: int
    n_seqs: int
    tokens: torch.Tensor  # [rows] int32
    positions: torch.Tensor  # [rows] int32
    seq_of_row: torch.Tensor  # [rows] int32
    slots: torch.Tensor  # [requests] int32
    logit_rows: Optional[torch.Tensor]  # [wanted] int32 row numbers
    n_logit_rows: int
    host: dict = field(default_factory=dict)
    req_row0: Optional[torch.Tensor] = None  # [requests] int32
    req_count: Optional[torch.Tensor] = None
    req_start: Optional[torch.Tensor] = None
    static_max_len: Optional[int] = None  # a captured step: every request brings one token, none is longer than this
    plans: dict = field(default_factory=dict)

    @classmethod
    def single_tokens(cls, tokens, positions, slot_of_row, row_numbers, max_len: int) -> "StepBatch":
        """A step of static device buffers in which every row is one request's single next token (rows with slot
        -1 are padding) and every row's logits are wanted: the form a captured decode step has. `row_numbers` is
        0..rows-1 on the device; `positions` doubles as the requests' cached lengths."""
        n = tokens.shape[0]
        return cls(n_rows=n, n_seqs=n, tokens=tokens, positions=positions, seq_of_row=slot_of_row, slots=slot_of_row,
                   logit_rows=row_numbers, n_logit_rows=n, host={"counts": [1] * n}, req_row0=row_numbers,
                   req_count=torch.ones_like(row_numbers), req_start=positions, static_max_len=int(max_len))

    def all_single(self) -> bool:
        return self.static_max_len is not None or all(c == 1 for c in self.host.get("counts", [0]))


class _Staging:
    """A ring of pinned buffers, so a step's upload never waits for the previous one."""

    def __init__(self, device, n: int = 8, ints: int = 1 << 16):
        self.device = device
        self.bufs = [torch.empty(ints, dtype=torch.int32).pin_memory() for _ in range(n)]
        self.events = [None] * n
        self.i = 0
        self.bytes_sent = 0  # host-to-device bytes of every upload so far

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
        self.bytes_sent += 4 * n
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
        slots, wanted rows, the per-request description (first row, count, cached length) and the page-table entries
        that changed."""
        lib, pools = host.load(), self.pools
        n = len(entries)
        counts = [len(e.tokens) for e in entries]
        flat_tokens = [int(t) for e in entries for t in e.tokens]
        n_want = [len(e.want) for e in entries]
        flat_want = [int(w) for e in entries for w in e.want]
        seqs = host.ints(e.blocks.handle for e in entries)
        slots_c = host.ints(e.slot for e in entries)
        sizes = (ctypes.c_int * (N_FIXED_SECTIONS + 2 * pools.n_groups))()
        meta = (ctypes.c_int * 4)()
        args = (pools._h, n, seqs, slots_c, host.ints(counts), host.ints(flat_tokens), host.ints(n_want),
                host.ints(flat_want), self.context_length, self.vocab, self.cache.max_sequences, self.cache.table_width)
        buf = self._staging.take()
        code = lib.cuca_host_step_pack(*args, buf.data_ptr(), buf.shape[0], sizes, meta)
        if code == host.TOO_SMALL:
            buf = self._staging.take(meta[3])
            code = lib.cuca_host_step_pack(*args, buf.data_ptr(), buf.shape[0], sizes, meta)
        if code:
            raise StepError(host.last_error())
        T, S, R, total = list(meta)
        at_start = 3 * T + S + R + 2 * S  # where the requests' cached lengths stand in the buffer
        starts = buf[at_start:at_start + S].tolist()
        dev = self._staging.send(total)
        views, off = [], 0
        for k in sizes:
            views.append(dev[off:off + k])
            off += k
        for gi in range(pools.n_groups):
            idx, val = views[N_FIXED_SECTIONS + 2 * gi], views[N_FIXED_SECTIONS + 2 * gi + 1]
            if idx.shape[0]:
                ops.scatter_int(self.cache.tables[gi], idx, val)
        return StepBatch(n_rows=T, n_seqs=S, tokens=views[0], positions=views[1], seq_of_row=views[2],
                         slots=views[3], logit_rows=views[4] if R else None, n_logit_rows=R,
                         host={"counts": counts, "slots": [e.slot for e in entries], "tokens": flat_tokens,
                               "starts": starts},
                         req_row0=views[5], req_count=views[6], req_start=views[7])

    # ------------------------------------------------------------ steps whose rows already live on the device
    def check_single_tokens(self, handles, slots, tokens) -> None:
        """The host-side refusals of `build`, for a captured step that brings one token per request."""
        n = len(handles)
        self._validate_single(n, host.ints(handles), host.ints(slots), host.ints([1] * n), host.ints(tokens))

    def _validate_single(self, n, hs, ss, ones, ts) -> None:
        if host.load().cuca_host_step_validate(self.pools._h, n, hs, ss, ones, ts, self.context_length, self.vocab,
                                               self.cache.max_sequences):
            raise StepError(host.last_error())

    def upload_table_updates(self, handles, slots) -> None:
        """Page-table entries of these requests that changed since they were last sent, to the device tables."""
        self._upload_tables(len(handles), host.ints(handles), host.ints(slots))

    def _upload_tables(self, n, hs, ss) -> None:
        lib, staging, pools = host.load(), self._staging, self.pools
        for gi in range(pools.n_groups):
            buf = staging.take()
            count = lib.cuca_host_table_updates(pools._h, hs, ss, n, self.cache.table_width, gi, buf.data_ptr(),
                                                buf.shape[0])
            if count == -1:  # more new pages than the buffer holds: the widest case is every entry of every table
                buf = staging.take(2 * n * self.cache.table_width)
                count = lib.cuca_host_table_updates(pools._h, hs, ss, n, self.cache.table_width, gi, buf.data_ptr(),
                                                    buf.shape[0])
            if count < 0:
                raise StepError(host.last_error() or "page-table updates do not fit their staging buffer")
            if count > 0:
                dev = staging.send(2 * count)
                ops.scatter_int(self.cache.tables[gi], dev[:count], dev[count:])

    def advance(self, handles, counts) -> None:
        """Every request has `counts[i]` more positions cached; pages behind windows go back."""
        if host.load().cuca_host_step_advance(self.pools._h, host.ints(handles), host.ints(counts), len(handles)):
            raise StepError(host.last_error())

    def single_token_step(self, handles, slots, tokens):
        """What a captured step of one token per request needs of the host before it runs: the refusals of an eager
        step and the page-table upload, with the requests' handles and slots converted once. Returns a function
        that advances every request by one position, to be called when the step has run."""
        n = len(handles)
        hs, ss, ones = host.ints(handles), host.ints(slots), host.ints([1] * n)
        self._validate_single(n, hs, ss, ones, host.ints(tokens))
        self._upload_tables(n, hs, ss)

        def advance():
            if host.load().cuca_host_step_advance(self.pools._h, hs, ones, n):
                raise StepError(host.last_error())
        return advance

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; returns logits [wanted, vocab] (32-bit, on the device) or None if nothing is wanted."""
        if not entries:
            raise StepError("a step needs at least one request")
        batch = self.build(entries)
        logits = self.model.forward(batch, self.cache)
        self.advance([e.blocks.handle for e in entries], [len(e.tokens) for e in entries])
        self.steps += 1
        return logits

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

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.device import DeviceCache
from ..cache.pages import NO_BLOCK, KvPools, SeqBlocks
from ..kernels import ops


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

    def upload(self, arr: np.ndarray) -> torch.Tensor:
        n = arr.shape[0]
        i = self.i
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i].shape[0] < n:
            self.bufs[i] = torch.empty(max(n, 2 * self.bufs[i].shape[0]), dtype=torch.int32).pin_memory()
        self.bufs[i][:n].numpy()[:] = arr
        dev = torch.empty(n, dtype=torch.int32, device=self.device)
        dev.copy_(self.bufs[i][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


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

    # ------------------------------------------------------------ validation
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one request")
        bs = self.pools.block_size
        seen = set()
        for e in entries:
            t = len(e.tokens)
            if t == 0:
                raise StepError("a request in a step brings no tokens")
            if e.blocks.released:
                raise StepError("a request in a step has given its pages back already")
            if not 0 <= e.slot < self.cache.max_sequences:
                raise StepError(f"state slot {e.slot} is outside 0..{self.cache.max_sequences - 1}")
            if e.slot in seen:
                raise StepError(f"state slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            start = e.blocks.length
            if start + t > self.context_length:
                raise StepError(f"positions {start}..{start + t - 1} exceed the context length {self.context_length}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab:
                raise StepError(f"token id {hi if hi >= self.vocab else lo} is outside the vocabulary of {self.vocab}")
            for table in e.blocks.tables:
                if len(table) * bs < start + t:
                    raise StepError(f"the request holds pages for {len(table) * bs} positions but the step "
                                    f"writes up to position {start + t - 1}")
                first, last = start // bs, (start + t - 1) // bs
                if any(table[i] == NO_BLOCK for i in range(first, last + 1)):
                    raise StepError("a page the step writes was given back already")
            for w in e.want:
                if not 0 <= w < t:
                    raise StepError(f"wanted place {w} is outside the request's {t} tokens")

    # ------------------------------------------------------------ the step
    def build(self, entries: Sequence[StepEntry]) -> StepBatch:
        tokens, positions, slot_of_row, slots, logit_rows = [], [], [], [], []
        starts, counts = [], []
        row = 0
        for e in entries:
            t = len(e.tokens)
            start = e.blocks.length
            tokens.extend(int(x) for x in e.tokens)
            positions.extend(range(start, start + t))
            slot_of_row.extend([e.slot] * t)
            slots.append(e.slot)
            logit_rows.extend(row + int(w) for w in e.want)
            starts.append(start)
            counts.append(t)
            row += t
        T, S, R = row, len(entries), len(logit_rows)
        # attention plan: single-token requests are decode rows, longer portions are cut into tiles of 64 rows
        decode_rows, tile_row0, tile_nrows, big_row0, big_nrows, max_len = [], [], [], [], [], 1
        r0 = 0
        for start, t in zip(starts, counts):
            if t == 1:
                decode_rows.append(r0)
                max_len = max(max_len, start + 1)
            else:
                for off in range(0, t, 64):
                    tile_row0.append(r0 + off)
                    tile_nrows.append(min(64, t - off))
                for off in range(0, t, 128):
                    big_row0.append(r0 + off)
                    big_nrows.append(min(128, t - off))
            r0 += t
        # heavy tiles (late positions see most keys) first
        order = sorted(range(len(tile_row0)), key=lambda i: -positions[tile_row0[i]])
        tile_row0 = [tile_row0[i] for i in order]
        tile_nrows = [tile_nrows[i] for i in order]
        order = sorted(range(len(big_row0)), key=lambda i: -positions[big_row0[i]])
        big_row0 = [big_row0[i] for i in order]
        big_nrows = [big_nrows[i] for i in order]
        identity = len(decode_rows) == T
        # page-table entries that changed since they were last uploaded
        upd_idx, upd_val = [[] for _ in self.pools.groups], [[] for _ in self.pools.groups]
        W = self.cache.table_width
        for e in entries:
            for gi, table in enumerate(e.blocks.tables):
                lo = e.blocks.dirty_from[gi]
                if lo < len(table):
                    upd_idx[gi].extend(range(e.slot * W + lo, e.slot * W + len(table)))
                    upd_val[gi].extend(table[lo:])
                    e.blocks.dirty_from[gi] = len(table)
        parts = [tokens, positions, slot_of_row, slots, logit_rows, [] if identity else decode_rows, tile_row0,
                 tile_nrows, big_row0, big_nrows]
        n_fixed = len(parts)
        for gi in range(len(self.pools.groups)):
            parts += [upd_idx[gi], upd_val[gi]]
        sizes = [len(p) for p in parts]
        flat = np.fromiter((x for p in parts for x in p), dtype=np.int32, count=sum(sizes))
        dev = self._staging.upload(flat)
        views, off = [], 0
        for n in sizes:
            views.append(dev[off:off + n])
            off += n
        for gi in range(len(self.pools.groups)):
            idx, val = views[n_fixed + 2 * gi], views[n_fixed + 1 + 2 * gi]
            if idx.shape[0]:
                ops.scatter_int(self.cache.tables[gi], idx, val)
        return StepBatch(n_rows=T, n_seqs=S, tokens=views[0], positions=views[1], seq_of_row=views[2],
                         slots=views[3], logit_rows=views[4] if R else None, n_logit_rows=R,
                         host={"starts": starts, "counts": counts, "slots": slots, "tokens": tokens,
                               "positions": positions},
                         attention_plan=AttentionPlan(None if identity else views[5], len(decode_rows), max_len,
                                                      views[6] if tile_row0 else None,
                                                      views[7] if tile_row0 else None, len(tile_row0),
                                                      tile128_row0=views[8] if big_row0 else None,
                                                      tile128_nrows=views[9] if big_row0 else None,
                                                      n_tiles128=len(big_row0)))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one step; returns logits [wanted, vocab] (32-bit, on the device) or None if nothing is wanted."""
        self._validate(entries)
        batch = self.build(entries)
        logits = self.model.forward(batch, self.cache)
        for e in entries:
            e.blocks.length += len(e.tokens)
            self.pools.release_window(e.blocks)
        self.steps += 1
        return logits

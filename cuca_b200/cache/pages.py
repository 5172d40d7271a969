"""Host-side bookkeeping of the paged key/value cache: which request holds which page.

A page (block) is `block_size` consecutive positions of one request, for every
cache of a *group*; layers whose mixers have equal needs (key heads, head size,
window) share a group, each group has a pool of its own, and each request has
one block table per group (src/provider/local/model/paged.rs:6-16,52-103,
344-489 of the reference). Pages go back to the pool when a request ends and,
in a windowed group, as soon as the window has passed them
(model/paged.rs:736-761). No tensors live here; `cache/device.py` owns the
memory the page ids index.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

NO_BLOCK = -1  # a table entry whose page was given back (behind a window)


class PoolExhausted(RuntimeError):
    """No free page is left in a group's pool."""


class CacheBookkeepingError(AssertionError):
    """A page was freed twice, is held twice, or got lost."""


@dataclass(frozen=True)
class GroupLayout:
    """One group of caches with equal needs."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    cache_ids: tuple  # caches (run-order cache numbers) that live in this group
    n_blocks: int


class BlockPool:
    """Free list of one group's pages; pops from the back, as the reference's does."""

    def __init__(self, n_blocks: int):
        if n_blocks <= 0:
            raise ValueError("a pool needs at least one page")
        self.n_blocks = n_blocks
        self._free = list(range(n_blocks - 1, -1, -1))
        self._held = [False] * n_blocks

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return self.n_blocks - len(self._free)

    def alloc(self) -> Optional[int]:
        if not self._free:
            return None
        b = self._free.pop()
        if self._held[b]:
            raise CacheBookkeepingError(f"page {b} was on the free list while held")
        self._held[b] = True
        return b

    def release(self, b: int) -> None:
        if not 0 <= b < self.n_blocks or not self._held[b]:
            raise CacheBookkeepingError(f"page {b} is freed but not held")
        self._held[b] = False
        self._free.append(b)

    def reset(self) -> None:
        self._free = list(range(self.n_blocks - 1, -1, -1))
        self._held = [False] * self.n_blocks


@dataclass(eq=False)  # identity: two requests with equal tables are still two requests
class SeqBlocks:
    """One request's block tables (one per group) and how many positions it has cached."""

    tables: list
    length: int = 0
    released: bool = False
    first_live: list = field(default_factory=list)  # per group: index of the first table entry still held
    dirty_from: list = field(default_factory=list)  # per group: table entries from here on are not yet on the device


class KvPools:
    """All groups' pools and the requests' tables."""

    def __init__(self, groups: list, block_size: int):
        if block_size <= 0:
            raise ValueError("block size must be positive")
        self.groups = list(groups)
        self.block_size = block_size
        self.pools = [BlockPool(g.n_blocks) for g in self.groups]
        self._live: list = []

    # ------------------------------------------------------------ requests
    def new_seq(self) -> SeqBlocks:
        seq = SeqBlocks(tables=[[] for _ in self.groups], first_live=[0 for _ in self.groups],
                        dirty_from=[0 for _ in self.groups])
        self._live.append(seq)
        return seq

    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.block_size)

    def owed(self, seq: Optional[SeqBlocks], tokens: int) -> list:
        """Pages each group still has to give before the request can hold `tokens` positions."""
        need = self.blocks_for(tokens)
        if seq is None:
            return [need for _ in self.groups]
        return [max(0, need - len(t)) for t in seq.tables]

    def can_give(self, owed: list) -> bool:
        return all(p.free >= o for p, o in zip(self.pools, owed))

    def reserve(self, seq: SeqBlocks, upto: int) -> None:
        """Give the request pages for positions < upto in every group; all or nothing."""
        if seq.released:
            raise CacheBookkeepingError("reserve on a released request")
        owed = self.owed(seq, upto)
        if not self.can_give(owed):
            raise PoolExhausted("the K/V page pool is exhausted")
        for table, pool, n in zip(seq.tables, self.pools, owed):
            for _ in range(n):
                table.append(pool.alloc())

    def release_window(self, seq: SeqBlocks) -> int:
        """Give back pages that every later query of a windowed group has passed; returns how many."""
        n = 0
        for gi, (g, table, pool) in enumerate(zip(self.groups, seq.tables, self.pools)):
            if g.window is None:
                continue
            # the next query sits at position seq.length and sees keys >= length - (window - 1)
            first_needed = max(0, seq.length - (g.window - 1))
            upto = min(first_needed // self.block_size, len(table))
            for i in range(seq.first_live[gi], upto):
                if table[i] != NO_BLOCK:
                    pool.release(table[i])
                    table[i] = NO_BLOCK
                    n += 1
            seq.first_live[gi] = max(seq.first_live[gi], upto)
        return n

    def truncate(self, seq: SeqBlocks, length: int) -> None:
        """Roll the request back to `length` positions, giving back the pages beyond."""
        keep = self.blocks_for(length)
        for gi, (table, pool) in enumerate(zip(seq.tables, self.pools)):
            while len(table) > keep:
                b = table.pop()
                if b != NO_BLOCK:
                    pool.release(b)
            seq.dirty_from[gi] = min(seq.dirty_from[gi], len(table))
        seq.length = min(seq.length, length)

    def release(self, seq: SeqBlocks) -> None:
        """The request ended: every page it holds goes back."""
        if seq.released:
            raise CacheBookkeepingError("a request's pages are released twice")
        for table, pool in zip(seq.tables, self.pools):
            for b in table:
                if b != NO_BLOCK:
                    pool.release(b)
            table.clear()
        seq.released = True
        self._live.remove(seq)

    def reset(self) -> None:
        """After a failed step: forget every request, every page is free again."""
        for p in self.pools:
            p.reset()
        for s in self._live:
            s.released = True
            for t in s.tables:
                t.clear()
        self._live.clear()

    # ------------------------------------------------------------ accounting
    def check(self) -> None:
        """Every page is either free or held by exactly one live request."""
        for gi, pool in enumerate(self.pools):
            held = {}
            for s in self._live:
                for b in s.tables[gi]:
                    if b == NO_BLOCK:
                        continue
                    if b in held:
                        raise CacheBookkeepingError(f"group {gi}: page {b} is held twice")
                    held[b] = s
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise CacheBookkeepingError(f"group {gi}: a page is on the free list twice")
            if free & set(held):
                raise CacheBookkeepingError(f"group {gi}: pages {sorted(free & set(held))} are free and held")
            if len(free) + len(held) != pool.n_blocks:
                lost = set(range(pool.n_blocks)) - free - set(held)
                raise CacheBookkeepingError(f"group {gi}: pages {sorted(lost)} are lost")

    def stats(self) -> dict:
        return {"free_blocks": [p.free for p in self.pools], "used_blocks": [p.used for p in self.pools],
                "total_blocks": [p.n_blocks for p in self.pools], "live_requests": len(self._live)}


class StateSlots:
    """Fixed-size per-request state: slot ids 0..max_sequences-1, handed out last-in first-out
    (src/provider/local/model/mod.rs:247-251, engine/scheduler.rs:741-750,890-891)."""

    def __init__(self, max_sequences: int):
        self.max_sequences = max_sequences
        self._free = list(range(max_sequences))
        self._held = [False] * max_sequences

    @property
    def free(self) -> int:
        return len(self._free)

    def alloc(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.max_sequences or not self._held[slot]:
            raise CacheBookkeepingError(f"state slot {slot} is freed but not held")
        self._held[slot] = False
        self._free.append(slot)

    def reset(self) -> None:
        self._free = list(range(self.max_sequences))
        self._held = [False] * self.max_sequences

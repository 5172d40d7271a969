"""Host-side bookkeeping of the paged key/value cache: which request holds which page.

A page (block) is `block_size` consecutive positions of one request, for every
cache of a *group*; layers whose mixers have equal needs (key heads, head size,
window) share a group, each group has a pool of its own, and each request has
one block table per group (src/provider/local/model/paged.rs:6-16,52-103,
344-489 of the reference). Pages go back to the pool when a request ends and,
in a windowed group, as soon as the window has passed them
(model/paged.rs:736-761). No tensors live here; `cache/device.py` owns the
memory the page ids index.

The books themselves are kept by the C++ host core (`csrc/host/kv_pools.cpp`);
the classes here hold a handle and translate its status codes into exceptions.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

from ..native import host

NO_BLOCK = -1  # a table entry whose page was given back (behind a window)


class PoolExhausted(RuntimeError):
    """No free page is left in a group's pool."""


class StatefulCacheError(ValueError):
    """Asked of pages what only works when pages are all a request keeps: some mixer also keeps state."""


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


def _raise(code: int) -> None:
    msg = host.last_error()
    if code == host.EXHAUSTED:
        raise PoolExhausted(msg or "the K/V page pool is exhausted")
    raise CacheBookkeepingError(msg or f"cache bookkeeping error {code}")


class BlockPool:
    """Free list of one group's pages; pops from the back, as the reference's does."""

    def __init__(self, n_blocks: int):
        if n_blocks <= 0:
            raise ValueError("a pool needs at least one page")
        self.n_blocks = n_blocks
        self._lib = host.load()
        self._h = self._lib.cuca_host_blockpool_new(n_blocks)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.cuca_host_blockpool_free(self._h)
            self._h = None

    @property
    def free(self) -> int:
        return self._lib.cuca_host_blockpool_free_count(self._h)

    @property
    def used(self) -> int:
        return self.n_blocks - self.free

    def alloc(self) -> Optional[int]:
        b = self._lib.cuca_host_blockpool_alloc(self._h)
        if b == -2:
            raise CacheBookkeepingError("a page was on the free list while held")
        return None if b < 0 else b

    def release(self, b: int) -> None:
        if self._lib.cuca_host_blockpool_release(self._h, int(b)) != 0:
            raise CacheBookkeepingError(f"page {b} is freed but not held")

    def reset(self) -> None:
        self._lib.cuca_host_blockpool_reset(self._h)


class _GroupPool:
    """One group's pool inside `KvPools`, for reading its counts."""

    def __init__(self, pools: "KvPools", gi: int):
        self._pools, self._gi = pools, gi

    @property
    def n_blocks(self) -> int:
        return self._pools._lib.cuca_host_pools_total_blocks(self._pools._h, self._gi)

    @property
    def free(self) -> int:
        return self._pools._lib.cuca_host_pools_free_blocks(self._pools._h, self._gi)

    @property
    def used(self) -> int:
        return self.n_blocks - self.free

    @property
    def cached(self) -> int:
        """Unreferenced pages kept for their name (counted in `free`: an allocation may take them)."""
        return self._pools._lib.cuca_host_pools_cached_blocks(self._pools._h, self._gi)


class _PerGroup:
    """`first_live` / `dirty_from` of a request: a list-like view of one integer per group."""

    def __init__(self, seq: "SeqBlocks", base: int):
        self._seq, self._base = seq, base

    def __len__(self):
        return self._seq._pools.n_groups

    def __getitem__(self, gi: int) -> int:
        return self._seq._get(self._base + range(len(self))[gi])

    def __setitem__(self, gi: int, value: int) -> None:
        self._seq._set(self._base + range(len(self))[gi], int(value))

    def __iter__(self):
        return (self[i] for i in range(len(self)))

    def __eq__(self, other):
        return list(self) == list(other)

    def __repr__(self):
        return repr(list(self))


class SeqBlocks:
    """One request's block tables (one per group) and how many positions it has cached.

    Identity is the handle: two requests with equal tables are still two requests."""

    __slots__ = ("_pools", "handle", "_owns", "__weakref__")

    def __init__(self, pools: "KvPools", handle: int, owns: bool = True):
        self._pools, self.handle, self._owns = pools, handle, owns

    def __del__(self):
        # the record goes back to the host core with its last owner (tables the scheduler made are the scheduler's)
        try:
            pools = self._pools
            if self._owns and pools._h:
                pools._lib.cuca_host_pools_drop_seq(pools._h, self.handle)
        except Exception:  # interpreter shutdown
            pass

    def _get(self, field: int) -> int:
        return self._pools._lib.cuca_host_seq_get(self._pools._h, self.handle, field)

    def _set(self, field: int, value: int) -> None:
        if self._pools._lib.cuca_host_seq_set(self._pools._h, self.handle, field, value) != 0:
            raise CacheBookkeepingError(host.last_error())

    @property
    def length(self) -> int:
        return self._get(0)

    @length.setter
    def length(self, value: int) -> None:
        self._set(0, int(value))

    @property
    def released(self) -> bool:
        return self._get(1) != 0

    @property
    def tables(self) -> list:
        """A copy of the request's tables: one list of page ids per group."""
        lib, h = self._pools._lib, self._pools._h
        out = []
        for gi in range(self._pools.n_groups):
            n = lib.cuca_host_seq_table(h, self.handle, gi, None, 0)
            buf = (ctypes.c_int * max(1, n))()
            lib.cuca_host_seq_table(h, self.handle, gi, buf, n)
            out.append(list(buf[:n]))
        return out

    @property
    def first_live(self):
        return _PerGroup(self, 2)

    @property
    def dirty_from(self):
        return _PerGroup(self, 2 + self._pools.n_groups)

    @dirty_from.setter
    def dirty_from(self, values) -> None:
        for gi, v in enumerate(values):
            self._set(2 + self._pools.n_groups + gi, int(v))


class KvPools:
    """All groups' pools and the requests' tables."""

    def __init__(self, groups: list, block_size: int):
        if block_size <= 0:
            raise ValueError("block size must be positive")
        self.groups = list(groups)
        self.block_size = block_size
        self.n_groups = len(self.groups)
        for g in self.groups:
            if g.n_blocks <= 0:
                raise ValueError("a pool needs at least one page")
        self._lib = host.load()
        self._h = self._lib.cuca_host_pools_new(
            self.n_groups, host.ints(g.n_blocks for g in self.groups),
            host.ints(-1 if g.window is None else int(g.window) for g in self.groups), block_size)
        if not self._h:
            raise ValueError("the page pools could not be made")
        self.pools = [_GroupPool(self, gi) for gi in range(self.n_groups)]
        # True when some mixer of the model keeps per-request state of fixed size besides these pages: what
        # rests on "the pages are all a request has" (rolling back, starting from cached pages) is refused then
        self.stateful = False

    def __del__(self):
        if getattr(self, "_h", None):
            h, self._h = self._h, None
            self._lib.cuca_host_pools_free(h)

    # ------------------------------------------------------------ requests
    def new_seq(self) -> SeqBlocks:
        return SeqBlocks(self, self._lib.cuca_host_pools_new_seq(self._h))

    def new_seq_with_prefix(self, prompt) -> SeqBlocks:
        """A new request that starts with the longest cached prefix of `prompt` (whole pages, at most
        len(prompt) - 1 positions): its tables share those pages and `length` says how many positions they hold."""
        prompt = [int(t) for t in prompt]
        return SeqBlocks(self, self._lib.cuca_host_pools_new_seq_with_prefix(self._h, host.ints(prompt), len(prompt)))

    def publish(self, seq: SeqBlocks, ids) -> None:
        """Name every full page of the request (`ids`: the tokens at its cached positions) for later prompts."""
        ids = [int(t) for t in ids]
        code = self._lib.cuca_host_pools_publish(self._h, seq.handle, host.ints(ids), len(ids))
        if code:
            _raise(code)

    def finish(self, seq: SeqBlocks, ids) -> None:
        """`publish`, then `release`: the request's full pages stay in the pool as cached."""
        ids = [int(t) for t in ids]
        code = self._lib.cuca_host_pools_finish(self._h, seq.handle, host.ints(ids), len(ids))
        if code:
            _raise(code)

    def adopt(self, handle: int) -> SeqBlocks:
        """A view of tables that the host core made itself (the scheduler admits requests there)."""
        return SeqBlocks(self, handle, owns=False)

    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.block_size)

    def owed(self, seq: Optional[SeqBlocks], tokens: int) -> list:
        """Pages each group still has to give before the request can hold `tokens` positions."""
        out = (ctypes.c_int * max(1, self.n_groups))()
        self._lib.cuca_host_pools_owed(self._h, -1 if seq is None else seq.handle, int(tokens), out)
        return list(out[:self.n_groups])

    def can_give(self, owed: list) -> bool:
        return bool(self._lib.cuca_host_pools_can_give(self._h, host.ints(owed)))

    def reserve(self, seq: SeqBlocks, upto: int) -> None:
        """Give the request pages for positions < upto in every group; all or nothing."""
        code = self._lib.cuca_host_pools_reserve(self._h, seq.handle, int(upto))
        if code:
            _raise(code)

    def release_window(self, seq: SeqBlocks) -> int:
        """Give back pages that every later query of a windowed group has passed; returns how many."""
        n = self._lib.cuca_host_pools_release_window(self._h, seq.handle)
        if n < 0:
            _raise(host.BOOKKEEPING)
        return n

    def truncate(self, seq: SeqBlocks, length: int) -> None:
        """Roll the request back to `length` positions, giving back the pages beyond. Refused when some mixer
        keeps per-request state of fixed size: pages can be cut back, a running state cannot."""
        if self.stateful:
            raise StatefulCacheError("a request cannot be rolled back: a mixer of this model keeps per-request state "
                            "besides its pages, and that state has moved on")
        code = self._lib.cuca_host_pools_truncate(self._h, seq.handle, int(length))
        if code:
            _raise(code)

    def release(self, seq: SeqBlocks) -> None:
        """The request ended: every page it holds goes back."""
        code = self._lib.cuca_host_pools_release(self._h, seq.handle)
        if code:
            _raise(code)

    def reset(self) -> None:
        """After a failed step: forget every request, every page is free again."""
        self._lib.cuca_host_pools_reset(self._h)

    # ------------------------------------------------------------ accounting
    def check(self) -> None:
        """Every page is either free or held by exactly one live request."""
        code = self._lib.cuca_host_pools_check(self._h)
        if code:
            _raise(code)

    def stats(self) -> dict:
        return {"free_blocks": [p.free for p in self.pools], "used_blocks": [p.used for p in self.pools],
                "total_blocks": [p.n_blocks for p in self.pools], "cached_blocks": [p.cached for p in self.pools],
                "live_requests": self._lib.cuca_host_pools_live(self._h)}


class StateSlots:
    """Fixed-size per-request state: slot ids 0..max_sequences-1, handed out last-in first-out
    (src/provider/local/model/mod.rs:247-251, engine/scheduler.rs:741-750,890-891)."""

    def __init__(self, max_sequences: int):
        self.max_sequences = max_sequences
        self._lib = host.load()
        self._h = self._lib.cuca_host_slots_new(max_sequences)

    def __del__(self):
        if getattr(self, "_h", None):
            h, self._h = self._h, None
            self._lib.cuca_host_slots_free(h)

    @property
    def free(self) -> int:
        return self._lib.cuca_host_slots_free_count(self._h)

    def alloc(self) -> Optional[int]:
        s = self._lib.cuca_host_slots_alloc(self._h)
        return None if s < 0 else s

    def release(self, slot: int) -> None:
        if self._lib.cuca_host_slots_release(self._h, int(slot)) != 0:
            raise CacheBookkeepingError(f"state slot {slot} is freed but not held")

    def reset(self) -> None:
        self._lib.cuca_host_slots_reset(self._h)

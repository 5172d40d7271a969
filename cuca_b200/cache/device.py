"""Device memory of the cache: one pair of slabs per group, state arrays per cache.

Keys and values of a group live in two slabs `[caches, pages, kv heads,
block, head_dim]`; a page id indexes the same rows in every cache of its group
(src/provider/local/model/paged.rs:6-16; pool layout model/cpu.rs:678-714).
Per-request state of fixed size lives in `[max_sequences, ...]` arrays indexed
by the request's slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .pages import GroupLayout

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


def plan_groups(cache_needs: dict, kv_tokens: int, block_size: int, max_sequences: int,
                max_step_tokens: int, window_pools: str = "sized") -> list:
    """Group caches by (key heads, head size, window) and size each group's pool.

    A group that keeps all keys gets ceil(kv_tokens / block) pages. A windowed
    group needs at most `max_sequences * (ceil((w - 1 + max_step_tokens) / block) + 2)`
    pages (src/provider/local/model/paged.rs:175-220); `window_pools="full"` sizes
    it like a full group instead.
    """
    by_key: dict = {}
    for cid in sorted(cache_needs):
        kv = cache_needs[cid].kv
        if kv is None:
            continue
        by_key.setdefault((kv.n_kv_heads, kv.head_dim, kv.window), []).append(cid)
    full = -(-kv_tokens // block_size)
    groups = []
    for (nkv, d, window), ids in by_key.items():
        n = full
        if window is not None and window_pools == "sized":
            n = min(full, max_sequences * (-(-(window - 1 + max_step_tokens) // block_size) + 2))
        groups.append(GroupLayout(nkv, d, window, tuple(ids), max(1, n)))
    return groups


@dataclass
class CacheView:
    """What one run of a layer sees of the cache during a step."""

    k: Optional[torch.Tensor]  # [pages, kv heads, block, head_dim]
    v: Optional[torch.Tensor]
    tables: Optional[torch.Tensor]  # [max_sequences, width] int32: this group's page ids, one row per slot
    block_size: int
    group: int
    state: Optional[torch.Tensor]  # [max_sequences, ...] this cache's per-request state
    slots: Optional[torch.Tensor]  # [requests in the step] int32 slot of each request (a row's is step.seq_of_row)


class DeviceCache:
    def __init__(self, runtime, groups: list, block_size: int, cache_needs: dict, max_sequences: int,
                 context_length: int):
        self.rt = runtime
        self.groups = groups
        self.block_size = block_size
        self.max_sequences = max_sequences
        self.table_width = -(-context_length // block_size)
        self.k, self.v = [], []
        self._where = {}
        # page tables live on the device, one row per slot; a step only uploads the entries that changed
        self.tables = [torch.full((max_sequences, self.table_width), -1, dtype=torch.int32, device=runtime.device)
                       for _ in groups]
        for gi, g in enumerate(groups):
            shape = (len(g.cache_ids), g.n_blocks, g.n_kv_heads, block_size, g.head_dim)
            self.k.append(torch.zeros(shape, dtype=runtime.dtype, device=runtime.device))
            self.v.append(torch.zeros(shape, dtype=runtime.dtype, device=runtime.device))
            for j, cid in enumerate(g.cache_ids):
                self._where[cid] = (gi, j)
        self.state = {}
        for cid, needs in cache_needs.items():
            if needs.state is not None:
                self.state[cid] = torch.zeros((max_sequences, *needs.state.shape),
                                              dtype=_STATE_DTYPES[needs.state.dtype], device=runtime.device)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v) + \
            sum(t.numel() * t.element_size() for t in self.state.values())

    def bytes_per_token(self) -> int:
        """Key/value bytes one cached position occupies over all caches."""
        return sum(2 * len(g.cache_ids) * g.n_kv_heads * g.head_dim * self.k[i].element_size()
                   for i, g in enumerate(self.groups))

    def clear_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    def view(self, cache_id: int, step) -> CacheView:
        gi, j = self._where.get(cache_id, (None, None))
        if gi is None:
            return CacheView(None, None, None, self.block_size, -1, self.state.get(cache_id), step.slots)
        return CacheView(self.k[gi][j], self.v[gi][j], self.tables[gi], self.block_size, gi,
                         self.state.get(cache_id), step.slots)

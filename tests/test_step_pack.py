"""The host core's step packer (csrc/host/step_pack.cpp) without a GPU: what goes into the one buffer a step
uploads, and what is refused before anything changes."""
import ctypes

import numpy as np
import pytest

from cuca_b200.cache.pages import GroupLayout, KvPools
from cuca_b200.native import host


def _pack(pools, entries, context=256, vocab=100, max_sequences=8, width=16, cap=4096):
    """entries: (SeqBlocks, slot, tokens, want). Returns (code, sections, meta)."""
    lib = host.load()
    out = np.full(cap, -7, dtype=np.int32)
    sizes = (ctypes.c_int * (8 + 2 * pools.n_groups))()
    meta = (ctypes.c_int * 4)()
    code = lib.cuca_host_step_pack(
        pools._h, len(entries), host.ints(e[0].handle for e in entries), host.ints(e[1] for e in entries),
        host.ints(len(e[2]) for e in entries), host.ints(t for e in entries for t in e[2]),
        host.ints(len(e[3]) for e in entries), host.ints(w for e in entries for w in e[3]),
        context, vocab, max_sequences, width, out.ctypes.data, cap, sizes, meta)
    sections, off = [], 0
    for k in sizes:
        sections.append(out[off:off + k].tolist())
        off += k
    return code, sections, list(meta)


def _pools(window=None):
    groups = [GroupLayout(2, 16, None, (0,), 32)]
    if window:
        groups.append(GroupLayout(1, 16, window, (1,), 32))
    return KvPools(groups, 8)


def test_a_mixed_step_is_packed_into_sections():
    kv = _pools()
    a, b, c = kv.new_seq(), kv.new_seq(), kv.new_seq()
    kv.reserve(a, 10)          # a decodes its 10th token
    a.length = 9
    kv.reserve(b, 150)         # b brings 150 prompt tokens
    kv.reserve(c, 21)          # c has 20 cached and brings one token
    c.length = 20
    code, sec, meta = _pack(kv, [(a, 3, [5], [0]), (b, 0, list(range(50)) * 3, [149]), (c, 7, [9], [])])
    assert code == 0
    rows, requests, wanted, total = meta
    assert (rows, requests, wanted) == (152, 3, 2)
    tokens, positions, slot_of_row, slots, logit_rows, req_row0, req_count, req_start = sec[:8]
    assert tokens[0] == 5 and tokens[1:151] == list(range(50)) * 3 and tokens[151] == 9
    assert positions == [9] + list(range(150)) + [20]
    assert slot_of_row == [3] + [0] * 150 + [7] and slots == [3, 0, 7]
    assert logit_rows == [0, 150]
    # the per-request description every mixer plans from: first row, tokens brought, positions cached before
    assert (req_row0, req_count, req_start) == ([0, 1, 151], [1, 150, 1], [9, 0, 20])
    # page-table entries: all of them are new; they are marked as sent
    idx, val = sec[8], sec[9]
    assert idx == [3 * 16, 3 * 16 + 1] + list(range(19)) + [7 * 16 + i for i in range(3)]
    assert val == a.tables[0] + b.tables[0] + c.tables[0]
    assert list(a.dirty_from) == [2] and list(b.dirty_from) == [19]
    assert total == sum(len(s) for s in sec)
    # nothing is new the second time
    code, sec, _ = _pack(kv, [(a, 3, [5], [0])])
    assert code == 0 and sec[8] == [] and sec[5:8] == [[0], [1], [9]]


def test_refusals_change_nothing():
    kv = _pools(window=16)
    a = kv.new_seq()
    kv.reserve(a, 16)
    cases = [
        ([], "at least one request"),
        ([(a, 0, [], [])], "no tokens"),
        ([(a, 9, [1], [])], "slot 9"),
        ([(a, 0, [1], []), (a, 0, [1], [])], "twice"),
        ([(a, 0, [100], [])], "vocabulary"),
        ([(a, 0, [-1], [])], "vocabulary"),
        ([(a, 0, [1] * 17, [])], "pages for 16 positions"),
        ([(a, 0, [1, 2], [2])], "wanted place 2"),
    ]
    for entries, why in cases:
        code, _, _ = _pack(kv, entries)
        assert code == host.INVALID and why in host.last_error(), (why, host.last_error())
        assert list(a.dirty_from) == [0, 0] and a.length == 0
    code, _, _ = _pack(kv, [(a, 0, [1] * 16, [])], context=10)
    assert code == host.INVALID and "context length 10" in host.last_error()
    # a page behind the window was given back: a step may not write there
    a.length = 40
    kv.reserve(a, 48)
    assert kv.release_window(a) == 3
    a.length = 8
    code, _, _ = _pack(kv, [(a, 0, [1], [])])
    assert code == host.INVALID and "given back" in host.last_error()
    b = kv.new_seq()
    kv.reserve(b, 8)
    kv.release(b)
    code, _, _ = _pack(kv, [(b, 1, [1], [])])
    assert code == host.INVALID and "given its pages back" in host.last_error()


def test_a_buffer_too_small_reports_what_is_needed():
    kv = _pools()
    a = kv.new_seq()
    kv.reserve(a, 64)
    code, _, meta = _pack(kv, [(a, 0, [1] * 64, [63])], cap=10)
    assert code == host.TOO_SMALL and meta[3] == 3 * 64 + 1 + 1 + 3 + 2 * 8
    assert list(a.dirty_from) == [0]                       # nothing was marked as sent
    code, sec, _ = _pack(kv, [(a, 0, [1] * 64, [63])], cap=meta[3])
    assert code == 0 and sec[8] == list(range(8))


@pytest.mark.parametrize("seed", [0, 1])
def test_advance_moves_lengths_and_releases_behind_windows(seed):
    kv = _pools(window=12)
    lib = host.load()
    a, b = kv.new_seq(), kv.new_seq()
    kv.reserve(a, 40)
    kv.reserve(b, 8)
    assert lib.cuca_host_step_advance(kv._h, host.ints([a.handle, b.handle]), host.ints([40, 3]), 2) == 0
    assert (a.length, b.length) == (40, 3)
    assert a.tables[1][:3] == [-1, -1, -1] and a.tables[1][3] != -1 and all(x != -1 for x in a.tables[0])
    kv.check()


def test_validation_alone_for_steps_that_live_on_the_device():
    """A captured decode step brings one token per request from device buffers; the host still refuses what it
    would refuse of a packed step (token range, context, missing pages), and nothing is marked as sent."""
    kv = _pools()
    lib = host.load()
    a = kv.new_seq()
    kv.reserve(a, 9)
    a.length = 8

    def check(tokens, context=256):
        return lib.cuca_host_step_validate(kv._h, 1, host.ints([a.handle]), host.ints([2]), host.ints([1]),
                                           host.ints(tokens), context, 100, 8)

    assert check([5]) == 0 and list(a.dirty_from) == [0]
    assert check([100]) == host.INVALID and "vocabulary" in host.last_error()
    assert check([5], context=8) == host.INVALID and "context length 8" in host.last_error()
    a.length = 16
    assert check([5]) == host.INVALID and "pages for 16 positions" in host.last_error()

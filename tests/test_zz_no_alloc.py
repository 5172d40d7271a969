"""The allocation-free decode attention entry point, called through its exported C symbol.

Some users of this library cannot call cudaMalloc where they call us: a plugin invoked inside someone else's
graph capture, a real-time loop, a host with a memory pool of its own. `cuca_attention_decode_noalloc` keeps its
scratch inside the library image instead of asking for a buffer. This test drives it with ctypes only (no
wrapper of the package), twice in a row, and compares with `cuca_attention_decode` given ordinary scratch.

The file name sorts last on purpose: if this entry point is broken, every other test has run before it fails.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from cuca_b200.kernels import build
    lib = ctypes.CDLL(str(build.build(verbose=False)))
    P, I, F = c_void_p, c_int, c_float
    common = [P, I, P, I, P, P, I, I, P, P, P, I, P, I, I, I, I, F, I, I, I]
    lib.cuca_attention_decode.argtypes = common + [P, P, P, P]
    lib.cuca_attention_decode.restype = I
    lib.cuca_attention_decode_noalloc.argtypes = common + [P, P]
    lib.cuca_attention_decode_noalloc.restype = I
    lib.cuca_last_error.restype = ctypes.c_char_p
    return lib


def _problem(dev, n_rows, nh, nkv, d, bs, lens, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    n_blocks = sum(-(-l // bs) for l in lens) + 2
    kpool = torch.randn(n_blocks, nkv, bs, d, device=dev, generator=g).bfloat16()
    vpool = torch.randn(n_blocks, nkv, bs, d, device=dev, generator=g).bfloat16()
    width = max(-(-l // bs) for l in lens)
    tables = torch.full((n_rows, width), -1, dtype=torch.int32, device=dev)
    perm = torch.randperm(n_blocks, device=dev, generator=g).tolist()
    k = 0
    for s, l in enumerate(lens):
        for b in range(-(-l // bs)):
            tables[s, b] = perm[k]
            k += 1
    q = torch.randn(n_rows, nh * d, device=dev, generator=g).bfloat16()
    positions = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
    seq = torch.arange(n_rows, dtype=torch.int32, device=dev)
    return q, kpool, vpool, tables, positions, seq


def test_noalloc_entry_point_matches_the_ordinary_one_twice():
    lib = _lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    nh, nkv, d, bs, chunk = 8, 2, 64, 16, 64
    stream = torch.cuda.current_stream().cuda_stream
    for call, lens in enumerate(([300, 17, 129, 64, 1], [5, 500, 260, 31, 192])):
        n_rows = len(lens)
        q, kpool, vpool, tables, positions, seq = _problem(dev, n_rows, nh, nkv, d, bs, lens, seed=call)
        n_splits = -(-max(lens) // chunk)
        want = torch.zeros(n_rows, nh * d, device=dev, dtype=torch.bfloat16)
        got = torch.zeros_like(want)
        part = torch.empty(n_rows * nh * n_splits * (d + 2), dtype=torch.float32, device=dev)
        counters = torch.zeros(n_rows * nkv, dtype=torch.int32, device=dev)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        args = (q.data_ptr(), nh * d, None, nh * d, kpool.data_ptr(), vpool.data_ptr(), kpool.shape[0], bs,
                positions.data_ptr(), seq.data_ptr(), tables.data_ptr(), tables.shape[1], None, n_rows, nh, nkv, d,
                1.0 / math.sqrt(d), 0, chunk, n_splits)

        def with_out(t):
            return args[:2] + (t.data_ptr(),) + args[3:]

        rc = lib.cuca_attention_decode(*with_out(want), part.data_ptr(), counters.data_ptr(), err.data_ptr(), stream)
        assert rc == 0, lib.cuca_last_error()
        rc = lib.cuca_attention_decode_noalloc(*with_out(got), err.data_ptr(), stream)
        assert rc == 0, lib.cuca_last_error()
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        assert float(want.float().abs().max()) > 0
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), f"call {call}"


def test_noalloc_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    dev = torch.device("cuda:0")
    dummy = torch.zeros(16, dtype=torch.int32, device=dev)
    p = dummy.data_ptr()
    # 64 rows x 32 heads x 64 chunks x (128 + 2) floats is far beyond the built-in 1 Mi floats
    rc = lib.cuca_attention_decode_noalloc(p, 4096, p, 4096, p, p, 8, 16, p, p, p, 8, None, 64, 32, 8, 128, 0.1, 0, 64,
                                           64, p, torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    assert b"built-in scratch" in lib.cuca_last_error()

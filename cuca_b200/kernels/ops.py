"""Thin Python wrappers over the kernel library: tensors in, launches out.

Each function checks what the kernel cannot (device, dtype, contiguity) and
launches on torch's current stream. Nothing here computes on the host or falls
back to torch operators.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import library

F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
_CODES = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise library.KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle. Asked of torch's C entry where there is one: `torch.cuda.current_stream()` builds
    a Python object per call, 2.5 us of the 19 us of host time that a launch cost (a prompt step of a few tokens is
    230 launches whose kernels take 16 us each: the host set its pace)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise library.KernelError("kernel arguments must live on the CUDA device (there is no CPU path)")


def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    _cuda(table, tokens, out)
    lib = library.load()
    V, E = table.shape
    library.check(lib.cuca_embed(_p(table), dtype_code(table.dtype), _p(tokens), _p(out), tokens.shape[0], E, V,
                                 _p(err), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows=None) -> None:
    _cuda(x, weight, out)
    lib = library.load()
    n = out.shape[0] if rows is None else rows.shape[0]
    library.check(lib.cuca_rmsnorm(_p(x), _p(weight), dtype_code(weight.dtype), _p(out), dtype_code(out.dtype),
                                   _p(rows), n, x.shape[-1], float(eps), _stream()), "rmsnorm")


def rope_store(qkv, positions, seq_of_row, tables, cos, sin, rotary_dim, kpool, vpool, block_size,
               n_heads, n_kv_heads, head_dim, err) -> None:
    """Rotate q (in place) and k, write k and v to their pages. `tables` is [S, width] int32;
    pools are [n_blocks, n_kv_heads, block_size, head_dim] (None with n_kv_heads == 0)."""
    _cuda(qkv, positions, seq_of_row)
    lib = library.load()
    n_blocks = kpool.shape[0] if kpool is not None else 0
    table_rows = cos.shape[0] if cos is not None else 0
    library.check(lib.cuca_rope_store(
        _p(qkv), dtype_code(qkv.dtype), _p(positions), _p(seq_of_row), _p(tables),
        tables.shape[1] if tables is not None else 0, _p(cos), _p(sin), table_rows, int(rotary_dim),
        _p(kpool), _p(vpool), n_blocks, int(block_size), qkv.shape[0], n_heads, n_kv_heads, head_dim,
        _p(err), _stream()), "rope_store")


def random_normal(out: torch.Tensor, key: int, first: int, mean: float, scale: float) -> None:
    """out.view(-1)[i] = mean + normal(key, first + i) * (2 * 65536 * scale): the counter-based generator of the
    random-weights mode (`weights/loader.py:host_normal` is its host form, bit for bit)."""
    _cuda(out)
    lib = library.load()
    library.check(lib.cuca_random_normal(_p(out), dtype_code(out.dtype), out.numel(), int(first), int(key),
                                         float(mean), float(scale), _stream()), "random_normal")


def swiglu(gate_up, out) -> None:
    _cuda(gate_up, out)
    lib = library.load()
    library.check(lib.cuca_swiglu(_p(gate_up), _p(out), dtype_code(out.dtype), out.shape[0], out.shape[1],
                                  _stream()), "swiglu")


def add_to_stream(x, delta) -> None:
    _cuda(x, delta)
    lib = library.load()
    library.check(lib.cuca_add_to_stream(_p(x), _p(delta), dtype_code(delta.dtype), x.numel(), _stream()),
                  "add_to_stream")


def gemm_simt(a, w, out, epilogue=EPI_STORE, bias=None) -> None:
    """out = epilogue(a @ w.T) on CUDA cores; a: [M, K] (row stride >= K), w: [N or 2N, K]."""
    _cuda(a, w, out)
    lib = library.load()
    M, K = a.shape
    N = out.shape[1]
    library.check(lib.cuca_gemm_simt(_p(a), _p(w), _p(bias), _p(out), dtype_code(a.dtype), dtype_code(out.dtype),
                                     M, N, K, a.stride(0), out.stride(0), epilogue, _stream()), "gemm_simt")


def attention_generic(q, q_stride, out, kpool, vpool, positions, seq_of_row, tables, n_heads, n_kv_heads,
                      head_dim, scale, window, err) -> None:
    _cuda(q, out, kpool, vpool)
    lib = library.load()
    library.check(lib.cuca_attention_generic(
        _p(q), int(q_stride), _p(out), out.stride(0), dtype_code(out.dtype), _p(kpool), _p(vpool), kpool.shape[0],
        kpool.shape[2], _p(positions), _p(seq_of_row), _p(tables), tables.shape[1], out.shape[0], n_heads,
        n_kv_heads, head_dim, float(scale), int(window or 0), _p(err), _stream()), "attention_generic")


def argmax(logits, out) -> None:
    _cuda(logits, out)
    lib = library.load()
    library.check(lib.cuca_argmax(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(out),
                                  _stream()), "argmax")


_scratch: dict = {}
WORKSPACE_BYTES = 48 << 20
N_COUNTERS = 1024


def gemm_scratch(device):
    """Split-K scratch of the tensor-core contraction: 32-bit partial tiles and per-tile arrival counters
    (zeroed once; the kernel leaves them zeroed)."""
    key = (device.type, device.index)
    if key not in _scratch:
        _scratch[key] = (torch.empty(WORKSPACE_BYTES // 4, dtype=torch.float32, device=device),
                         torch.zeros(N_COUNTERS, dtype=torch.int32, device=device))
    return _scratch[key]


_tc_supported: dict = {}


def gemm_tc_supported(a, w) -> bool:
    """Whether the tensor-core kernel takes this problem (the library's answer, remembered by what it depends on:
    K, the row stride, the operands' alignment and whether the problem is empty)."""
    pa, pw = a.data_ptr(), w.data_ptr()
    key = (a.shape[1], a.stride(0), pa & 15, pw & 15, a.shape[0] > 0, w.shape[0] > 0)
    ok = _tc_supported.get(key)
    if ok is None:
        lib = library.load()
        ok = _tc_supported[key] = bool(lib.cuca_gemm_tc_supported(pa, pw, a.shape[0], w.shape[0], a.shape[1], a.stride(0)))
    return ok


def gemm_tc(a, w, out, epilogue=EPI_STORE, bias=None, err=None, max_splits=16) -> None:
    """out = epilogue(a @ w.T) on the tcgen05 tensor cores; bf16 operands, K and the row stride multiples of 8."""
    _cuda(a, w, out)
    lib = library.load()
    M, K = a.shape
    N = out.shape[1]
    ws, counters = gemm_scratch(a.device)
    library.check(lib.cuca_gemm_tc(_p(a), _p(w), _p(bias), _p(out), dtype_code(out.dtype), M, N, K, a.stride(0),
                                   out.stride(0), epilogue, _p(ws), ws.numel() * 4, _p(counters), counters.numel(),
                                   int(max_splits), _p(err), _stream()), "gemm_tc")


def gemm_pair_mode(mode: int) -> None:
    """When contractions over many tokens run as pairs of CTAs on one tile (`tcgen05.mma.cta_group::2`): 1 where
    the library's rule expects them to be faster, 0 never, 2 wherever they can (tests and measurements), -1 as the
    environment variable CUCA_GEMM_PAIR says."""
    library.load().cuca_gemm_pair_mode(int(mode))
    _partial_slices.clear()  # what was remembered of the library's choices depended on the mode
    _partial_max.clear()


def gemm(a, w, out, epilogue=EPI_STORE, bias=None, err=None) -> None:
    """out = epilogue(a @ w.T), on the kernel that fits dtype and shape: tensor cores for bfloat16
    (rows of 16-byte multiples), CUDA cores for the 32-bit path and for shapes the former refuses."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16) \
            and gemm_tc_supported(a, w):
        gemm_tc(a, w, out, epilogue, bias, err)
    else:
        gemm_simt(a, w, out, epilogue, bias)


class AttentionPlan:
    """How a step's rows are handed to the attention kernels, derived from the step's per-request description:
    requests that bring one token go to the split-key decode form (their row numbers; None when every row is
    one), longer portions in tiles of consecutive rows to a prefill form. The tile heights are the kernel
    library's; the lists are made on the device (`cuca_attention_plan`), the counts on the host from the same
    per-request counts. One plan serves every attention layer of a step; tiles of a height and the key chunking
    for a (key heads, head size) pair are made when first asked for."""

    def __init__(self, step):
        counts = step.host["counts"]
        self.step = step
        self.static = step.static_max_len is not None
        if self.static:
            self.n_decode, self.max_len = step.n_rows, step.static_max_len
            self.n_portions = 0
        else:
            starts = step.host["starts"]
            single = [s + 1 for c, s in zip(counts, starts) if c == 1]
            self.n_decode, self.max_len = len(single), max(single, default=1)
            self.n_portions = len(counts) - self.n_decode
        self.identity = self.n_portions == 0  # every row is a single token: decode rows are 0..rows-1
        self._counts = counts
        self._decode_rows = None
        self._tiles: dict = {}
        self._chunking: dict = {}

    @property
    def decode_rows(self):
        if self.identity or self.n_decode == 0:
            return None
        if self._decode_rows is None:
            self._make(tile_rows(0))  # the list of single rows comes with the first tiling asked for
        return self._decode_rows

    def tiles(self, rows_per_tile: int):
        """(first rows, row counts, number of tiles) of the portions cut into tiles of this height."""
        if rows_per_tile not in self._tiles:
            self._make(rows_per_tile)
        return self._tiles[rows_per_tile]

    def _make(self, rows_per_tile: int) -> None:
        step = self.step
        n_tiles = sum(-(-c // rows_per_tile) for c in self._counts if c > 1)
        want_rows = self._decode_rows is None and not self.identity and self.n_decode > 0
        buf = torch.empty(2 * n_tiles + (self.n_decode if want_rows else 0), dtype=torch.int32,
                          device=step.positions.device)
        row0, nrows, rows = buf[:n_tiles], buf[n_tiles:2 * n_tiles], buf[2 * n_tiles:]
        lib = library.load()
        library.check(lib.cuca_attention_plan(_p(step.req_row0), _p(step.req_count), _p(step.req_start), step.n_seqs,
                                              rows_per_tile, _p(rows) if want_rows else None,
                                              self.n_decode if want_rows else 0, _p(row0), _p(nrows), n_tiles,
                                              _stream()), "attention_plan")
        self._tiles[rows_per_tile] = (row0, nrows, n_tiles)
        if want_rows:
            self._decode_rows = rows

    def chunk(self, n_kv_heads: int, head_dim: int):
        key = (n_kv_heads, head_dim)
        if key not in self._chunking:
            self._chunking[key] = decode_chunking(self.n_decode, n_kv_heads, self.max_len, head_dim)
        return self._chunking[key]


def attention_plan(step):
    """The step's plan for the attention kernels (made once per step), or None for a hand-made batch that carries
    no per-request description: such a batch runs through the plain kernel."""
    if getattr(step, "req_start", None) is None or "counts" not in step.host:
        return None
    plan = step.plans.get("paged_attention")
    if plan is None:
        plan = step.plans["paged_attention"] = AttentionPlan(step)
    return plan


_tile_rows: dict = {}


def tile_rows(which: int) -> int:
    """Rows per tile of a prefill form, asked of the kernel library: 0 the `mma.sync` form, 1 the tcgen05 form."""
    if which not in _tile_rows:
        _tile_rows[which] = int(library.load().cuca_attention_tile_rows(which))
    return _tile_rows[which]


_attn_scratch: dict = {}
_attn_scratch_retired: list = []  # superseded buffers: a captured graph may still hold their addresses
USE_TC_ATTENTION = True  # prompt portions through the tcgen05 attention where the shape allows


def attention_scratch(device, floats: int, counters: int):
    """Scratch of the split-key decode attention: partial (acc, max, sum) per chunk, arrival counters
    (zeroed once; the kernel leaves them zeroed). Grows (by doubling at least) when a step needs more. A captured
    graph keeps the addresses it was captured with, so a superseded buffer is never freed: replays of an older
    graph go on writing into memory that is still this module's, and its counters still start at zero."""
    key = (device.type, device.index)
    part, cnt = _attn_scratch.get(key, (None, None))
    if part is None or part.numel() < floats:
        if part is not None:
            _attn_scratch_retired.append(part)
        part = torch.empty(max(floats, 1 << 20, 2 * (part.numel() if part is not None else 0)), dtype=torch.float32,
                           device=device)
    if cnt is None or cnt.numel() < counters:
        if cnt is not None:
            _attn_scratch_retired.append(cnt)
        cnt = torch.zeros(max(counters, 4096, 2 * (cnt.numel() if cnt is not None else 0)), dtype=torch.int32,
                          device=device)
    _attn_scratch[key] = (part, cnt)
    return part, cnt


def attention_mma_supported(n_heads, n_kv_heads, head_dim, q_stride, out_stride) -> bool:
    lib = library.load()
    return bool(lib.cuca_attention_mma_supported(n_heads, n_kv_heads, head_dim, q_stride, out_stride))


_sms: dict = {}


def sm_count() -> int:
    """SMs of the current device, asked of the kernel library once per device."""
    dev = torch.cuda.current_device()
    if dev not in _sms:
        _sms[dev] = int(library.load().cuca_sm_count())
    return _sms[dev]


def decode_chunking(n_rows: int, n_kv_heads: int, max_len: int, head_dim: int = 128, sms: int | None = None):
    """(chunk, n_splits) of the decode attention. chunk 0: every row spreads its own keys evenly over the
    chunks it uses (the kernel repeats this choice per row from the row's own length, never above n_splits).
    n_splits minimises the time on the critical path in units of one 64-key tile: rounds of CTAs the GPU needs
    (a CTA holds three stages of a key and a value tile in shared memory) times (tiles per chunk + about three
    tiles' worth of fixed work per CTA); at most 32 and at most one chunk per tile of the longest row."""
    if sms is None:
        sms = sm_count()
    tiles = max(1, -(-max_len // 64))
    forced = os.environ.get("CUCA_DECODE_SPLITS")  # a measuring aid: this many equal chunks for every row
    if forced:
        n = max(1, min(32, tiles, int(forced)))
        return -(-tiles // n) * 64, n
    slots = _decode_slots(head_dim, sms)
    pairs = max(1, n_rows * n_kv_heads)
    best, best_cost = 1, None
    for n in range(1, min(32, tiles) + 1):
        rounds = -(-pairs * n // slots)
        # the merge: none for one chunk, through distributed shared memory where a row's chunks run as a cluster,
        # through global memory and a last arriver else (measured: about a tile's time more, growing with the chunks)
        merge = 0 if n == 1 else 2 if _merge_as_cluster(pairs, n, slots) else 10 + n // 2
        cost = rounds * (-(-tiles // n) + 3) * 8 + merge
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return 0, best


CLUSTER_MERGE = os.environ.get("CUCA_ATTN_CLUSTER", "1") != "0"
MAX_CLUSTER = 8  # the portable cluster size


def _decode_slots(head_dim: int, sms: int | None = None) -> int:
    """CTAs of the decode attention that are resident at once."""
    smem = 3 * 2 * 64 * (head_dim + 8) * 2 + 2048  # three stages of a key and a value tile
    return (sms or sm_count()) * max(1, min(8, (227 * 1024) // smem))


def _merge_as_cluster(pairs: int, n_splits: int, slots: int) -> bool:
    """Whether a row's chunk CTAs run as a thread-block cluster and merge through distributed shared memory. A
    cluster's CTAs keep their places until its slowest one has finished, a cluster lies within one GPC, and sizes
    that do not divide a GPC's places leave some empty: so only where every cluster is resident at once (clusters of
    two or four: the launch fits the GPU's places; of eight: half of them, since eight pack a GPC's places badly),
    and only for 2, 4 or 8 chunks. Measured: Llama-3.1-8B shape, batch 1, eight chunks: +1.3 % tokens/s as clusters;
    batch 8, 64 clusters of four (256 of 296 places): +0.5 %; batch 4, 32 clusters of eight (256 places): -9 %;
    Llama-2-13B shape, batch 8, 1,280 CTAs in five rounds: -11 %; batch 1, clusters of seven: -7 %."""
    return CLUSTER_MERGE and n_splits in (2, 4, 8) and pairs * n_splits * (2 if n_splits == 8 else 1) <= slots


def _decode_scratch(device, n_rows, n_heads, n_kv_heads, head_dim, n_splits):
    """Scratch of a split-key decode launch, or (None, None) when the row's chunk CTAs merge as a thread-block
    cluster through distributed shared memory: nothing then goes through global memory."""
    if n_splits == 1 or _merge_as_cluster(n_rows * n_kv_heads, n_splits, _decode_slots(head_dim)):
        return None, None
    return attention_scratch(device, n_rows * n_heads * n_splits * (head_dim + 2), n_rows * n_kv_heads)


def attention_decode(q, q_stride, out, kpool, vpool, positions, seq_of_row, tables, rows, n_rows, n_heads,
                     n_kv_heads, head_dim, scale, window, chunk, n_splits, err) -> None:
    lib = library.load()
    part, cnt = _decode_scratch(out.device, n_rows, n_heads, n_kv_heads, head_dim, n_splits)
    library.check(lib.cuca_attention_decode(
        _p(q), int(q_stride), _p(out), out.stride(0), _p(kpool), _p(vpool), kpool.shape[0], kpool.shape[2],
        _p(positions), _p(seq_of_row), _p(tables), tables.shape[1], _p(rows), n_rows, n_heads, n_kv_heads, head_dim,
        float(scale), int(window or 0), chunk, n_splits, _p(part), _p(cnt), _p(err), _stream()), "attention_decode")


def attention_decode_fused(partial, bias, cos, sin, rotary_dim, has_kv, out, kpool, vpool, positions, seq_of_row, tables,
                           rows, n_rows, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits, err) -> None:
    """The decode form fed by the stacked q/k/v projection's unadded K slices (`PartialSums`): adds them, rotates
    q and k, stores k and v in the pages and attends, in one launch. Every row of the step is a single token."""
    lib = library.load()
    part, cnt = _decode_scratch(out.device, n_rows, n_heads, n_kv_heads, head_dim, n_splits)
    library.check(lib.cuca_attention_decode_fused(
        _p(partial.data), partial.slices, partial.slice_stride, _p(bias), _p(cos), _p(sin),
        cos.shape[0] if cos is not None else 0, int(rotary_dim), int(bool(has_kv)), _p(out), out.stride(0), _p(kpool),
        _p(vpool), kpool.shape[0], kpool.shape[2], _p(positions), _p(seq_of_row), _p(tables), tables.shape[1], _p(rows),
        n_rows, n_heads, n_kv_heads, head_dim, float(scale), int(window or 0), chunk, n_splits, _p(part), _p(cnt),
        _p(err), _stream()), "attention_decode_fused")


def attention_decode_fused_supported(plan, cache, out_dtype, n_rows, n_heads, n_kv_heads, head_dim) -> bool:
    """True when every row of the step is a single token of its request and the tensor-core decode form takes
    the shape: then rotate-and-store and attention are one launch."""
    bs = cache.block_size
    return (out_dtype == torch.bfloat16 and plan is not None and plan.identity and plan.n_decode == n_rows
            and n_rows > 0 and bs & (bs - 1) == 0 and head_dim % 16 == 0
            and attention_mma_supported(n_heads, n_kv_heads, head_dim, 2, n_heads * head_dim))


def attention_prefill(q, q_stride, out, kpool, vpool, positions, seq_of_row, tables, tile_row0, tile_nrows, n_tiles,
                      n_heads, n_kv_heads, head_dim, scale, window, err) -> None:
    lib = library.load()
    library.check(lib.cuca_attention_prefill(
        _p(q), int(q_stride), _p(out), out.stride(0), _p(kpool), _p(vpool), kpool.shape[0], kpool.shape[2],
        _p(positions), _p(seq_of_row), _p(tables), tables.shape[1], _p(tile_row0), _p(tile_nrows), n_tiles, n_heads,
        n_kv_heads, head_dim, float(scale), int(window or 0), _p(err), _stream()), "attention_prefill")


def attention_tc_supported(q, out, kpool, vpool, n_heads, n_kv_heads, head_dim) -> bool:
    lib = library.load()
    return bool(lib.cuca_attention_tc_supported(n_heads, n_kv_heads, head_dim, kpool.shape[2], q.stride(0),
                                                out.stride(0), _p(q), _p(kpool), _p(vpool)))


# The largest head size the attention kernels take (`cuca_attention_max_head_dim` says the same; a constant here so
# that describing a model, as for writing a folder of random weights, does not need the kernel library).
ATTENTION_MAX_HEAD_DIM = 256


def attention_pair_tiles_mode(mode: int) -> None:
    """When a CTA of the tcgen05 prefill attention takes two tiles in turn (a heavy and a light one): 1 where that
    makes one round of CTAs out of more, 0 never, 2 whenever a launch has two tiles (tests), -1 as the environment
    variable CUCA_ATTN_PAIR_TILES says."""
    library.load().cuca_attention_pair_tiles_mode(int(mode))


def attention_prefill_tc(q, out, kpool, vpool, positions, seq_of_row, tables, tile_row0, tile_nrows, n_tiles,
                         n_heads, n_kv_heads, head_dim, scale, window, err) -> None:
    """Prefill attention on tcgen05; tiles of up to 128 consecutive rows of one request."""
    lib = library.load()
    library.check(lib.cuca_attention_prefill_tc(
        _p(q), q.stride(0), q.shape[0], _p(out), out.stride(0), _p(kpool), _p(vpool), kpool.shape[0], kpool.shape[2],
        _p(positions), _p(seq_of_row), _p(tables), tables.shape[1], _p(tile_row0), _p(tile_nrows), n_tiles, n_heads,
        n_kv_heads, head_dim, float(scale), int(window or 0), _p(err), _stream()), "attention_prefill_tc")


def attention(qkv, out, cache, step, plan, n_heads, n_kv_heads, head_dim, scale, window, err) -> None:
    """Paged causal attention of every row of the step; q is the head of each `qkv` row. bfloat16 with head
    sizes 16..128 in steps of 16 runs on tensor cores: single-token requests through the split-key decode form,
    portions of prompts through the prefill form; everything else (the 32-bit path, other head sizes) through
    the plain kernel."""
    bs = cache.block_size
    if (out.dtype == torch.bfloat16 and plan is not None and bs & (bs - 1) == 0
            and attention_mma_supported(n_heads, n_kv_heads, head_dim, qkv.stride(0), out.stride(0))):
        if plan.n_portions:
            if USE_TC_ATTENTION and attention_tc_supported(qkv, out, cache.k, cache.v, n_heads, n_kv_heads, head_dim):
                row0, nrows, n = plan.tiles(tile_rows(1))
                attention_prefill_tc(qkv, out, cache.k, cache.v, step.positions, step.seq_of_row, cache.tables,
                                     row0, nrows, n, n_heads, n_kv_heads, head_dim, scale, window, err)
            else:
                row0, nrows, n = plan.tiles(tile_rows(0))
                attention_prefill(qkv, qkv.stride(0), out, cache.k, cache.v, step.positions, step.seq_of_row,
                                  cache.tables, row0, nrows, n, n_heads, n_kv_heads, head_dim, scale, window, err)
        if plan.n_decode:
            chunk, n_splits = plan.chunk(n_kv_heads, head_dim)
            attention_decode(qkv, qkv.stride(0), out, cache.k, cache.v, step.positions, step.seq_of_row,
                             cache.tables, plan.decode_rows, plan.n_decode, n_heads, n_kv_heads, head_dim, scale,
                             window, chunk, n_splits, err)
        return
    attention_generic(qkv, qkv.stride(0), out, cache.k, cache.v, step.positions, step.seq_of_row, cache.tables,
                      n_heads, n_kv_heads, head_dim, scale, window, err)


def scatter_int(dst, idx, val) -> None:
    """dst.view(-1)[idx[i]] = val[i] on the device (page-table updates)."""
    _cuda(dst, idx, val)
    lib = library.load()
    library.check(lib.cuca_scatter_int(_p(dst), _p(idx), _p(val), idx.shape[0], dst.numel(), _stream()), "scatter_int")


def suppress_tokens(logits, ids) -> None:
    """logits[:, ids] = -inf on the device (`ids`: int32 tensor): tokens that must never be sampled."""
    _cuda(logits, ids)
    lib = library.load()
    library.check(lib.cuca_suppress_tokens(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(ids),
                                           ids.shape[0], _stream()), "suppress_tokens")


def sample_scratch_words(vocab: int) -> int:
    n = 1
    while n < vocab:
        n <<= 1
    return n


class SampleSplit:
    """Scratch with which the greedy rows of a large vocabulary are cut over several CTAs each: per row the best of
    every part and a counter of the parts that have arrived (left zeroed by every launch). One per engine; a
    launch with more rows than it holds runs one CTA per row."""

    def __init__(self, rows: int, device):
        self.rows = int(rows)
        self.best = torch.zeros(self.rows * int(library.load().cuca_sample_max_split()), dtype=torch.int64, device=device)
        self.count = torch.zeros(self.rows, dtype=torch.int32, device=device)


def sample(logits, temperature, top_k, top_p, rng_state, slot_of_row, out, scratch=None, split: SampleSplit | None = None) -> None:
    """One token per row of `logits` [R, V] (32-bit). temperature/top_p: float32 [slots]; top_k: int32 [slots];
    rng_state: int64 [slots] SplitMix64 states, advanced for rows that draw; slot_of_row: int32 [R];
    scratch: int64 [R, words] for rows whose cut is wider than 1024 candidates (see `sample_scratch_words`)."""
    _cuda(logits, temperature, top_k, top_p, rng_state, slot_of_row, out)
    lib = library.load()
    library.check(lib.cuca_sample(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(temperature),
                                  _p(top_k), _p(top_p), _p(rng_state), _p(slot_of_row), _p(out), _p(scratch),
                                  0 if scratch is None else scratch.shape[1],
                                  None if split is None else _p(split.best), None if split is None else _p(split.count),
                                  0 if split is None else split.rows, _stream()), "sample")


def decode_advance(tokens, positions, slot_of_row, sampled, history, counter, max_steps, err=None,
                   err_out=None) -> None:
    """tokens <- sampled, positions += 1 for live rows; history[counter] <- sampled; counter += 1;
    err_out[0] <- err[0] (the device error word rides along with the sampled tokens)."""
    lib = library.load()
    library.check(lib.cuca_decode_advance(_p(tokens), _p(positions), _p(slot_of_row), _p(sampled), _p(history),
                                          _p(counter), tokens.shape[0], int(max_steps), _p(err), _p(err_out),
                                          _stream()), "decode_advance")


# ------------------------------------------------------------------ partial sums (decode)
class PartialSums:
    """The result of a contraction over few tokens, left as K slices: `data` is [slices, rows, features] in
    32-bit; the kernel that reads it adds the slices in order (`add_partials_rmsnorm`, `rope_store_partial`)."""

    __slots__ = ("data", "slices")

    def __init__(self, data, slices):
        self.data, self.slices = data, slices

    @property
    def slice_stride(self) -> int:
        return self.data.stride(0)


_partial_max: list = []


def partial_max_tokens() -> int:
    """Most tokens for which a contraction may leave its K slices unadded (asked of the kernel library)."""
    if not _partial_max:
        _partial_max.append(int(library.load().cuca_gemm_tc_partial_max_tokens()))
    return _partial_max[0]


def _partial_plan(M: int, N: int, K: int, max_slices: int):
    """(slices, rows of a slice's slab) the library will use for this shape; slices 0: it does not take it."""
    key = (M, N, K, max_slices)
    plan = _partial_slices.get(key)
    if plan is None:
        lib = library.load()
        plan = _partial_slices[key] = (int(lib.cuca_gemm_tc_partial_slices(M, N, K, max_slices)),
                                       int(lib.cuca_gemm_tc_partial_rows(M, N)))
    return plan


def gemm_partial_supported(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= partial_max_tokens()
            and gemm_tc_supported(a, w) and _partial_plan(a.shape[0], w.shape[0], a.shape[1], 16)[0] > 0)


_partial_slices: dict = {}  # (rows, features, K, most slices) -> (slices the kernel writes, rows of a slice's slab)
_slices_written = ctypes.c_int(0)  # where a launch reports how many it wrote
_SLICES_WRITTEN_AT = ctypes.addressof(_slices_written)


def gemm_partial(a, w, err=None, max_slices=16) -> PartialSums:
    """a @ w.T for few rows (`partial_max_tokens`), as partial sums over K slices (see `PartialSums`)."""
    _cuda(a, w)
    lib = library.load()
    M, K = a.shape
    N = w.shape[0]
    plan = _partial_plan(M, N, K, max_slices)
    slices, slab_rows = plan
    if slices <= 0:
        raise library.KernelError("gemm_partial: unsupported shape")
    # a slice's slab may be padded to the rows its kernel stores at once; the readers see [slices, M, N] of it
    data = torch.empty(slices, slab_rows, N, dtype=torch.float32, device=a.device)
    if slab_rows != M:
        data = data[:, :M]
    library.check(lib.cuca_gemm_tc_partial(_p(a), _p(w), _p(data), M, N, K, a.stride(0), max_slices,
                                           _SLICES_WRITTEN_AT, _p(err), _stream()), "gemm_partial")
    if _slices_written.value != slices:
        raise library.KernelError(f"gemm_partial: {_slices_written.value} slices written, {slices} expected")
    return PartialSums(data, slices)


def add_partials_rmsnorm(x, partial: PartialSums, weight, out, eps, rows=None) -> None:
    """x += sum of the slices (rows named by `rows`, else all); out = RMSNorm(x) * weight."""
    lib = library.load()
    n = out.shape[0]
    library.check(lib.cuca_add_partials_rmsnorm(_p(x), _p(partial.data), partial.slices, partial.slice_stride,
                                                _p(weight), _p(out), dtype_code(out.dtype), _p(rows), n, x.shape[-1],
                                                float(eps), _stream()), "add_partials_rmsnorm")


def add_partials(x, partial: PartialSums) -> None:
    lib = library.load()
    library.check(lib.cuca_add_partials(_p(x), _p(partial.data), partial.slices, partial.slice_stride, x.numel(),
                                        _stream()), "add_partials")


# Most rows for which q/k/v are made from unadded slices: beyond, the rotate-and-store kernel that adds them (one
# block per row, every slice read again) costs more than the slices save (first token of a 300-token prompt on the
# Llama-3.1-8B shape: 7.9 ms that way, 7.4 ms with the projection written out and rotated in place).
ROPE_PARTIAL_MAX_ROWS = 256


def rope_store_partial(partial: PartialSums, bias, q_out, positions, seq_of_row, tables, cos, sin, rotary_dim, kpool,
                       vpool, block_size, n_heads, n_kv_heads, head_dim, err) -> None:
    lib = library.load()
    n_blocks = kpool.shape[0] if kpool is not None else 0
    table_rows = cos.shape[0] if cos is not None else 0
    library.check(lib.cuca_rope_store_partial(
        _p(partial.data), partial.slices, partial.slice_stride, _p(bias), _p(q_out), _p(positions), _p(seq_of_row),
        _p(tables), tables.shape[1] if tables is not None else 0, _p(cos), _p(sin), table_rows, int(rotary_dim),
        _p(kpool), _p(vpool), n_blocks, int(block_size), q_out.shape[0], n_heads, n_kv_heads, head_dim, _p(err),
        _stream()), "rope_store_partial")

"""Each kernel alone against a plain 32-bit PyTorch reference of the same operation, at sizes other than the engine's."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from cuca_b200.kernels import library
    library.load()
    return torch.device("cuda:0")


def _ref_gemm(a, w, epilogue, bias, prior):
    from cuca_b200.kernels import ops
    y = a.float() @ w.float().T
    if epilogue == ops.EPI_SWIGLU:
        n = w.shape[0] // 2
        return torch.nn.functional.silu(y[:, :n]) * y[:, n:]
    if bias is not None:
        y = y + bias.float()
    if epilogue == ops.EPI_RESIDUAL:
        y = prior + y
    return y


GEMM_SHAPES = [(1, 64, 64), (3, 96, 96), (8, 176, 64), (16, 128, 200), (17, 331, 120), (33, 1000, 320),
               (64, 512, 1024), (100, 264, 4096), (130, 640, 256), (300, 384, 136), (8, 4096, 4096),
               (65, 176, 96), (256, 1000, 320), (640, 128, 64), (40, 2304, 512),
               (2048, 4096, 512), (1300, 5000, 1160),  # more tiles than SMs: the last round's K steps are dealt out
               (160, 20000, 512), (192, 1000, 4096), (200, 5000, 320)]  # 129..256 tokens, more tiles than SMs


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("epilogue", [0, 1, 2])
def test_gemm_simt_fp32(dev, M, N, K, epilogue):
    from cuca_b200.kernels import ops
    if M * N * K > 4e8:
        pytest.skip("large case is for the tensor-core kernel")
    g = torch.Generator(device=dev).manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device=dev, generator=g)
    w = torch.randn((2 if epilogue == 2 else 1) * N, K, device=dev, generator=g) / math.sqrt(K)
    bias = torch.randn(N, device=dev, generator=g) if epilogue != 2 and M % 2 else None
    out = torch.randn(M, N, device=dev, generator=g)
    prior = out.clone()
    ops.gemm_simt(a, w, out, epilogue, bias)
    ref = _ref_gemm(a.double(), w.double(), epilogue, None if bias is None else bias.double(), prior.double())
    assert torch.allclose(out.double(), ref.double(), atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("epilogue", [0, 1, 2])
@pytest.mark.parametrize("max_splits", [1, 16])
def test_gemm_tcgen05(dev, M, N, K, epilogue, max_splits):
    """tcgen05 contraction against 32-bit math on the same bf16 inputs: store, residual add, SwiGLU; with and
    without split-K; K tails, N tails, M from 1 to 300."""
    from cuca_b200.kernels import ops
    g = torch.Generator(device=dev).manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn((2 if epilogue == 2 else 1) * N, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev, generator=g).bfloat16() if epilogue != 2 and M % 2 else None
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out_dtype = torch.float32 if epilogue == 1 or (epilogue == 0 and N % 2 == 0) else torch.bfloat16
    out = torch.randn(M, N, device=dev, generator=g).to(out_dtype)
    prior = out.clone()
    assert ops.gemm_tc_supported(a, w)
    ops.gemm_tc(a, w, out, epilogue, bias, err, max_splits=max_splits)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = _ref_gemm(a, w, epilogue, bias, prior.float())
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol), float((out.float() - ref).abs().max())
    # the scratch counters are left zeroed for the next launch
    assert int(ops.gemm_scratch(dev)[1].abs().sum().item()) == 0


@pytest.mark.parametrize("M,N,K", [(129, 256, 64), (256, 256, 512), (300, 384, 136), (512, 1000, 320), (2048, 4096, 512),
                                   (1300, 5000, 1160), (700, 20000, 264)])
@pytest.mark.parametrize("epilogue", [0, 1, 2])
def test_gemm_tcgen05_pairs_of_ctas(dev, M, N, K, epilogue):
    """The two-SM form (a cluster of two CTAs on a tile of 256 tokens x 256 weight rows, `cta_group::2`), forced for
    every shape it takes: ragged rows and columns, K no multiple of the stage, more tiles than pairs."""
    from cuca_b200.kernels import ops
    g = torch.Generator(device=dev).manual_seed(M * 7 + N + K + epilogue)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    rows = N * (2 if epilogue == ops.EPI_SWIGLU else 1)
    w = (torch.randn(rows, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev, generator=g).bfloat16() if epilogue == ops.EPI_STORE else None
    out = torch.randn(M, N, device=dev, generator=g).to(torch.float32 if epilogue == ops.EPI_RESIDUAL else torch.bfloat16)
    prior = out.float().clone()
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.gemm_pair_mode(2)
    try:
        ops.gemm_tc(a, w, out, epilogue, bias, err)
        torch.cuda.synchronize()
    finally:
        ops.gemm_pair_mode(-1)
    assert int(err.item()) == 0
    want = _ref_gemm(a, w, epilogue, bias, prior)
    tol = 2e-3 if epilogue == ops.EPI_RESIDUAL else 2e-2
    assert torch.allclose(out.float(), want, atol=tol, rtol=tol), float((out.float() - want).abs().max())


@pytest.mark.parametrize("M,N,K,out_dtype,epilogue", [
    (256, 4096, 512, torch.float32, 1), (200, 3072, 192, torch.bfloat16, 0), (130, 4000, 1024, torch.float32, 0),
    (300, 2001, 320, torch.bfloat16, 0), (65, 6144, 256, torch.bfloat16, 0)])
def test_gemm_tcgen05_column_pieces(dev, M, N, K, out_dtype, epilogue):
    """More than 64 tokens but fewer whole tiles than SMs: the contraction cuts narrower column pieces, one per
    CTA. Ragged M and N, rows that are and are not 16-byte multiples (copy-engine and plain stores), a bias."""
    from cuca_b200.kernels import ops
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev, generator=g).bfloat16() if M % 2 else None
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.randn(M, N, device=dev, generator=g).to(out_dtype)
    prior = out.clone()
    ops.gemm_tc(a, w, out, epilogue, bias, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = _ref_gemm(a, w, epilogue, bias, prior.float())
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert torch.allclose(out.float(), ref, atol=tol, rtol=tol), float((out.float() - ref).abs().max())


@pytest.mark.parametrize("M,N,K", [(130, 2048, 8256), (256, 4096, 8320), (65, 1024, 9000 // 8 * 8)])
def test_gemm_tcgen05_k_slices_added_in_turn(dev, M, N, K):
    """More than 64 tokens, few tiles, long K, into the 32-bit stream: every CTA takes one K slice of a tile and the
    slices add themselves in K order. Same bits on every run; ragged M, a K tail, a bias that is added once."""
    from cuca_b200.kernels import ops
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev, generator=g).bfloat16() if M % 2 else None
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    prior = torch.randn(M, N, device=dev, generator=g)
    outs = []
    for _ in range(3):
        out = prior.clone()
        ops.gemm_tc(a, w, out, ops.EPI_RESIDUAL, bias, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        outs.append(out)
    ref = _ref_gemm(a, w, ops.EPI_RESIDUAL, bias, prior)
    assert torch.allclose(outs[0], ref, atol=2e-3, rtol=2e-3), float((outs[0] - ref).abs().max())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert int(ops.gemm_scratch(dev)[1].abs().sum().item()) == 0


@pytest.mark.parametrize("M,N,K", [(1, 20000, 4096), (8, 33000, 4096), (33, 20008, 4096), (64, 50000, 1024),
                                   (8, 128256, 4096), (64, 128256, 4096)])
def test_gemm_tcgen05_many_tiles_per_cta_few_tokens(dev, M, N, K):
    """The output head's shape: up to 64 tokens against a vocabulary-sized weight, 32-bit logits out. With the
    weight rows as the 128-row operand there are far more tiles (1,002 at 128,256 rows) than persistent CTAs, so
    every CTA walks several tiles and alternates its two accumulators; a ragged last tile at N = 20,008."""
    from cuca_b200.kernels import ops
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    for trial in range(2):  # the second launch finds the scratch as the first one left it
        out = torch.full((M, N), float("nan"), device=dev)
        ops.gemm_tc(a, w, out, ops.EPI_STORE, None, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        ref = a.float() @ w.float().T
        bad = ~torch.isclose(out, ref, atol=2e-3, rtol=2e-3)
        assert not bool(bad.any()), (f"{int(bad.sum())} wrong logits; first at row, column "
                                     f"{bad.nonzero()[0].tolist()} (tile {int(bad.nonzero()[0][1]) // 128})")
    assert int(ops.gemm_scratch(dev)[1].abs().sum().item()) == 0


def test_gemm_tcgen05_refuses_unaligned(dev):
    from cuca_b200.kernels import ops
    a = torch.zeros(4, 100, device=dev, dtype=torch.bfloat16)  # K = 100 is no multiple of 8
    w = torch.zeros(32, 100, device=dev, dtype=torch.bfloat16)
    assert not ops.gemm_tc_supported(a, w)
    out = torch.zeros(4, 32, device=dev, dtype=torch.bfloat16)
    ops.gemm(a, w, out)  # falls to the CUDA-core kernel instead of computing something wrong


def test_rmsnorm(dev):
    from cuca_b200.kernels import ops
    for T, E, eps in [(1, 64, 1e-5), (7, 96, 1e-6), (33, 1000, 1e-5), (5, 4096, 1e-5)]:
        x = torch.randn(T, E, device=dev) * 3
        w = torch.randn(E, device=dev)
        ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            out = torch.empty(T, E, device=dev, dtype=dt)
            ops.rmsnorm(x, w, out, eps)
            assert torch.allclose(out.float(), ref, atol=tol, rtol=tol)
        rows = torch.tensor([T - 1, 0], device=dev, dtype=torch.int32)
        out = torch.empty(2, E, device=dev)
        ops.rmsnorm(x, w, out, eps, rows)
        assert torch.allclose(out, ref[[T - 1, 0]], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("E,dtype", [(24, torch.bfloat16), (4096, torch.bfloat16), (4100, torch.bfloat16), (30, torch.bfloat16),
                                     (24, torch.float32), (22, torch.float32)])
def test_embed_and_bad_token(dev, E, dtype):
    """Rows of 16-byte multiples take the vector path, others one value at a time."""
    from cuca_b200.kernels import ops
    table = torch.randn(50, E, device=dev).to(dtype)
    toks = torch.tensor([3, 49, 0, 7], device=dev, dtype=torch.int32)
    out = torch.empty(4, E, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.embed(table, toks, out, err)
    assert torch.equal(out, table[toks.long()].float()) and int(err.item()) == 0
    ops.embed(table, torch.tensor([50], device=dev, dtype=torch.int32), out[:1], err)
    assert int(err.item()) == 1  # recorded, not faulted


def test_swiglu_and_argmax(dev):
    from cuca_b200.kernels import ops
    gu = torch.randn(9, 2 * 40, device=dev)
    out = torch.empty(9, 40, device=dev)
    ops.swiglu(gu, out)
    assert torch.allclose(out, torch.nn.functional.silu(gu[:, :40]) * gu[:, 40:], atol=1e-6)
    logits = torch.randn(5, 1003, device=dev)
    logits[2, 10] = logits[2, 900] = 50.0  # first maximum wins
    logits[3, :] = float("-inf")
    ids = torch.empty(5, dtype=torch.int32, device=dev)
    ops.argmax(logits, ids)
    want = logits.argmax(-1).tolist()
    want[2], want[3] = 10, 0
    assert ids.tolist() == want


def _paged_setup(dev, dtype, lens, nh, nkv, d, bs, n_blocks, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    S = len(lens)
    width = max(-(-l // bs) for l in lens) + 1
    perm = torch.randperm(n_blocks, device=dev, generator=g).tolist()  # scrambled pages
    tables = torch.full((S, width), -1, dtype=torch.int32, device=dev)
    k = [torch.randn(l, nkv, d, device=dev, generator=g) for l in lens]
    v = [torch.randn(l, nkv, d, device=dev, generator=g) for l in lens]
    kpool = torch.zeros(n_blocks, nkv, bs, d, device=dev, dtype=dtype)
    vpool = torch.zeros_like(kpool)
    nxt = 0
    for s, l in enumerate(lens):
        for b in range(-(-l // bs)):
            page = perm[nxt]
            nxt += 1
            tables[s, b] = page
            n = min(bs, l - b * bs)
            kpool[page, :, :n] = k[s][b * bs:b * bs + n].transpose(0, 1).to(dtype)
            vpool[page, :, :n] = v[s][b * bs:b * bs + n].transpose(0, 1).to(dtype)
    return k, v, kpool, vpool, tables


def _ref_attention(q, k, v, pos, scale, window):
    # q: [nh, d]; k, v: [len, nkv, d]; keys lo..pos
    nh, nkv = q.shape[0], k.shape[1]
    lo = max(0, pos - (window - 1)) if window else 0
    out = torch.empty_like(q)
    for h in range(nh):
        kv = h // (nh // nkv)
        s = (k[lo:pos + 1, kv] @ q[h]) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, kv]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,bs,window", [(4, 2, 16, 16, None), (3, 1, 32, 16, None), (6, 3, 48, 8, 20),
                                                (8, 8, 64, 32, None), (8, 2, 128, 16, 33), (2, 1, 256, 16, None)])
def test_attention_generic_paged(dev, dtype, nh, nkv, d, bs, window):
    """Paged attention over scrambled page tables against contiguous 32-bit attention; lengths around page and
    tile edges; rows of several requests in one launch; one far key made to stand out."""
    from cuca_b200.kernels import ops
    lens = [1, 2, 15, 16, 17, 33, 50, 129]
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs, n_blocks=64)
    g = torch.Generator(device=dev).manual_seed(1)
    rows, ref = [], []
    for s, l in enumerate(lens):
        for pos in sorted({0, l // 2, l - 1}):
            q = torch.randn(nh, d, device=dev, generator=g)
            if pos > 3:
                q[0] = k[s][1, 0] * 4.0  # a far key among many: its score stands out
            rows.append((s, pos, q))
            kk, vv = k[s].to(dtype).float(), v[s].to(dtype).float()
            ref.append(_ref_attention(q.to(dtype).float(), kk, vv, pos, 1.0 / math.sqrt(d), window))
    T = len(rows)
    qbuf = torch.stack([r[2] for r in rows]).reshape(T, nh * d).to(dtype).contiguous()
    positions = torch.tensor([r[1] for r in rows], dtype=torch.int32, device=dev)
    seq = torch.tensor([r[0] for r in rows], dtype=torch.int32, device=dev)
    out = torch.empty(T, nh * d, device=dev, dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.attention_generic(qbuf, nh * d, out, kpool, vpool, positions, seq, tables, nh, nkv, d, 1.0 / math.sqrt(d),
                          window, err)
    assert int(err.item()) == 0
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    got = out.float().view(T, nh, d)
    for i in range(T):
        assert torch.allclose(got[i], ref[i], atol=tol, rtol=tol), (rows[i][0], rows[i][1])
    # a row alone gives the same bits as the row in the batch
    one = torch.empty(1, nh * d, device=dev, dtype=dtype)
    i = T - 2
    ops.attention_generic(qbuf[i:i + 1], nh * d, one, kpool, vpool, positions[i:i + 1], seq[i:i + 1], tables, nh, nkv,
                          d, 1.0 / math.sqrt(d), window, err)
    assert torch.equal(one[0], out[i])
    # a missing page is recorded, not read
    bad = tables.clone()
    bad[seq[i], 0] = -1
    ops.attention_generic(qbuf[i:i + 1], nh * d, one, kpool, vpool, positions[i:i + 1], seq[i:i + 1], bad, nh, nkv, d,
                          1.0 / math.sqrt(d), None, err)
    assert int(err.item()) == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rot", [(6, 2, 48, 32), (6, 2, 48, 48), (5, 5, 128, 128), (4, 1, 80, 80)])
def test_rope_store(dev, dtype, nh, nkv, d, rot):
    """Rotation of q and k (half-split pairs, partial and whole rotary size; whole heads of 16-multiples take the
    vector kernel in bf16) and the write of k, v to their pages."""
    from cuca_b200.kernels import ops
    from cuca_b200.parts.rope import rope_tables
    bs = 8
    T, n_blocks = 11, 9
    cos, sin = rope_tables(64, rot, 10000.0)
    cos, sin = cos.to(dev), sin.to(dev)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device=dev).to(dtype)
    orig = qkv.float().clone()
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 40, 41], dtype=torch.int32, device=dev)
    seq = torch.tensor([0] * 9 + [1, 1], dtype=torch.int32, device=dev)
    tables = torch.full((2, 8), -1, dtype=torch.int32, device=dev)
    tables[0, 0], tables[0, 1], tables[1, 5] = 4, 2, 7
    kpool = torch.zeros(n_blocks, nkv, bs, d, device=dev, dtype=dtype)
    vpool = torch.zeros_like(kpool)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.rope_store(qkv, positions, seq, tables, cos, sin, rot, kpool, vpool, bs, nh, nkv, d, err)
    assert int(err.item()) == 0

    def rotate(x, p):  # x: [heads, d]
        c, s = cos[p], sin[p]
        a, b = x[:, :rot // 2], x[:, rot // 2:rot]
        return torch.cat([a * c - b * s, a * s + b * c, x[:, rot:]], dim=1)

    tol = 1e-6 if dtype == torch.float32 else 2e-2
    for r in range(T):
        p, s = int(positions[r]), int(seq[r])
        page, off = int(tables[s, p // bs]), p % bs
        heads = orig[r].view(nh + 2 * nkv, d)
        assert torch.allclose(qkv[r].float().view(-1, d)[:nh], rotate(heads[:nh], p), atol=tol)
        assert torch.allclose(kpool[page, :, off].float(), rotate(heads[nh:nh + nkv], p), atol=tol)
        assert torch.equal(vpool[page, :, off].float(), heads[nh + nkv:])
    assert int((kpool.float().abs().sum(dim=(1, 2, 3)) > 0).sum()) == 3  # only the three pages named were written


MMA_SHAPES = [(4, 2, 16, 16, None), (3, 1, 32, 16, None), (6, 3, 48, 8, 20), (8, 8, 64, 32, None),
              (8, 2, 128, 16, 33), (32, 8, 128, 16, None), (16, 1, 80, 64, 100), (2, 2, 112, 4, None)]


@pytest.mark.parametrize("nh,nkv,d,bs,window", MMA_SHAPES)
@pytest.mark.parametrize("chunk", [64, 256, 0])
def test_attention_decode_mma(dev, nh, nkv, d, bs, window, chunk):
    """Split-key decode attention on tensor cores against contiguous 32-bit attention: scrambled pages,
    lengths around page, tile and chunk edges, a row list with gaps, one far key that stands out."""
    from cuca_b200.kernels import ops
    dtype = torch.bfloat16
    lens = [1, 2, 15, 16, 17, 63, 64, 65, 129, 300, 513]
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs,
                                              n_blocks=sum(-(-l // bs) for l in lens) + 5, seed=3)
    g = torch.Generator(device=dev).manual_seed(2)
    T = len(lens) + 2
    qbuf = torch.randn(T, nh * d, device=dev, generator=g)
    positions = torch.zeros(T, dtype=torch.int32, device=dev)
    seq = torch.full((T,), -1, dtype=torch.int32, device=dev)
    rows, ref = [], {}
    for s, l in enumerate(lens):
        r = s + 1  # row 0 and the last row are not decode rows
        pos = l - 1
        if pos > 3:
            qbuf[r, :d] = k[s][1, 0] * 4.0
        positions[r], seq[r] = pos, s
        rows.append(r)
        ref[r] = _ref_attention(qbuf[r].to(dtype).float().view(nh, d), k[s].to(dtype).float(), v[s].to(dtype).float(),
                                pos, 1.0 / math.sqrt(d), window)
    qb = qbuf.to(dtype).contiguous()
    out = torch.zeros(T, nh * d, device=dev, dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    rows_t = torch.tensor(rows, dtype=torch.int32, device=dev)
    n_splits = -(-max(lens) // chunk) if chunk else 5  # chunk 0: each row spreads its keys over 5 chunks
    for _ in range(2):  # twice: the arrival counters must be left zeroed
        out.zero_()
        ops.attention_decode(qb, nh * d, out, kpool, vpool, positions, seq, tables, rows_t, len(rows), nh, nkv, d,
                             1.0 / math.sqrt(d), window, chunk, n_splits, err)
        assert int(err.item()) == 0
        for r in rows:
            got = out[r].float().view(nh, d)
            assert torch.allclose(got, ref[r], atol=2e-2, rtol=2e-2), (r, float((got - ref[r]).abs().max()))
    assert float(out[0].abs().sum()) == 0 and float(out[-1].abs().sum()) == 0  # rows not listed stay untouched


@pytest.mark.parametrize("nh,nkv,d,bs,window", MMA_SHAPES)
@pytest.mark.parametrize("chunk,partial_rotary,has_kv", [(64, False, True), (0, True, True), (0, False, False)])
def test_attention_decode_fused_with_rotation_and_store(dev, nh, nkv, d, bs, window, chunk, partial_rotary, has_kv):
    """The decode form fed by the projection's K slices: it adds them, rotates q and k, writes k and v to the page
    and attends, against the same steps done one by one in 32-bit. The page slot of the new position holds a
    large stale value beforehand, so a read of the page instead of the new key would show."""
    from cuca_b200.kernels import ops
    from cuca_b200.parts.rope import rope_tables
    dtype = torch.bfloat16
    lens = [1, 2, 16, 17, 64, 65, 129, 300, 513]
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs,
                                              n_blocks=sum(-(-l // bs) for l in lens) + 5, seed=5)
    rot = d // 2 if partial_rotary else d
    cos, sin = rope_tables(600, rot, 10000.0)
    cos, sin = cos.to(dev), sin.to(dev)
    g = torch.Generator(device=dev).manual_seed(4)
    T = len(lens) + 1  # the last row is padding
    width = (nh + (2 * nkv if has_kv else 0)) * d
    slices = torch.randn(3, T, width, device=dev, generator=g) * 0.6
    bias = (torch.randn(width, device=dev, generator=g) * 0.1).to(dtype)
    total = slices.sum(0) + bias.float()
    positions = torch.zeros(T, dtype=torch.int32, device=dev)
    seq = torch.full((T,), -1, dtype=torch.int32, device=dev)

    def rotate(x, p):
        c, s_ = cos[p], sin[p]
        a, b = x[:, :rot // 2], x[:, rot // 2:rot]
        return torch.cat([a * c - b * s_, a * s_ + b * c, x[:, rot:]], dim=1)

    ref, new_kv = {}, {}
    for s, l in enumerate(lens):
        pos = l - 1
        positions[s], seq[s] = pos, s
        heads = total[s].view(-1, d)
        q = rotate(heads[:nh], pos).to(dtype).float()
        ks, vs = k[s].to(dtype).float().clone(), v[s].to(dtype).float().clone()
        page, off = int(tables[s, pos // bs]), pos % bs
        if has_kv:
            ks[pos] = rotate(heads[nh:nh + nkv], pos).to(dtype).float()
            vs[pos] = heads[nh + nkv:].to(dtype).float()
            new_kv[s] = (page, off, ks[pos], vs[pos])
            kpool[page, :, off] = 100.0  # stale
            vpool[page, :, off] = 100.0
        ref[s] = _ref_attention(q, ks, vs, pos, 1.0 / math.sqrt(d), window)
    out = torch.zeros(T, nh * d, device=dev, dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    n_splits = -(-max(lens) // chunk) if chunk else 5
    ops.attention_decode_fused(ops.PartialSums(slices, 3), bias, cos, sin, rot, has_kv, out, kpool, vpool, positions,
                               seq, tables, None, T, nh, nkv, d, 1.0 / math.sqrt(d), window, chunk, n_splits, err)
    assert int(err.item()) == 0
    for s in range(len(lens)):
        got = out[s].float().view(nh, d)
        assert torch.allclose(got, ref[s], atol=3e-2, rtol=3e-2), (s, float((got - ref[s]).abs().max()))
        if has_kv:
            page, off, kn, vn = new_kv[s]
            assert torch.allclose(kpool[page, :, off].float(), kn, atol=2e-2, rtol=2e-2)
            assert torch.allclose(vpool[page, :, off].float(), vn, atol=2e-2, rtol=2e-2)
    assert float(out[-1].abs().sum()) == 0


@pytest.mark.parametrize("nh,nkv,d,bs,window", MMA_SHAPES)
def test_attention_prefill_mma(dev, nh, nkv, d, bs, window):
    """Prefill attention on tensor cores: portions that start at position 0 and in the middle of a request
    (keys partly from earlier steps), tiles of 64 rows and ragged tails, against 32-bit attention."""
    from cuca_b200.kernels import ops
    dtype = torch.bfloat16
    lens = [5, 64, 70, 200, 131]
    starts = [0, 0, 33, 90, 129]  # the portion covers positions start..len-1
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs,
                                              n_blocks=sum(-(-l // bs) for l in lens) + 3, seed=5)
    g = torch.Generator(device=dev).manual_seed(4)
    pos_list, seq_list, tile_row0, tile_nrows = [], [], [], []
    for s, (l, st) in enumerate(zip(lens, starts)):
        r0 = len(pos_list)
        n = l - st
        pos_list += list(range(st, l))
        seq_list += [s] * n
        for off in range(0, n, 64):
            tile_row0.append(r0 + off)
            tile_nrows.append(min(64, n - off))
    T = len(pos_list)
    qbuf = torch.randn(T, nh * d, device=dev, generator=g).to(dtype)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=dev)
    seq = torch.tensor(seq_list, dtype=torch.int32, device=dev)
    out = torch.zeros(T, nh * d, device=dev, dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.attention_prefill(qbuf, nh * d, out, kpool, vpool, positions, seq, tables,
                          torch.tensor(tile_row0, dtype=torch.int32, device=dev),
                          torch.tensor(tile_nrows, dtype=torch.int32, device=dev), len(tile_row0), nh, nkv, d,
                          1.0 / math.sqrt(d), window, err)
    assert int(err.item()) == 0
    for r in range(T):
        s, pos = seq_list[r], pos_list[r]
        want = _ref_attention(qbuf[r].float().view(nh, d), k[s].to(dtype).float(), v[s].to(dtype).float(), pos,
                              1.0 / math.sqrt(d), window)
        got = out[r].float().view(nh, d)
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (r, s, pos, float((got - want).abs().max()))


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 4096, 4096), (8, 6144, 4096), (3, 96, 96), (17, 331, 120),
                                   (64, 512, 1024), (40, 2304, 512), (5, 128256 // 8, 256),
                                   (100, 2304, 512), (130, 4096, 1024), (256, 6144, 4096), (200, 331, 120),
                                   (129, 264, 64), (300, 1000, 320), (512, 4096, 14336), (511, 6144, 4096),
                                   (257, 5000, 1160)])
def test_gemm_partial_sums_and_their_readers(dev, M, N, K):
    """The decode contraction that leaves its K slices unadded, and the kernels that add them while reading:
    RMSNorm over the residual stream and rotate-and-store of the q/k/v projection."""
    from cuca_b200.kernels import ops
    from cuca_b200.parts.rope import rope_tables
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) / math.sqrt(K)).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    assert ops.gemm_partial_supported(a, w)
    ps = ops.gemm_partial(a, w, err)
    assert ps.data.shape == (ps.slices, M, N) and int(err.item()) == 0
    ref = a.float() @ w.float().T
    assert torch.allclose(ps.data.sum(0), ref, atol=2e-3, rtol=2e-3)
    if K >= 1024 and N <= 6144 and M <= 256:
        assert ps.slices > 1  # few tiles, long K: the SMs share the K range
    # reader 1: x += slices; h = RMSNorm(x)
    x = torch.randn(M, N, device=dev, generator=g)
    wn = torch.randn(N, device=dev, generator=g)
    want_x = x + ref
    want_h = want_x * torch.rsqrt((want_x * want_x).mean(-1, keepdim=True) + 1e-5) * wn
    h = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    ops.add_partials_rmsnorm(x, ps, wn, h, 1e-5)
    assert torch.allclose(x, want_x, atol=2e-3, rtol=2e-3)
    assert torch.allclose(h.float(), want_h, atol=3e-2, rtol=3e-2)
    # reader 2: plain add
    y = torch.zeros(M, N, device=dev)
    ops.add_partials(y, ps)
    assert torch.allclose(y, ref, atol=2e-3, rtol=2e-3)


def test_rope_store_from_partial_sums(dev):
    from cuca_b200.kernels import ops
    from cuca_b200.parts.rope import rope_tables
    nh, nkv, d, rot, bs, T = 6, 2, 32, 32, 8, 5
    width = (nh + 2 * nkv) * d
    cos, sin = rope_tables(64, rot, 10000.0)
    cos, sin = cos.to(dev), sin.to(dev)
    slices = torch.randn(3, T, width, device=dev)
    bias = torch.randn(width, device=dev).bfloat16()
    total = slices.sum(0) + bias.float()
    positions = torch.tensor([0, 1, 2, 17, 18], dtype=torch.int32, device=dev)
    seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=dev)
    tables = torch.full((2, 8), -1, dtype=torch.int32, device=dev)
    tables[0, 0], tables[1, 2] = 3, 1
    kpool = torch.zeros(5, nkv, bs, d, device=dev, dtype=torch.bfloat16)
    vpool = torch.zeros_like(kpool)
    q = torch.zeros(T, nh * d, device=dev, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.rope_store_partial(ops.PartialSums(slices, 3), bias, q, positions, seq, tables, cos, sin, rot, kpool, vpool, bs,
                           nh, nkv, d, err)
    assert int(err.item()) == 0

    def rotate(x, p):
        c, s = cos[p], sin[p]
        a, b = x[:, :rot // 2], x[:, rot // 2:rot]
        return torch.cat([a * c - b * s, a * s + b * c, x[:, rot:]], dim=1)

    for r in range(T):
        p, s = int(positions[r]), int(seq[r])
        page, off = int(tables[s, p // bs]), p % bs
        heads = total[r].view(nh + 2 * nkv, d)
        assert torch.allclose(q[r].float().view(nh, d), rotate(heads[:nh], p), atol=3e-2, rtol=3e-2)
        assert torch.allclose(kpool[page, :, off].float(), rotate(heads[nh:nh + nkv], p), atol=3e-2, rtol=3e-2)
        assert torch.allclose(vpool[page, :, off].float(), heads[nh + nkv:], atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("nh,nkv,bs,window", [(4, 2, 16, None), (8, 8, 32, None), (8, 2, 16, 150), (2, 1, 8, None),
                                              (3, 1, 64, 40)])
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("two_tiles_per_cta", [False, True])
def test_attention_prefill_tcgen05(dev, nh, nkv, bs, window, d, two_tiles_per_cta):
    """Prefill attention on tcgen05 (head size 128 or 64): portions that start at position 0 and in the middle of a
    request, tiles of 128 rows and ragged tails, several key tiles, against 32-bit attention; with one tile per CTA
    and with two in turn (an odd number of tiles, so that the middle one stays alone)."""
    from cuca_b200.kernels import ops
    dtype = torch.bfloat16
    lens = [5, 128, 200, 390, 131, 60]
    starts = [0, 0, 33, 129, 129, 0]   # nine tiles
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs,
                                              n_blocks=sum(-(-l // bs) for l in lens) + 3, seed=6)
    g = torch.Generator(device=dev).manual_seed(8)
    pos_list, seq_list, tile_row0, tile_nrows = [], [], [], []
    for s, (l, st) in enumerate(zip(lens, starts)):
        r0 = len(pos_list)
        n = l - st
        pos_list += list(range(st, l))
        seq_list += [s] * n
        for off in range(0, n, 128):
            tile_row0.append(r0 + off)
            tile_nrows.append(min(128, n - off))
    T = len(pos_list)
    width = (nh + 2 * nkv) * d  # q is the head of a wider row, as in the engine
    qkv = torch.randn(T, width, device=dev, generator=g).to(dtype)
    positions = torch.tensor(pos_list, dtype=torch.int32, device=dev)
    seq = torch.tensor(seq_list, dtype=torch.int32, device=dev)
    out = torch.zeros(T, nh * d, device=dev, dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    assert ops.attention_tc_supported(qkv, out, kpool, vpool, nh, nkv, d)
    ops.attention_pair_tiles_mode(2 if two_tiles_per_cta else 0)
    try:
        ops.attention_prefill_tc(qkv, out, kpool, vpool, positions, seq, tables,
                                 torch.tensor(tile_row0, dtype=torch.int32, device=dev),
                                 torch.tensor(tile_nrows, dtype=torch.int32, device=dev), len(tile_row0), nh, nkv, d,
                                 1.0 / math.sqrt(d), window, err)
        torch.cuda.synchronize()
    finally:
        ops.attention_pair_tiles_mode(-1)
    assert int(err.item()) == 0
    for r in range(T):
        s, pos = seq_list[r], pos_list[r]
        want = _ref_attention(qkv[r, :nh * d].float().view(nh, d), k[s].to(dtype).float(), v[s].to(dtype).float(), pos,
                              1.0 / math.sqrt(d), window)
        got = out[r].float().view(nh, d)
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (r, s, pos, float((got - want).abs().max()))


def test_rmsnorm_many_rows_equals_few_rows_to_the_bit(dev):
    """Launches with many rows use narrower blocks; a row's bits must not depend on that."""
    from cuca_b200.kernels import ops
    for E in (4096, 5120, 8192):
        x = torch.randn(200, E, device=dev) * 2
        w = torch.randn(E, device=dev)
        many = torch.empty(200, E, device=dev)
        ops.rmsnorm(x, w, many, 1e-5)
        few = torch.empty(3, E, device=dev)
        ops.rmsnorm(x[100:103].contiguous(), w, few, 1e-5)
        assert torch.equal(many[100:103], few)
        ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
        assert torch.allclose(many, ref, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("n_req,longest,tile", [(1, 1, 64), (3, 150, 64), (40, 300, 128), (1500, 3, 64),
                                                (700, 700, 64), (9, 2048, 128)])
def test_attention_plan_on_the_device(dev, n_req, longest, tile):
    """The attention part's plan is made on the device from the step's per-request description: the rows of the
    requests that bring one token, and the longer portions cut into tiles, heaviest (latest positions) first.
    More requests than the kernel's block has threads, and more tiles than it ranks (then in request order)."""
    import numpy as np
    from cuca_b200.kernels import library, ops
    rs = np.random.default_rng(n_req + longest)
    counts = rs.integers(1, longest + 1, size=n_req)
    counts[rs.random(n_req) < 0.4] = 1
    starts = rs.integers(0, 5000, size=n_req)
    row0 = np.concatenate([[0], np.cumsum(counts)[:-1]])
    n_decode = int((counts == 1).sum())
    n_tiles = int(sum(-(-c // tile) for c in counts if c > 1))
    t = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=dev)
    rows = torch.full((max(1, n_decode),), -1, dtype=torch.int32, device=dev)
    t0 = torch.full((max(1, n_tiles),), -1, dtype=torch.int32, device=dev)
    tn = torch.full((max(1, n_tiles),), -1, dtype=torch.int32, device=dev)
    lib = library.load()
    d_row0, d_counts, d_starts = t(row0), t(counts), t(starts)
    library.check(lib.cuca_attention_plan(d_row0.data_ptr(), d_counts.data_ptr(), d_starts.data_ptr(), n_req, tile,
                                          rows.data_ptr(), n_decode, t0.data_ptr(), tn.data_ptr(), n_tiles,
                                          torch.cuda.current_stream().cuda_stream), "attention_plan")
    assert rows[:n_decode].tolist() == [int(r) for r, c in zip(row0, counts) if c == 1]
    want = [(int(r + off), int(min(tile, c - off)), int(s + off))
            for r, c, s in zip(row0, counts, starts) if c > 1 for off in range(0, c, tile)]
    got = list(zip(t0[:n_tiles].tolist(), tn[:n_tiles].tolist()))
    assert sorted(got) == sorted((a, b) for a, b, _ in want)          # every portion is covered exactly once
    if n_tiles <= 2048:
        ranked = sorted(range(len(want)), key=lambda i: (-want[i][2], i))
        assert got == [(want[i][0], want[i][1]) for i in ranked]       # heaviest first, ties in request order
    else:
        assert got == [(a, b) for a, b, _ in want]
    assert ops.tile_rows(0) == 64 and ops.tile_rows(1) == 128


def test_a_bounded_wait_that_runs_out_returns_an_error_and_leaves_the_library_usable(dev):
    """Every wait inside a kernel has a limit. Here two roles of one CTA wait for 1 ms and for 1 s on barriers that
    nobody arrives at: the first runs out, records error 3 in the error word and raises the CTA's abort flag; the
    second gives up on seeing the flag long before its own limit; the kernel returns, the host reads the error as
    `DeviceFault`, and the next kernel runs as if nothing had happened."""
    import time
    from cuca_b200.kernels import library, ops
    from cuca_b200.runtime import DeviceFault, Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    report = torch.full((3,), -1, dtype=torch.int32, device=dev)
    lib = library.load()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    library.check(lib.cuca_wait_probe(1_000_000, rt.err.data_ptr(), report.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream), "wait_probe")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5, "the second role must give up on the flag, not wait out its own second"
    assert report.tolist() == [0, 0, 1]
    with pytest.raises(DeviceFault, match="bounded wait"):
        rt.check_device_errors()
    rt.check_device_errors()  # the word was cleared
    a = torch.randn(8, 256, device=dev).bfloat16()
    w = torch.randn(64, 256, device=dev).bfloat16()
    out = rt.linear(a, w)
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), a.float() @ w.float().T, atol=0.2, rtol=2e-2)
    rt.check_device_errors()


@pytest.mark.parametrize("d,nh,nkv", [(128, 4, 2), (64, 6, 2)])
def test_attention_over_tens_of_thousands_of_keys(dev, d, nh, nkv):
    """Forty thousand keys of one request: the key/value rings of both tensor-core kernels wrap more than a hundred
    times and the page table is read in seventy-eight batches. Decode: the last position, with its keys in one
    chunk per row's own choice, in a cluster of eight chunks and in thirty-two chunks through scratch. Prefill: the
    last 300 rows as a portion that starts deep inside the request. One query is pointed at the key of position 7,
    another at a key in the middle, so that a lost page shows."""
    from cuca_b200.kernels import ops
    dtype, bs = torch.bfloat16, 16
    lens = [40_000, 33_333]
    k, v, kpool, vpool, tables = _paged_setup(dev, dtype, lens, nh, nkv, d, bs,
                                              n_blocks=sum(-(-l // bs) for l in lens) + 7, seed=12)
    g = torch.Generator(device=dev).manual_seed(13)
    scale = 1.0 / math.sqrt(d)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    kf = [x.to(dtype).float() for x in k]
    vf = [x.to(dtype).float() for x in v]
    # ---- decode: one row per request at its last position
    q = torch.randn(2, nh * d, device=dev, generator=g)
    q[0, :d] = k[0][7, 0] * 3.0            # head 0 of request 0 looks at position 7
    q[1, :d] = k[1][17_001, 0] * 3.0       # head 0 of request 1 at a key in the middle
    qb = q.to(dtype).contiguous()
    positions = torch.tensor([lens[0] - 1, lens[1] - 1], dtype=torch.int32, device=dev)
    seq = torch.tensor([0, 1], dtype=torch.int32, device=dev)
    want = [_ref_attention(qb[r].float().view(nh, d), kf[r], vf[r], lens[r] - 1, scale, None) for r in range(2)]
    for chunk, n_splits in ((0, 5), (0, 8), (-(-lens[0] // 32 // 64) * 64, 32)):
        out = torch.zeros(2, nh * d, device=dev, dtype=dtype)
        ops.attention_decode(qb, nh * d, out, kpool, vpool, positions, seq, tables, None, 2, nh, nkv, d, scale, None,
                             chunk, n_splits, err)
        assert int(err.item()) == 0
        for r in range(2):
            got = out[r].float().view(nh, d)
            assert torch.allclose(got, want[r], atol=2e-2, rtol=2e-2), (n_splits, r, float((got - want[r]).abs().max()))
    # ---- prefill on tcgen05: the last 300 rows of request 0
    n = 300
    start = lens[0] - n
    width = (nh + 2 * nkv) * d
    qkv = torch.randn(n, width, device=dev, generator=g)
    qkv[-1, :d] = k[0][7, 0] * 3.0
    qkv[5, d:2 * d] = k[0][20_000, 0] * 3.0
    qkv = qkv.to(dtype)
    pos = torch.arange(start, lens[0], dtype=torch.int32, device=dev)
    seq_p = torch.zeros(n, dtype=torch.int32, device=dev)
    out = torch.zeros(n, nh * d, device=dev, dtype=dtype)
    assert ops.attention_tc_supported(qkv, out, kpool, vpool, nh, nkv, d)
    row0 = torch.tensor([0, 128, 256], dtype=torch.int32, device=dev)
    nrows = torch.tensor([128, 128, 44], dtype=torch.int32, device=dev)
    ops.attention_prefill_tc(qkv, out, kpool, vpool, pos, seq_p, tables, row0, nrows, 3, nh, nkv, d, scale, None, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    for r in (0, 5, 127, 128, 200, 299):
        ref = _ref_attention(qkv[r, :nh * d].float().view(nh, d), kf[0], vf[0], start + r, scale, None)
        got = out[r].float().view(nh, d)
        assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), (r, float((got - ref).abs().max()))

"""The plain implementation checked against the definitions it restates (no GPU, no product code)."""
import math

import numpy as np
import torch

import plain_llama as pl
import tiny


def test_rms_norm_definition():
    x = torch.tensor([[3.0, 4.0]])
    out = pl.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[3 * r * 2, 4 * r * 0.5]]))


def test_rope_table_is_the_definition_and_position_zero_is_identity():
    cos, sin = pl.rope_tables(5, 8, 10000.0, None)
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)
    assert abs(float(cos[3, 1]) - math.cos(3 * 10000.0 ** (-2 / 8))) < 1e-7
    x = torch.randn(5, 2, 8)
    assert torch.equal(pl.rotate_half_split(x, cos, sin)[0], x[0])
    # a rotation keeps every pair's length
    y = pl.rotate_half_split(x, cos, sin)
    assert torch.allclose(x[..., :4] ** 2 + x[..., 4:] ** 2, y[..., :4] ** 2 + y[..., 4:] ** 2, atol=1e-5)


def test_half_split_pairs_equal_adjacent_pairs_on_permuted_rows():
    """The reference permutes q/k rows (row j*half + i -> 2i + j) and rotates adjacent pairs
    (src/provider/local/convert/tensors.rs:250-271, model/cpu.rs:4247-4275): same scores."""
    d, t = 16, 6
    half = d // 2
    cos, sin = pl.rope_tables(t, d, 500000.0, None)
    q, k = torch.randn(t, 1, d), torch.randn(t, 1, d)
    perm = torch.empty(d, dtype=torch.long)
    for j in range(2):
        for i in range(half):
            perm[2 * i + j] = j * half + i

    def rotate_adjacent(x):
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * cos[:, None, :] - b * sin[:, None, :]
        out[..., 1::2] = a * sin[:, None, :] + b * cos[:, None, :]
        return out

    s1 = pl.rotate_half_split(q, cos, sin)[:, 0] @ pl.rotate_half_split(k, cos, sin)[:, 0].T
    s2 = rotate_adjacent(q[..., perm])[:, 0] @ rotate_adjacent(k[..., perm])[:, 0].T
    assert torch.allclose(s1, s2, atol=1e-5)


def test_llama3_factors_have_three_regimes():
    f = pl.llama3_factors(tiny.TINY_B, 32)
    assert f[0] == 1.0 and f[-1] == 8.0 and any(1.0 < v < 8.0 for v in f)
    assert pl.llama3_factors(tiny.TINY_A, 16) is None
    assert pl.linear_freq_scale(tiny.TINY_C) == 0.5


def test_attention_mask_window_and_groups():
    t, nh, nkv, d = 9, 4, 2, 8
    g = torch.Generator().manual_seed(4)  # (unseeded draws made the far-key check below fail once in a while)
    q, k, v = (torch.randn(t, nh, d, generator=g), torch.randn(t, nkv, d, generator=g),
               torch.randn(t, nkv, d, generator=g))
    out = pl.causal_attention(q, k, v, 0.3)
    # row 0 sees only key 0; head h reads kv head h // 2
    assert torch.allclose(out[0, 3], v[0, 1])
    rep = pl.causal_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), 0.3)
    assert torch.allclose(out, rep, atol=1e-6)
    # window 1: every row sees itself only
    assert torch.allclose(pl.causal_attention(q, k, v, 0.3, window=1)[:, 0], v[:, 0])
    # a far key that stands out is found
    q2 = q.clone()
    q2[8, 0] = k[1, 0] * 50
    assert torch.allclose(pl.causal_attention(q2, k, v, 1.0)[8, 0], v[1, 0], atol=1e-4)
    assert not torch.allclose(pl.causal_attention(q2, k, v, 1.0, window=3)[8, 0], v[1, 0], atol=1e-2)


def test_forward_is_causal_and_deterministic(tmp_path):
    tiny.write_tiny(tmp_path / "a", "A")
    cfg, w = pl.load_model_dir(tmp_path / "a")
    toks = tiny.random_tokens(12, 256, 0)
    full = pl.forward(cfg, w, toks)
    assert full.shape == (12, 256)
    assert torch.allclose(pl.forward(cfg, w, toks[:7]), full[:7], atol=1e-6)  # later tokens do not leak back
    assert pl.generate_greedy(cfg, w, toks[:3], 4) == pl.generate_greedy(cfg, w, toks[:3], 4)


def test_sampler_follows_the_reference_rules():
    rng = pl.SplitMix64(0)
    assert rng.next_u64() == 0xE220A8397B1DCDAF and rng.next_u64() == 0x6E789E6AA1B965F4
    logits = [0.1, 2.0, 0.5, 1.9, -1.0, 1.95, 0.0]  # the reference's own test vector (sampler.rs:366-368)
    assert pl.greedy([1.0, 3.0, 3.0, 2.0]) == 1
    for seed in range(32):
        assert pl.sample(logits, 0.0, 0, 1.0, pl.SplitMix64(seed)) == 1
        assert pl.sample(logits, 1.5, 1, 1.0, pl.SplitMix64(seed)) == 1       # top_k = 1 is greedy
        assert pl.sample(logits, 1.0, 0, 1e-6, pl.SplitMix64(seed)) == 1      # a tiny top_p is greedy
        assert pl.sample(logits, 5.0, 3, 1.0, pl.SplitMix64(seed)) in (1, 3, 5)
    masked = [-np.inf, 0.0, -np.inf, 0.0]
    assert all(pl.sample(masked, 1.0, 0, 1.0, pl.SplitMix64(s)) in (1, 3) for s in range(32))
    a = [pl.sample(logits, 1.0, 5, 0.95, r) for r in [pl.SplitMix64(7)] for _ in range(16)]
    b = [pl.sample(logits, 1.0, 5, 0.95, r) for r in [pl.SplitMix64(7)] for _ in range(16)]
    assert a == b

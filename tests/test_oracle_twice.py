"""The oracle pinned twice over: by the literal vectors of the reference's own unit tests, and by a second plain
implementation written the reference's way (`plain_twin.py`: converted rows, adjacent pairs, token by token,
64-bit) that must agree with `plain_llama.py` on every tiny configuration."""
import numpy as np
import pytest
import torch

import plain_llama as pl
import plain_twin as twin
import tiny


def test_llama3_divisors_equal_the_references_literal_check():
    """src/provider/local/convert/config.rs:1266-1293: head size 16, theta 5e5, factor 32, low 1, high 4, original
    8192: eight divisors, the first exactly 1.0 ("highest frequency is unscaled"), the last exactly 32.0."""
    from cuca_b200.parts.rope import llama3_factors
    cfg = {"rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                                     "high_freq_factor": 4.0,
                                                     "original_max_position_embeddings": 8192}}
    ours = llama3_factors(16, 500000.0, 32.0, 1.0, 4.0, 8192)
    plain = pl.llama3_factors(cfg, 16)
    second, _ = twin.pair_divisors(cfg, 16)
    for f in (list(ours), plain, second):
        assert len(f) == 8 and f[0] == 1.0 and f[7] == 32.0
    assert list(ours) == plain == second


def test_row_permutation_equals_the_references_literal_check():
    """src/provider/local/convert/tensors.rs:1425-1473: two heads of four rows, per head rows [0, 1, 2, 3] become
    [0, 2, 1, 3]; one key head of four rows likewise."""
    rows = np.arange(8, dtype=np.float64)[:, None] * 2 + np.array([0.0, 1.0])
    assert twin.permute_rows(rows, 2)[:, 0].tolist() == [2.0 * i for i in (0, 2, 1, 3, 4, 6, 5, 7)]
    assert twin.permute_rows(rows[:4], 1)[:, 0].tolist() == [2.0 * i for i in (0, 2, 1, 3)]


def test_rope_tables_equal_the_references_definition_checks():
    """src/provider/local/model/rope.rs:176-219: the table is cos/sin of pos * base^(-2i/n) within 1e-6; a linear
    scale of 0.125 divides the angle."""
    cos, sin = pl.rope_tables(5, 8, 10_000.0, None)
    for pos in range(5):
        for i in range(4):
            theta = pos * 10_000.0 ** (-(2.0 * i) / 8.0)
            assert abs(float(cos[pos, i]) - np.cos(theta)) < 1e-6 and abs(float(sin[pos, i]) - np.sin(theta)) < 1e-6
    cos, _ = pl.rope_tables(3, 4, 100.0, None, freq_scale=0.125)
    for pos in range(3):
        for i in range(2):
            assert abs(float(cos[pos, i]) - np.cos(pos * 100.0 ** (-(2.0 * i) / 4.0) * 0.125)) < 1e-6
    from cuca_b200.parts.rope import rope_tables
    c2, s2 = rope_tables(5, 8, 10_000.0)
    c1, s1 = pl.rope_tables(5, 8, 10_000.0, None)
    assert torch.allclose(c1, c2, atol=1e-7) and torch.allclose(s1, s2, atol=1e-7)


@pytest.mark.parametrize("which,n", [("A", 40), ("B", 70), ("C", 33), ("D", 20), ("E", 24)])
def test_two_plain_implementations_agree(tmp_path, which, n):
    """Whole-sequence 32-bit matrices with a mask on Hugging Face row order, against token by token in 64-bit on
    converted rows with adjacent pairs: within 32-bit rounding of each other (the reference's own bound between
    its two computations is 5e-4 absolute, convert/oracle_local.rs:1-14). C carries non-zero attention biases,
    B and D llama3 divisors, C linear scaling, B and E tied embeddings."""
    d = tiny.write_tiny(tmp_path / which, which)
    cfg, w = pl.load_model_dir(d)
    tokens = tiny.random_tokens(n, cfg["vocab_size"], seed=17)
    a = pl.forward(cfg, w, tokens).double().numpy()
    cfg2, t2 = twin.read_folder(d)
    b = twin.logits_token_by_token(cfg2, t2, tokens)
    assert a.shape == b.shape
    scale = np.abs(b).max(axis=1, keepdims=True)
    assert float((np.abs(a - b) / scale).max()) < 2e-5
    assert (a.argmax(axis=1) == b.argmax(axis=1)).mean() > 0.9  # top-1 equal except at near ties
    if which == "C":
        assert any(k.endswith("q_proj.bias") for k in t2)

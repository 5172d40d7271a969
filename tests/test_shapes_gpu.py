"""Shapes off the beaten track through mixed replay against the plain implementation: head sizes 80, 96 and 112
(no tensor-core attention over prompt portions, no TMA-fed decode), one key/value head for 8 and for 16 query heads,
as many key/value heads as query heads, a width and vocabularies that are no powers of two, a bias, tied
embeddings; pages of 8 and of 64 positions."""
import pytest
import torch

import replay_util as ru
import tiny

pytestmark = pytest.mark.gpu


def _cfg(layers, hidden, nh, nkv, d, ff, vocab, tie=False, bias=False):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers,
            "hidden_size": hidden, "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": d,
            "intermediate_size": ff, "vocab_size": vocab, "max_position_embeddings": 1024, "rms_norm_eps": 1e-5,
            "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": tie, "attention_bias": bias}


SHAPES = {
    "d80_mha": _cfg(2, 160, 2, 2, 80, 328, 515),
    "d96_g2": _cfg(1, 200, 2, 1, 96, 264, 300, tie=True),
    "d112_bias": _cfg(1, 224, 2, 2, 112, 136, 999, bias=True),
    "d64_g8": _cfg(2, 512, 8, 1, 64, 520, 1001),
    "d128_g16": _cfg(1, 2048, 16, 1, 128, 1032, 640),
    "d128_g3": _cfg(2, 384, 3, 1, 128, 392, 2000, tie=True),
}
# relative to the largest logit of a row, from the measured error of a correct engine with headroom
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from cuca_b200.weights.random_init import write_random_model
    out = {}
    for name, cfg in SHAPES.items():
        d = tmp_path_factory.mktemp(name)
        write_random_model(d, cfg, 3, std=0.02, dtype=torch.bfloat16)
        out[name] = d
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("block_size", [8, 64])
@pytest.mark.parametrize("name", list(SHAPES))
def test_odd_shapes_mixed(folders, name, block_size, dtype):
    vocab = SHAPES[name]["vocab_size"]
    reqs = {f"r{n}": tiny.random_tokens(n, vocab, seed=n) for n in (3, 66, 150, 333, 520)}
    steps = ru.trace_mixed(reqs, max_live=4, seed=5)
    got = ru.run_in_process(folders[name], dtype, steps, ru.peak_tokens(steps), block_size=block_size)
    ru.compare(steps, got, reqs, ru.Oracle(folders[name]), TOL[dtype])


@pytest.mark.parametrize("name", ["d128_g16", "d64_g8", "d112_bias"])
def test_odd_shapes_whole_prompts(folders, name):
    """Whole prompts of several hundred tokens: the contractions over many tokens and the prompt attention."""
    vocab = SHAPES[name]["vocab_size"]
    reqs = {f"r{n}": tiny.random_tokens(n, vocab, seed=n) for n in (66, 333, 520)}
    steps = ru.trace_whole(reqs)
    got = ru.run_in_process(folders[name], "bfloat16", steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, ru.Oracle(folders[name]), TOL["bfloat16"])


@pytest.mark.parametrize("d,nh,nkv,hidden,ff,vocab", [(40, 4, 2, 96, 136, 301), (10, 6, 3, 64, 51, 13), (2, 3, 1, 7, 51, 301),
                                                      (136, 2, 1, 272, 136, 301), (250, 1, 1, 250, 51, 301)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_sizes_that_are_no_multiple_of_16(tmp_path, d, nh, nkv, hidden, ff, vocab, dtype):
    """Any even head size up to 256, odd widths, a vocabulary of 13: the plain kernels take them in both precisions."""
    from cuca_b200.weights.random_init import write_random_model
    cfg = _cfg(2, hidden, nh, nkv, d, ff, vocab)
    write_random_model(tmp_path, cfg, d, std=0.05, dtype=torch.bfloat16, norm_std=0.2)
    reqs = {f"r{n}": tiny.random_tokens(n, vocab, seed=n) for n in (5, 70, 200)}
    oracle = ru.Oracle(tmp_path)
    for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs), ru.trace_mixed(reqs, max_live=3, seed=1)):
        got = ru.run_in_process(tmp_path, dtype, steps, ru.peak_tokens(steps))
        ru.compare(steps, got, reqs, oracle, TOL[dtype])


def test_a_head_size_beyond_the_kernels_is_refused_when_the_model_is_built(tmp_path):
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.weights.random_init import write_random_model
    from cuca_b200.kernels import library, ops
    assert ops.ATTENTION_MAX_HEAD_DIM == int(library.load().cuca_attention_max_head_dim())
    with pytest.raises(ValueError, match="head size 320"):  # already when the parts are put together for the folder
        write_random_model(tmp_path, _cfg(1, 64, 2, 1, 320, 51, 301), 1, std=0.05, dtype=torch.bfloat16)
        EngineCore.from_folder(tmp_path, dtype="bfloat16", kv_tokens=256, max_sequences=4, block_size=16)

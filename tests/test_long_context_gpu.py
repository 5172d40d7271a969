"""Thousands of keys: one narrow layer at head sizes 128 and 64 with a context of 8,192, so that the key/value
rings of the attention kernels wrap many times and the page tables are read in many batches, while the plain
implementation on the CPU stays within seconds. Whole, in portions of 2,048 with a ragged tail, the last 64 tokens
one by one, four long requests mixed; and a sharp far key, so that one lost page would show even in bfloat16."""
import pytest
import torch

import plain_llama
import replay_util as ru
import sharp
import tiny

pytestmark = pytest.mark.gpu

LONG = {
    "128": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 256,
            "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 512,
            "vocab_size": 500, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 2048},
            "tie_word_embeddings": False},
    "64": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": 256,
           "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 392,
           "vocab_size": 377, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
           "rope_scaling": None, "tie_word_embeddings": True},
}
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = [6001, 4500, 5130, 3077]


@pytest.fixture(scope="module")
def long_models(tmp_path_factory):
    from cuca_b200.weights.random_init import write_random_model
    out = {}
    for which, cfg in LONG.items():
        d = tmp_path_factory.mktemp(f"long_{which}")
        write_random_model(d, cfg, seed=21, norm_std=0.2)
        reqs = {f"r{n}": tiny.random_tokens(n, cfg["vocab_size"], seed=600 + n) for n in LENGTHS}
        out[which] = (d, ru.Oracle(d), reqs)
    return out


def _sparse(steps, every=97):
    for s in steps:
        for e in s["entries"]:
            w = e["want"]
            if len(w) > 64:
                e["want"] = sorted(set(w[::every]) | set(w[-3:]))
    return steps


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("which", ["128", "64"])
def test_one_long_request_whole_in_portions_and_one_by_one(long_models, which, dtype):
    d, oracle, reqs = long_models[which]
    one = {"r6001": reqs["r6001"]}
    for steps in (_sparse(ru.trace_whole(one)),
                  ru.trace_portions(one, sizes=(2048, 2048, 1700, 141)),   # 6001 = 2048 + 2048 + 1700 + 141 + 64
                  ru.trace_tail_one_by_one(one, tail=64)):
        got = ru.run_in_process(d, dtype, steps, ru.peak_tokens(steps))
        ru.compare(steps, got, one, oracle, TOL[dtype])


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("which", ["128", "64"])
def test_four_long_requests_mixed(long_models, which, dtype):
    d, oracle, reqs = long_models[which]
    steps = ru.trace_mixed(reqs, max_live=3, seed=5, prefill_sizes=(2048, 700, 130, 64, 1111))
    peak = ru.peak_tokens(steps)
    assert peak < sum(ru.round64(len(t)) for t in reqs.values())  # the fourth request takes pages that were used
    got = ru.run_in_process(d, dtype, steps, peak)
    ru.compare(steps, got, reqs, oracle, TOL[dtype])


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("far", [3, 2617])
@pytest.mark.parametrize("which", ["128", "64"])
def test_a_far_key_among_thousands(tmp_path_factory, which, far, dtype):
    """The last position's logits hang on one key thousands of positions back (in the first page, or in the middle
    of the table), written by an earlier step: prefill in portions through the tensor-core attention, then single
    tokens through the TMA-fed decode attention."""
    from cuca_b200.weights.random_init import write_random_model
    cfg = LONG[which]
    d = tmp_path_factory.mktemp(f"sharp_{which}")
    write_random_model(d, cfg, seed=22, norm_std=0.2)
    V, last = cfg["vocab_size"], 5400
    key_tok, query_tok = V - 2, V - 1
    sharp.plant_far_key(d, last, far, key_tok, query_tok, qk_scale=4.0)
    toks = [t if t < V - 2 else V - 3 for t in tiny.random_tokens(last + 1, V, seed=31)]
    toks[far], toks[last] = key_tok, query_tok
    reqs = {"s": toks}
    cfgj, weights = plain_llama.load_model_dir(d)
    ref = plain_llama.forward(cfgj, weights, toks)
    moved = toks[:]
    moved[far] = 7
    influence = float((plain_llama.forward(cfgj, weights, moved)[-1] - ref[-1]).abs().max())
    assert influence > 10 * TOL[dtype] * float(ref[-1].abs().max()), "the far key must matter, or a lost page hides"
    oracle = ru.Oracle(d)
    oracle._cache["s"] = ref.numpy()
    for steps in (ru.trace_portions(reqs, sizes=(2048, 1000, 2, 2300, 52)), ru.trace_tail_one_by_one(reqs, tail=20)):
        got = ru.run_in_process(d, dtype, steps, ru.peak_tokens(steps))
        ru.compare(steps, got, reqs, oracle, TOL[dtype])

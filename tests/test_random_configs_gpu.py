"""Seeded random configurations and workloads: sizes, options and engine settings that no hand-written case names.

Replay: random tiny configurations (head sizes in steps of 16 up to 256, any number of heads and groups, widths and
vocabularies that are no multiple of eight, every rope scaling, biases, tied embeddings) through the four work splits
in both precisions against the plain implementation. Generation: in 32-bit the tokens of a batch of requests do not
depend on how many run together, on the page size, the portion size, the token budget, the size of the pool (with
preemption) or the prefix cache; the baseline is an engine that runs one request at a time."""
import random

import pytest
import torch

import replay_util as ru
import tiny

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def random_config(rng: random.Random) -> dict:
    d = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 192, 256])
    nkv = rng.choice([1, 2, 3, 4, 5, 8])
    nh = nkv * rng.choice([1, 2, 3, 4, 7, 8])
    if nh * d > 1024:
        nh = nkv = 1 if d > 128 else 2
    hidden = rng.choice([nh * d, 8 * rng.randint(4, 48), 2 * rng.randint(20, 200)])
    ff = rng.choice([8 * rng.randint(8, 90), 2 * rng.randint(30, 300), rng.randint(40, 500)])
    scaling = rng.choice([None, {"rope_type": "linear", "factor": rng.choice([2.0, 4.0, 1.5])},
                          {"rope_type": "llama3", "factor": rng.choice([8.0, 4.0, 32.0]), "low_freq_factor": 1.0,
                           "high_freq_factor": rng.choice([4.0, 2.0]),
                           "original_max_position_embeddings": rng.choice([64, 128, 256])}])
    return {"architectures": [rng.choice(["LlamaForCausalLM", "MistralForCausalLM"])], "model_type": "llama",
            "num_hidden_layers": rng.randint(1, 4), "hidden_size": min(hidden, 512), "num_attention_heads": nh,
            "num_key_value_heads": nkv, "head_dim": d, "intermediate_size": ff,
            "vocab_size": rng.choice([rng.randint(50, 400), rng.randint(400, 3000)]),
            "max_position_embeddings": rng.choice([512, 1024]), "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-5, 1e-4]),
            "rope_theta": rng.choice([10000.0, 500000.0, 25000.0, 1e6]), "rope_scaling": scaling,
            "tie_word_embeddings": rng.random() < 0.4, "attention_bias": rng.random() < 0.3}


def _folder(tmp_path, cfg, seed, std=0.02):
    from cuca_b200.weights.random_init import write_random_model
    write_random_model(tmp_path, cfg, seed, std=std, dtype=torch.bfloat16, norm_std=0.2)
    return tmp_path


@pytest.mark.parametrize("seed", range(8))
def test_replay_of_a_random_configuration(tmp_path, seed):
    rng = random.Random(7000 + seed)
    cfg = random_config(rng)
    folder = _folder(tmp_path, cfg, 7000 + seed)
    lens = sorted({rng.randint(1, 40), rng.randint(33, 140), rng.randint(100, 500), rng.randint(2, 400),
                   rng.randint(60, 250)})
    reqs = {f"r{n}": tiny.random_tokens(n, cfg["vocab_size"], seed=100 + n + seed) for n in lens}
    oracle = ru.Oracle(folder)
    for dtype in ("float32", "bfloat16"):
        for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs), ru.trace_portions(reqs),
                      ru.trace_mixed(reqs, max_live=4, seed=seed)):
            block = rng.choice([8, 16, 16, 32])
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=block)
            ru.compare(steps, got, reqs, oracle, TOL[dtype])


@pytest.mark.parametrize("seed", range(6))
def test_generation_does_not_depend_on_the_engines_settings(tmp_path, seed):
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig, SamplingConfig
    rng = random.Random(9000 + seed)
    nkv = rng.choice([1, 2, 3])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rng.randint(1, 3),
           "hidden_size": 8 * rng.randint(6, 30), "num_attention_heads": nkv * rng.choice([1, 2, 4]),
           "num_key_value_heads": nkv, "head_dim": rng.choice([16, 32, 48, 64, 128]),
           "intermediate_size": 8 * rng.randint(8, 50), "vocab_size": rng.randint(60, 900),
           "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
           "tie_word_embeddings": rng.random() < 0.5, "attention_bias": rng.random() < 0.3}
    folder = str(_folder(tmp_path, cfg, 9000 + seed, std=0.05))
    shared = tiny.random_tokens(rng.randint(20, 70), cfg["vocab_size"], seed=seed)
    prompts = []
    for r in range(rng.randint(3, 10)):
        own = tiny.random_tokens(rng.randint(1, 120), cfg["vocab_size"], seed=1000 * seed + r)
        prompts.append(shared + own if rng.random() < 0.5 else own)
    max_tokens, temperature, ctx = rng.randint(5, 60), rng.choice([0.0, 0.7]), 256

    def engine(**batching):
        block = batching.pop("block", 16)
        return LocalModel.load(LocalModelConfig(source=folder, dtype="float32", context_length=ctx, kv_block_size=block,
                                                sampling=SamplingConfig(seed=9), batching=BatchingConfig(**batching)))

    alone = engine(max_sequences=1)
    want = [alone.generate(p, max_tokens=max_tokens, temperature=temperature).tokens for p in prompts]
    del alone
    for _ in range(3):
        ms = rng.randint(2, 8)
        step = rng.choice([None, 64, 33, 128])
        settings = dict(max_sequences=ms, prefill_chunk=rng.choice([None, 16, 32, 7, 64]), max_step_tokens=step,
                        kv_tokens=rng.choice([None, ctx + 16, ctx + 64, 2 * ctx]), block=rng.choice([8, 16, 32]),
                        prefix_cache=rng.random() < 0.5)
        m = engine(**dict(settings))
        outs = m.generate(prompts, max_tokens=max_tokens, temperature=temperature)
        assert all(o.report.finish_reason == "length" for o in outs), settings
        assert [o.tokens for o in outs] == want, settings
        assert m.serving_stats().running == 0
        m.core.pools.check()
        del m

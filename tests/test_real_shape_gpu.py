"""The benchmarked layer sizes against the plain implementation: hidden 4096, 32 query heads on 8 key/value heads
of 128, feed-forward 14336, a vocabulary of 128,256, llama3 frequency scaling; two layers, so that the plain
implementation on the CPU stays within seconds. The four work splits in bfloat16 (the serving kernels at the sizes
they are timed at: the output head's many tiles per CTA, K slices left unadded over 4096 and 14336, the TMA-fed
decode attention with four query heads per key head), whole and mixed in 32-bit."""
import numpy as np
import pytest
import torch

import plain_llama
import replay_util as ru
import tiny

pytestmark = pytest.mark.gpu

REAL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "max_position_embeddings": 8192,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False,
}
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = [5, 70, 130, 300, 600]


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    """The folder (drawn on the device: the same bits as on the host, in seconds) and the oracle's logits."""
    from cuca_b200.weights.random_init import write_random_model
    d = tmp_path_factory.mktemp("real_shape")
    write_random_model(d, REAL, seed=5, norm_std=0.2, device="cuda:0")
    return d, ru.Oracle(d)


def _requests(extra=()):
    return {f"r{n}": tiny.random_tokens(n, REAL["vocab_size"], seed=300 + n) for n in list(LENGTHS) + list(extra)}


def _thin(steps, every=7):
    """Keep every `every`-th wanted place of long portions (and the last one): a row of logits is 0.5 MB."""
    for s in steps:
        for e in s["entries"]:
            w = e["want"]
            if len(w) > 16:
                e["want"] = sorted(set(w[::every]) | {w[-1]})
    return steps


def test_device_drawn_weights_equal_host_drawn(real):
    """The counter-based generator: the folder (drawn by the device kernel) holds the bits the host form gives."""
    from cuca_b200.weights.loader import host_normal, tensor_key
    _, w = plain_llama.load_model_dir(real[0])
    for name, first, n in (("model.layers.1.mlp.down_proj.weight", 4096 * 14336 - 5000, 5000),
                           ("lm_head.weight", 77_777_777, 3000), ("model.layers.0.self_attn.k_proj.weight", 0, 4096)):
        want = torch.from_numpy(host_normal(tensor_key(5, name), first, n, 0.0, 0.02)).bfloat16()
        assert torch.equal(w[name].view(-1)[first:first + n], want), name
    want = torch.from_numpy(host_normal(tensor_key(5, "model.norm.weight"), 0, 4096, 1.0, 0.2)).bfloat16()
    assert torch.equal(w["model.norm.weight"], want)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole(real, dtype):
    reqs = _requests()
    steps = _thin(ru.trace_whole(reqs))
    got = ru.run_in_process(real[0], dtype, steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, real[1], TOL[dtype])


def test_tail_one_by_one(real):
    reqs = _requests()
    steps = ru.trace_tail_one_by_one(reqs)
    got = ru.run_in_process(real[0], "bfloat16", steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, real[1], TOL["bfloat16"])


def test_portions(real):
    reqs = _requests()
    steps = ru.trace_portions(reqs, sizes=(5, 2, 130, 3, 2, 64, 7, 2, 65, 11))
    got = ru.run_in_process(real[0], "bfloat16", steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, real[1], TOL["bfloat16"])


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_mixed_pages_reused(real, dtype):
    reqs = _requests(extra=(40, 90))
    steps = ru.trace_mixed(reqs, max_live=3, seed=11, prefill_sizes=(9, 2, 70, 5, 130))
    peak = ru.peak_tokens(steps)
    assert peak < sum(ru.round64(len(t)) for t in reqs.values())
    got = ru.run_in_process(real[0], dtype, steps, peak)
    ru.compare(steps, got, reqs, real[1], TOL[dtype])


def test_greedy_tokens_through_captured_graphs(real):
    """Generation through the entry point at these sizes: prompts are prefilled eagerly, single tokens decode
    through captured graphs; every sampled token must be a near-maximum of the oracle's logits at its place."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, _ = real
    cfg, weights = plain_llama.load_model_dir(folder)
    prompts = [tiny.random_tokens(n, REAL["vocab_size"], seed=400 + n) for n in (3, 90)]
    m = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=512,
                                         batching=BatchingConfig(max_sequences=2)))
    outs = m.generate(prompts, max_tokens=12, temperature=0.0)
    assert m.backend.graph_steps >= 11
    for prompt, out in zip(prompts, outs):
        ref = plain_llama.forward(cfg, weights, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.03 * float(row.abs().max()), f"token {i} is no near-maximum"

"""The sampling kernel against the plain sampler (tests/plain_llama.py), and generation through the entry point."""
import numpy as np
import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu

GOLDEN, M64 = 0x9E3779B97F4A7C15, (1 << 64) - 1


def _signed(x):
    return x - (1 << 64) if x >= (1 << 63) else x


def _device_sample(logits, temperature, top_k, top_p, seeds, draws=1):
    """Each row samples `draws` tokens in a row from its own generator; returns [rows][draws]."""
    from cuca_b200.kernels import ops
    dev = torch.device("cuda:0")
    R, V = logits.shape
    lg = torch.tensor(logits, dtype=torch.float32, device=dev)
    rng = torch.tensor([_signed(s & M64) for s in seeds], dtype=torch.int64, device=dev)
    t = torch.tensor(temperature, dtype=torch.float32, device=dev)
    k = torch.tensor(top_k, dtype=torch.int32, device=dev)
    p = torch.tensor(top_p, dtype=torch.float32, device=dev)
    slots = torch.arange(R, dtype=torch.int32, device=dev)
    out = torch.empty(R, dtype=torch.int32, device=dev)
    scratch = torch.empty(R, ops.sample_scratch_words(V), dtype=torch.int64, device=dev)
    got = []
    for _ in range(draws):
        ops.sample(lg, t, k, p, rng, slots, out, scratch)
        got.append(out.tolist())
    return [list(col) for col in zip(*got)]


def _plain(logits_row, temperature, top_k, top_p, seed, draws):
    rng = plain_llama.SplitMix64(seed)
    return [plain_llama.sample(logits_row, temperature, top_k, top_p, rng) for _ in range(draws)]


def test_splitmix64_reference_vector():
    rng = plain_llama.SplitMix64(0)  # src/provider/local/sampler.rs:371-376
    assert rng.next_u64() == 0xE220A8397B1DCDAF and rng.next_u64() == 0x6E789E6AA1B965F4


@pytest.mark.parametrize("V", [7, 331, 5000])
def test_sampler_matches_plain_on_every_path(V):
    rs = np.random.default_rng(V)
    cases = [  # temperature, top_k, top_p
        (0.0, 0, 1.0), (0.8, 64, 0.95), (1.0, 5, 0.95), (1.5, 1, 1.0), (1.0, 3, 1.0), (0.7, 40, 0.5),
        (1.0, 0, 1.0), (1.3, 0, 1e-6), (1.0, 0, 0.3), (1.0, 0, 0.9), (2.0, 0, 0.97), (1.0, 2000, 0.9),
        (0.5, 2000, 1.0),
    ]
    R = len(cases)
    logits = (rs.standard_normal((R, V)) * 3).astype(np.float32)
    logits[:, 3] = logits[:, 5]  # ties: equal logits rank by ascending id
    logits[2, 1] = -np.inf
    seeds = [1000 + i for i in range(R)]
    got = _device_sample(logits, [c[0] for c in cases], [c[1] for c in cases], [c[2] for c in cases], seeds, draws=24)
    for i, (t, k, p) in enumerate(cases):
        want = _plain(logits[i], t, k, p, seeds[i], 24)
        wide = (k == 0 or k >= V or k > 1024) and t > 0
        if not wide:
            assert got[i] == want, f"case {i} {cases[i]}: {got[i]} != {want}"
        else:
            # wide cuts use parallel sums: same distribution, rounding may move a boundary draw
            same = sum(a == b for a, b in zip(got[i], want))
            assert same >= 22, f"case {i} {cases[i]}: only {same}/24 draws agree"


@pytest.mark.parametrize("V", [8193, 50000, 128256, 300000])
def test_greedy_rows_cut_over_several_ctas_give_the_one_ctas_token(V):
    """A greedy row of a large vocabulary is cut over several CTAs (`SampleSplit`): the first maximum wins as with one
    CTA, wherever it lies (in the first or the last part, at a part's edge, tied across parts), rows that draw and
    padding rows beside it are untouched, and the arrival counters are zero again after every launch."""
    import torch
    from cuca_b200.kernels import ops
    dev = torch.device("cuda:0")
    rs = np.random.default_rng(V)
    R = 9
    logits = torch.tensor((rs.standard_normal((R, V)) * 3).astype(np.float32), device=dev)
    per = -(-V // min(32, -(-V // 8192)))
    logits[0, V - 1] = 50.0                      # in the last part
    logits[1, 0] = 50.0                          # in the first
    logits[2, per - 1] = logits[2, per] = 50.0   # tied across the edge of two parts: the lower id wins
    logits[3, 7] = logits[3, V - 3] = 50.0       # tied across far parts
    logits[4, :] = float("-inf")                 # nothing above -inf: id 0
    logits[5, 5] = float("nan")                  # a NaN never wins
    slot_of_row = torch.tensor([0, 1, 2, 3, 4, 5, -1, 6, 7], dtype=torch.int32, device=dev)
    temperature = torch.tensor([0, 0, 0, 0, 0, 0, 0.8, 0], dtype=torch.float32, device=dev)
    top_k = torch.full((8,), 64, dtype=torch.int32, device=dev)
    top_p = torch.full((8,), 0.95, dtype=torch.float32, device=dev)
    split = ops.SampleSplit(16, dev)
    outs = []
    for use in (None, split, split):
        rng = torch.arange(8, dtype=torch.int64, device=dev) + 100
        out = torch.full((R,), -7, dtype=torch.int32, device=dev)
        ops.sample(logits, temperature, top_k, top_p, rng, slot_of_row, out, None, use)
        torch.cuda.synchronize()
        outs.append(out.tolist())
        assert int(split.count.abs().sum().item()) == 0
    assert outs[0] == outs[1] == outs[2]
    assert outs[0][:5] == [V - 1, 0, per - 1, 7, 0] and outs[0][6] == -1
    assert outs[0][5] == int(torch.argmax(torch.nan_to_num(logits[5], nan=-1e30)))
    assert outs[0][8] == int(torch.argmax(logits[8]))


def test_sampler_statistics_follow_the_distribution():
    V = 50
    logits = np.linspace(-2, 2, V, dtype=np.float32)[None, :].repeat(4, 0)
    got = _device_sample(logits, [1.0] * 4, [0, 0, 10, 10], [1.0, 0.8, 1.0, 0.8], [1, 2, 3, 4], draws=4000)
    p = np.exp(logits[0] - logits[0].max())
    p /= p.sum()
    freq = np.bincount(got[0], minlength=V) / 4000.0
    assert np.abs(freq - p).max() < 0.02
    assert set(got[2]) <= set(range(V - 10, V))  # top_k keeps the 10 best
    order = np.argsort(-p)
    nucleus = set(order[: int(np.searchsorted(np.cumsum(p[order]), 0.8)) + 1].tolist())
    assert set(got[1]) <= nucleus
    assert len(set(got[1])) > 5


def test_masked_ids_are_never_drawn_and_greedy_ignores_the_generator():
    V = 40
    logits = np.zeros((2, V), dtype=np.float32)
    logits[:, ::2] = -np.inf
    got = _device_sample(logits, [1.0, 0.0], [0, 0], [1.0, 1.0], [5, 5], draws=200)
    assert all(t % 2 == 1 for t in got[0])
    assert got[1] == [1] * 200  # first maximum


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for which in "AB":
        d = tmp_path_factory.mktemp(f"gen_{which}")
        tiny.write_tiny(d, which)
        out[which] = d
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(folders, dtype):
    """Tiny A's workload: prompts of 1/7/16/33 random ids (seed 1), 16 greedy tokens each, all four requests
    together under continuous batching, against the plain implementation re-run for every token."""
    from cuca_b200 import LocalModel, LocalModelConfig, BatchingConfig
    cfg, weights = plain_llama.load_model_dir(folders["A"])
    rs = np.random.default_rng(1)
    prompts = [rs.integers(0, cfg["vocab_size"], size=n).tolist() for n in (1, 7, 16, 33)]
    model = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype=dtype,
                                             batching=BatchingConfig(max_sequences=4)))
    outs = model.generate(prompts, max_tokens=16, temperature=0.0)
    for prompt, out in zip(prompts, outs):
        assert out.report.finish_reason == "length" and out.report.usage.completion_tokens == 16
        want = plain_llama.generate_greedy(cfg, weights, prompt, 16)
        if dtype == "float32":
            assert out.tokens == want
        else:
            # bfloat16 may take another branch where two logits nearly tie; until then it must agree
            ref = plain_llama.forward(cfg, weights, prompt + out.tokens)
            for i, tok in enumerate(out.tokens):
                row = ref[len(prompt) - 1 + i]
                assert float(row.max() - row[tok]) < 0.03 * float(row.abs().max()), f"token {i} is no near-maximum"
    # alone == together
    alone = model.generate(prompts[2], max_tokens=16, temperature=0.0)
    if dtype == "float32":
        assert alone.tokens == outs[2].tokens
    st = model.serving_stats()
    assert st.generated_tokens == 5 * 16 and st.running == 0 and st.used_blocks == 0


def test_seeded_sampling_matches_plain_in_32_bit(folders):
    """Tiny B's workload: 6 prompts of 3/12/40/64/90/130 ids (seed 3), portions of 32, pages of 16, 24 tokens at
    temperature 0.8 with seed 4: the engine's tokens equal the plain sampler run on the plain logits."""
    from cuca_b200 import LocalModel, LocalModelConfig, BatchingConfig, SamplingConfig
    cfg, weights = plain_llama.load_model_dir(folders["B"])
    rs = np.random.default_rng(3)
    prompts = [rs.integers(0, cfg["vocab_size"], size=n).tolist() for n in (3, 12, 40, 64, 90, 130)]
    model = LocalModel.load(LocalModelConfig(
        source=str(folders["B"]), dtype="float32", kv_block_size=16, sampling=SamplingConfig(seed=4),
        batching=BatchingConfig(max_sequences=4, max_step_tokens=64, prefill_chunk=32)))
    outs = model.generate(prompts, max_tokens=24, temperature=0.8)
    for prompt, out in zip(prompts, outs):
        rng = plain_llama.SplitMix64(4)  # every request restarts the generator from the seed
        ids = list(prompt)
        for i in range(24):
            logits = plain_llama.forward(cfg, weights, ids)[-1].numpy()
            tok = plain_llama.sample(logits, 0.8, 64, 0.95, rng)
            assert out.tokens[i] == tok, f"prompt of {len(prompt)}: token {i} differs"
            ids.append(tok)
    again = model.generate(prompts[1], max_tokens=24, temperature=0.8)
    assert again.tokens == outs[1].tokens  # a fixed seed reproduces
    other = model.generate(prompts[1], max_tokens=24, temperature=0.8, seed=5)
    assert other.tokens != outs[1].tokens
    k1 = model.generate(prompts[1], max_tokens=8, temperature=1.5, top_k=1)
    greedy = model.generate(prompts[1], max_tokens=8, temperature=0.0)
    assert k1.tokens == greedy.tokens  # top_k = 1 is greedy for any seed


def test_generation_with_so_few_pages_that_requests_queue_and_are_preempted(folders):
    from cuca_b200 import LocalModel, LocalModelConfig, BatchingConfig
    cfg, weights = plain_llama.load_model_dir(folders["A"])
    rs = np.random.default_rng(11)
    prompts = [rs.integers(0, cfg["vocab_size"], size=n).tolist() for n in (30, 28, 12, 40)]
    roomy = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype="float32",
                                             batching=BatchingConfig(max_sequences=4)))
    want = [o.tokens for o in roomy.generate(prompts, max_tokens=40, temperature=0.0)]
    tight = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype="float32", context_length=96,
                                             batching=BatchingConfig(max_sequences=4, kv_tokens=112)))  # 7 pages
    outs = tight.generate(prompts, max_tokens=40, temperature=0.0)
    assert [o.tokens for o in outs] == want
    st = tight.serving_stats()
    assert st.preemptions >= 1 and st.used_blocks == 0 and st.running == 0
    tight.core.pools.check()


def test_streaming_and_stop_token(folders):
    from cuca_b200 import LocalModel, LocalModelConfig
    model = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype="float32"))
    prompt = [5, 9, 200, 31]
    whole = model.generate(prompt, max_tokens=12, temperature=0.0)
    assert list(model.generate_tokens(prompt, max_tokens=12, temperature=0.0)) == whole.tokens
    cut = model.generate(prompt, max_tokens=12, temperature=0.0, stop_token_ids=[whole.tokens[5]])
    first = whole.tokens.index(whole.tokens[5])
    assert cut.tokens == whole.tokens[:first] and cut.report.finish_reason == "stop"


def test_stop_strings_and_text_with_a_tokenizer(folders, tmp_path):
    """A model folder with a tokenizer.json: prompts may be text, replies carry text, a stop string cuts the reply
    before its first occurrence and ends that request alone; without a tokenizer stop strings are refused."""
    import shutil
    import tokenizers
    from cuca_b200 import LocalModel, LocalModelConfig
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(folders["A"], folder)
    vocab = {f"w{i}": i for i in range(tiny.CONFIGS["A"]["vocab_size"])}
    tok = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="w0"))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    tok.save(str(folder / "tokenizer.json"))
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="float32"))
    prompt = "w5 w9 w200 w31"
    assert model.tokenize(prompt) == [5, 9, 200, 31]
    whole = model.generate(prompt, max_tokens=12, temperature=0.0)
    assert whole.tokens == model.generate([5, 9, 200, 31], max_tokens=12, temperature=0.0).tokens
    words = whole.text.split()
    assert words == [f"w{t}" for t in whole.tokens]
    stop = " ".join(words[5:7])                      # two tokens: the stop string is split across fragments
    at = whole.text.find(stop)
    fragments = []
    other = [7, 7, 7]
    cut, free = model.generate([prompt, other], max_tokens=12, temperature=0.0, stop=[stop],
                               on_text=lambda seq, frag: fragments.append((seq.id, frag)))
    assert cut.report.finish_reason == "stop" and cut.text == whole.text[:at]
    assert len(cut.tokens) < 12
    assert free.report.finish_reason == "length" and len(free.tokens) == 12 and stop not in free.text
    assert "".join(f for i, f in fragments if i == fragments[0][0]) in (cut.text, free.text)
    plain = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype="float32"))
    with pytest.raises(ValueError, match="tokenizer"):
        plain.generate([5, 9], max_tokens=2, stop=["x"])
    with pytest.raises(ValueError, match="tokenizer"):
        plain.generate("w5 w9", max_tokens=2)


def test_command_line(folders):
    import subprocess, sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "cuca_b200", "--model-dir", str(folders["A"]), "--prompt", "5 9 200 31",
                        "--max-tokens", "6", "--temperature", "0", "--dtype", "float32"],
                       capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert len(r.stdout.split()) == 6
    assert "load:" in r.stderr and "loaded on" in r.stderr and "timing: 4 prompt tokens" in r.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_from_cached_prefixes_equals_generation_from_scratch(folders, dtype):
    """With `prefix_cache` a request starts from the pages an earlier request left for the head of its prompt.
    Tokens must be those of an engine without it: in 32-bit exactly (the shared keys and values are the same
    bits), and the prompt rows that were found are not computed again."""
    from cuca_b200 import LocalModel, LocalModelConfig, BatchingConfig
    cfg, _ = plain_llama.load_model_dir(folders["A"])
    rs = np.random.default_rng(11)
    head = rs.integers(0, cfg["vocab_size"], size=50).tolist()
    prompts = [head + rs.integers(0, cfg["vocab_size"], size=n).tolist() for n in (5, 1, 23)] + [head[:37]]
    plain = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype=dtype,
                                             batching=BatchingConfig(max_sequences=4)))
    want = [plain.generate(p, max_tokens=12, temperature=0.0).tokens for p in prompts]
    cached = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype=dtype,
                                              batching=BatchingConfig(max_sequences=4, prefix_cache=True)))
    got, hits = [], []
    for p in prompts:                      # one after the other: each finds what the ones before left
        before = cached.serving_stats().prefix_hit_tokens
        got.append(cached.generate(p, max_tokens=12, temperature=0.0).tokens)
        hits.append(cached.serving_stats().prefix_hit_tokens - before)
    assert hits == [0, 48, 48, 32]         # whole pages of 16 below the last prompt token
    if dtype == "float32":
        assert got == want
    else:
        assert [g[:4] for g in got] == [w[:4] for w in want]
    # together: the first is admitted with nothing cached for `other`, later ones share pages with running requests
    other = rs.integers(0, cfg["vocab_size"], size=40).tolist()
    batch = [other + [1, 2], other + [3], other[:35]]
    outs = cached.generate(batch, max_tokens=8, temperature=0.0)
    if dtype == "float32":
        assert [o.tokens for o in outs] == [plain.generate(p, max_tokens=8, temperature=0.0).tokens for p in batch]
    st = cached.serving_stats()
    assert st.running == 0 and st.used_blocks == 0
    cached.core.pools.check()


def test_suppressed_tokens_are_never_sampled(folders):
    """`sampling.suppress_tokens`: their logits are -inf before sampling, in eager steps and in captured decode
    graphs alike; the tokens equal plain greedy decoding over the masked logits."""
    from cuca_b200 import LocalModel, LocalModelConfig, SamplingConfig
    from cuca_b200.kernels import ops
    dev = torch.device("cuda:0")
    lg = torch.randn(3, 50, device=dev)
    top = lg.argmax(-1)
    ops.suppress_tokens(lg, torch.tensor([int(top[0]), int(top[2]), 70, -3], dtype=torch.int32, device=dev))
    assert torch.isinf(lg[:, int(top[0])]).all() and torch.isinf(lg[:, int(top[2])]).all()
    assert int(torch.isinf(lg).sum()) == 3 * len({int(top[0]), int(top[2])})

    cfg, weights = plain_llama.load_model_dir(folders["A"])
    prompt = np.random.default_rng(21).integers(0, cfg["vocab_size"], size=9).tolist()
    free = plain_llama.generate_greedy(cfg, weights, prompt, 10)
    banned = sorted(set(free[:4]))
    want, ids = [], list(prompt)
    for _ in range(10):
        row = plain_llama.forward(cfg, weights, ids)[-1].clone()
        row[banned] = -float("inf")
        want.append(int(row.argmax()))
        ids.append(want[-1])
    model = LocalModel.load(LocalModelConfig(source=str(folders["A"]), dtype="float32",
                                             sampling=SamplingConfig(suppress_tokens=banned)))
    got = model.generate(prompt, max_tokens=10, temperature=0.0).tokens
    assert got == want and not set(got) & set(banned)
    sampled = model.generate(prompt, max_tokens=40, temperature=1.5, top_k=0, top_p=1.0, seed=3).tokens
    assert not set(sampled) & set(banned)

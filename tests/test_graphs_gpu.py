"""Decode through captured CUDA graphs: same tokens as the eager step, page tables kept in step, bursts."""
import numpy as np
import pytest

import plain_llama
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    d = tmp_path_factory.mktemp("graph_B")
    tiny.write_tiny(d, "B")
    return d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_decode_equals_eager_decode(folder, dtype):
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    rs = np.random.default_rng(21)
    prompts = [rs.integers(0, 512, size=n).tolist() for n in (3, 20, 47)]
    cfg = LocalModelConfig(source=str(folder), dtype=dtype, batching=BatchingConfig(max_sequences=4))
    with_graphs = LocalModel.load(cfg)
    assert with_graphs.backend.use_graphs
    a = with_graphs.generate(prompts, max_tokens=40, temperature=0.0)
    assert with_graphs.backend.graph_steps >= 39
    eager = LocalModel.load(cfg)
    eager.backend.use_graphs = False
    b = eager.generate(prompts, max_tokens=40, temperature=0.0)
    assert eager.backend.graph_steps == 0
    if dtype == "float32":
        assert [o.tokens for o in a] == [o.tokens for o in b]
        cfgj, weights = plain_llama.load_model_dir(folder)
        assert a[1].tokens == plain_llama.generate_greedy(cfgj, weights, prompts[1], 40)
    else:
        # bfloat16 may take another branch where two logits nearly tie (the split of keys over chunks differs
        # between the two paths): every token of either path must be a near-maximum of the oracle's logits
        cfgj, weights = plain_llama.load_model_dir(folder)
        for outs in (a, b):
            for prompt, out in zip(prompts, outs):
                ref = plain_llama.forward(cfgj, weights, prompt + out.tokens)
                for i, tok in enumerate(out.tokens):
                    row = ref[len(prompt) - 1 + i]
                    assert float(row.max() - row[tok]) < 0.03 * float(row.abs().max()), f"token {i}: no near-maximum"


@pytest.mark.parametrize("which", ["D", "E"])
def test_logits_inside_captured_graphs_match_plain(tmp_path_factory, which):
    """Head sizes 128 and 64 in bfloat16: a decode step is one captured graph whose attention is the fused,
    TMA-fed decode form reading unadded K slices. The logits each replay leaves are compared with the plain
    implementation at that position, and every sampled token is the first maximum of those logits."""
    import torch
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    d = tmp_path_factory.mktemp(f"graph_{which}")
    tiny.write_tiny(d, which)
    cfgj, weights = plain_llama.load_model_dir(d)
    vocab = cfgj["vocab_size"]
    prompts = [tiny.random_tokens(n, vocab, seed=500 + n) for n in (2, 61, 200, 500)]
    from cuca_b200.engine.graphs import DecodeGraphs
    DecodeGraphs.keep_logits = True  # the graphs of this engine keep the logits of their last replay
    try:
        m = LocalModel.load(LocalModelConfig(source=str(d), dtype="bfloat16", batching=BatchingConfig(max_sequences=4)))
        be, seen = m.backend, []
        _logits_of_graph_steps(m, be, seen, prompts, cfgj, weights)
    finally:
        DecodeGraphs.keep_logits = False


def _logits_of_graph_steps(m, be, seen, prompts, cfgj, weights):
    import torch
    run_graph = be._run_decode_graph

    def spy(plans):
        tokens = run_graph(plans)
        logits = be.last_graph.logits[:len(plans)].float().cpu()
        seen.extend((p.seq, p.seq.blocks.length - 1, logits[i], tokens[i]) for i, p in enumerate(plans))
        return tokens

    be._run_decode_graph = spy
    outs = m.generate(prompts, max_tokens=40, temperature=0.0)
    assert be.graph_steps >= 30 and len(seen) >= 100  # steps that also carry a prompt portion run eagerly
    refs = {}
    for seq, pos, logits, tok in seen:
        if id(seq) not in refs:
            refs[id(seq)] = plain_llama.forward(cfgj, weights, list(seq.request.prompt) + list(seq.completion))
        ref = refs[id(seq)][pos]
        err = float((logits - ref).abs().max()) / float(ref.abs().max())
        assert err <= 3e-2, f"position {pos}: relative error {err:.3e} inside the captured step"
        assert tok == int(torch.argmax(logits)), f"position {pos}: the sampled token is not the maximum"
    assert all(len(o.tokens) == 40 for o in outs)


def test_an_older_graph_survives_the_growth_of_the_attention_scratch(tmp_path_factory):
    """A captured step keeps the addresses of the decode attention's scratch. When a later, larger step makes that
    scratch grow, the older graph must still find its buffers alive and its counters zeroed."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.kernels import ops
    d = tmp_path_factory.mktemp("graph_grow")
    tiny.write_tiny(d, "D")
    vocab = tiny.CONFIGS["D"]["vocab_size"]
    prompt = tiny.random_tokens(300, vocab, seed=9)
    cfg = LocalModelConfig(source=str(d), dtype="bfloat16", batching=BatchingConfig(max_sequences=2))
    m = LocalModel.load(cfg)
    first = m.generate(prompt, max_tokens=12, temperature=0.0).tokens      # captures the one-row graph
    import torch
    dev = torch.device("cuda:0")
    part, cnt = ops.attention_scratch(dev, 1, 1)
    grown = ops.attention_scratch(dev, 2 * part.numel() + 1, 2 * cnt.numel() + 1)  # what a larger step would ask for
    assert grown[0].data_ptr() != part.data_ptr() and grown[1].data_ptr() != cnt.data_ptr()
    junk = [torch.full((part.numel(),), float("nan"), device=dev) for _ in range(4)]  # takes freed memory, if any
    again = m.generate(prompt, max_tokens=12, temperature=0.0).tokens      # replays the older graph
    assert again == first
    del junk


def test_sampled_decode_through_graphs_keeps_each_requests_generator(folder):
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    rs = np.random.default_rng(22)
    prompts = [rs.integers(0, 512, size=n).tolist() for n in (5, 9)]
    cfg = LocalModelConfig(source=str(folder), dtype="float32", batching=BatchingConfig(max_sequences=4))
    m = LocalModel.load(cfg)
    together = m.generate(prompts, max_tokens=20, temperature=0.9, seed=77)
    alone = [m.generate(p, max_tokens=20, temperature=0.9, seed=77) for p in prompts]
    assert [o.tokens for o in together] == [o.tokens for o in alone]


def test_a_capture_is_not_disturbed_by_the_collection_of_a_dropped_engine(folder):
    """A dropped engine lives on in dead reference cycles with its CUDA graphs and tensors until Python collects
    them. If that happened while another engine's step is being captured, resetting the old graphs would
    invalidate the capture: no automatic collection runs during a capture."""
    import gc
    import torch
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.engine import graphs
    cfg = LocalModelConfig(source=str(folder), dtype="float32", batching=BatchingConfig(max_sequences=4))
    prompt = np.random.default_rng(31).integers(0, 512, size=9).tolist()
    seen = []
    body = graphs.DecodeGraph._body

    def watched(self):
        if torch.cuda.is_current_stream_capturing():
            seen.append(gc.isenabled())
            [[] for _ in range(5000)]  # enough container allocations for several automatic collections
        return body(self)

    old_threshold = gc.get_threshold()
    gc.collect()
    gc.disable()
    try:
        first = LocalModel.load(cfg)
        want = first.generate(prompt, max_tokens=8, temperature=0.0).tokens
        del first                      # dead cycles now hold its captured graphs
        second = LocalModel.load(cfg)
        graphs.DecodeGraph._body = watched
        gc.set_threshold(50, 1, 1)     # collect all generations at every opportunity
        gc.enable()
        got = second.generate(prompt, max_tokens=8, temperature=0.0).tokens
    finally:
        graphs.DecodeGraph._body = body
        gc.set_threshold(*old_threshold)
        gc.enable()
    assert seen and not any(seen), "the collector was switched on during a capture"
    assert gc.isenabled() and got == want


def test_burst_feeds_tokens_back_on_the_device(folder):
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.engine.scheduler import DECODE, Request
    rs = np.random.default_rng(23)
    prompts = [rs.integers(0, 512, size=n).tolist() for n in (17, 30, 4)]
    m = LocalModel.load(LocalModelConfig(source=str(folder), dtype="float32",
                                         batching=BatchingConfig(max_sequences=4)))
    want = [o.tokens for o in m.generate(prompts, max_tokens=25, temperature=0.0)]
    seqs = [m.scheduler.submit(Request(p, max_tokens=100, temperature=0.0)) for p in prompts]
    while any(s.phase != DECODE for s in seqs):
        m.scheduler.turn()
    first = [s.pending for s in seqs]
    hist = m.backend.burst(seqs, first, 24).cpu().tolist()
    got = [[first[i]] + [row[i] for row in hist] for i in range(3)]
    assert got == want
    m.core.pools.check()


def test_a_fault_inside_a_replayed_step_fails_that_step_and_the_engine_goes_on(folder):
    """The device error word rides along with a captured step's sampled tokens. A page-table entry outside the
    pool (planted here; the kernels check every page id, record the error and skip the access) makes the step's
    tokens worthless: the step must raise before anything is applied, the running requests fail, pools and slots
    are reset, and the next request is served as if nothing had happened."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.engine.scheduler import DECODE, Request
    from cuca_b200.runtime import DeviceFault
    m = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", batching=BatchingConfig(max_sequences=2)))
    prompt = tiny.random_tokens(40, 512, seed=3)
    want = m.generate(prompt, max_tokens=6, temperature=0.0).tokens
    seq = m.scheduler.submit(Request(prompt, max_tokens=20, temperature=0.0))
    while seq.phase != DECODE:
        m.scheduler.turn()
    m.scheduler.turn()                                     # one good captured step
    assert m.backend.graph_steps >= 1 and len(seq.completion) == 2
    m.core.cache.tables[0][seq.slot, 0] = 1_000_000       # the first page of the request: no such page
    with pytest.raises(DeviceFault, match="page id"):
        m.scheduler.turn()
    assert seq.done and seq.finish_reason == "error" and len(seq.completion) == 2   # the lost step gave no token
    m.core.pools.check()
    assert m.core.pools.stats()["live_requests"] == 0
    assert m.generate(prompt, max_tokens=6, temperature=0.0).tokens == want

"""Trace replay on the GPU against the plain implementation: the four work splits, three tiny configurations and two
small ones at the head sizes of real models, 32-bit and bfloat16."""
import pytest
import torch

import replay_util as ru
import tiny

pytestmark = pytest.mark.gpu

# relative to the largest logit of a row; set from the measured error of a correct engine, with headroom
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"A": [1, 7, 16, 33, 65, 100, 128], "B": [3, 12, 40, 64, 90, 130, 255], "C": [2, 31, 77, 129, 300],
           "D": [5, 70, 130, 300, 700], "E": [33, 64, 200, 513, 640]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in "ABCDE":
        d = tmp_path_factory.mktemp(f"tiny_{which}")
        tiny.write_tiny(d, which)
        out[which] = d
    return out


def _requests(which):
    vocab = tiny.CONFIGS[which]["vocab_size"]
    return {f"r{n}": tiny.random_tokens(n, vocab, seed=100 + n) for n in LENGTHS[which]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_whole(models, which, dtype):
    reqs = _requests(which)
    steps = ru.trace_whole(reqs)
    got = ru.run_in_process(models[which], dtype, steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, ru.Oracle(models[which]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_tail_one_by_one(models, which, dtype):
    reqs = _requests(which)
    steps = ru.trace_tail_one_by_one(reqs)
    got = ru.run_in_process(models[which], dtype, steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, ru.Oracle(models[which]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_portions(models, which, dtype):
    reqs = _requests(which)
    steps = ru.trace_portions(reqs)
    got = ru.run_in_process(models[which], dtype, steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, ru.Oracle(models[which]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E"])
def test_mixed_pages_reused(models, which, dtype):
    reqs = _requests(which)
    reqs.update({f"s{n}": tiny.random_tokens(n, tiny.CONFIGS[which]["vocab_size"], seed=200 + n)
                 for n in LENGTHS[which][1:5]})
    steps = ru.trace_mixed(reqs, max_live=4, seed=7)
    peak = ru.peak_tokens(steps)
    total = sum(ru.round64(len(t)) for t in reqs.values())
    assert peak < total, "the pool must be so small that pages are used again"
    got = ru.run_in_process(models[which], dtype, steps, peak)
    ru.compare(steps, got, reqs, ru.Oracle(models[which]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, dtype):
    """bin/trace_run itself, as a subprocess."""
    reqs = {k: v for k, v in list(_requests("A").items())[:4]}
    steps = ru.trace_portions(reqs)
    got = ru.run_subprocess(models["A"], dtype, steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, ru.Oracle(models["A"]), TOL[dtype])


def test_fp32_splits_agree_to_the_bit(models):
    """In 32-bit a position's logits do not depend on how the tokens were cut: every kernel's arithmetic for a
    row is independent of the batch, so whole, one-by-one and portioned replays agree exactly."""
    import numpy as np
    reqs = {"r": tiny.random_tokens(100, tiny.CONFIGS["B"]["vocab_size"], seed=5)}
    whole = ru.trace_whole(reqs)
    a = ru.run_in_process(models["B"], "float32", whole, 128)[0]
    steps = ru.trace_portions(reqs)
    got = ru.run_in_process(models["B"], "float32", steps, 128)
    pos = 0
    for s in steps:
        e = s["entries"][0]
        for j, w in enumerate(e["want"]):
            assert np.array_equal(got[s["step"]][j], a[pos + w]), f"position {pos + w} differs between splits"
        pos += len(e["tokens"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_one_by_one(models, dtype):
    """A short prompt, then two hundred tokens one at a time: every position crosses page and key-tile edges."""
    reqs = {"long": tiny.random_tokens(250, tiny.CONFIGS["B"]["vocab_size"], seed=77)}
    steps = ru.trace_tail_one_by_one(reqs, tail=230)
    got = ru.run_in_process(models["B"], dtype, steps, 256)
    ru.compare(steps, got, reqs, ru.Oracle(models["B"]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_first_tokens_of_a_sequence(models, which, dtype):
    """Positions 0, 1, 2 ...: a request that starts with single tokens, beside one that starts with two."""
    vocab = tiny.CONFIGS[which]["vocab_size"]
    reqs = {"x": tiny.random_tokens(6, vocab, seed=1), "y": tiny.random_tokens(7, vocab, seed=2)}
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": reqs["x"][:1], "want": [0]},
                                     {"id": "y", "tokens": reqs["y"][:2], "want": [0, 1]}], "end": []}]
    for i in range(1, 6):
        steps.append({"step": i, "entries": [{"id": "x", "tokens": reqs["x"][i:i + 1], "want": [0]},
                                             {"id": "y", "tokens": reqs["y"][i + 1:i + 2], "want": [0]}],
                      "end": ["x", "y"] if i == 5 else []})
    got = ru.run_in_process(models[which], dtype, steps, 128)
    ru.compare(steps, got, reqs, ru.Oracle(models[which]), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_is_found_after_cuts(tmp_path_factory, dtype):
    """Random weights give flat attention that would hide a lost key. Here layer 0's query and key projections
    are scaled so that scores are sharp, and one embedding row is built so that the last token's query (head 0)
    points at the key of position 3: the last position's logits then hang on a key hundreds of positions back,
    in a page written by an earlier step."""
    import plain_llama
    from cuca_b200.weights import safetensors_io as st
    d = tmp_path_factory.mktemp("sharp")
    tiny.write_tiny(d, "B")
    cfg, w = plain_llama.load_model_dir(d)
    pre = "model.layers.0.self_attn."
    for name, scale in (("q_proj", 8.0), ("k_proj", 8.0), ("v_proj", 4.0), ("o_proj", 4.0)):
        w[pre + name + ".weight"] = (w[pre + name + ".weight"].float() * scale).to(torch.bfloat16)
    P, far, dh = 239, 3, cfg["head_dim"]
    cos, sin = plain_llama.rope_tables(P + 1, dh, cfg["rope_theta"], plain_llama.llama3_factors(cfg, dh))
    E = w["model.embed_tokens.weight"].float()
    wq, wk = w[pre + "q_proj.weight"].float()[:dh], w[pre + "k_proj.weight"].float()
    n_key = plain_llama.rms_norm(E[498:499], torch.ones(E.shape[1]), cfg["rms_norm_eps"])
    k_far = plain_llama.rotate_half_split((n_key @ wk.T).view(1, 1, dh), cos[far:far + 1], sin[far:far + 1])
    target = plain_llama.rotate_half_split(k_far, cos[P:P + 1], -sin[P:P + 1])[0, 0]  # rotate back from position P
    n_query = torch.linalg.pinv(wq) @ target
    E[499] = n_query / n_query.norm() * E[498].norm()
    w["model.embed_tokens.weight"] = E.to(torch.bfloat16)
    st.write_safetensors(d / "model.safetensors", w)

    toks = [t if t not in (498, 499) else 497 for t in tiny.random_tokens(P + 1, 512, seed=31)]
    toks[far], toks[P] = 498, 499
    reqs = {"s": toks}
    cfg, weights = plain_llama.load_model_dir(d)
    ref = plain_llama.forward(cfg, weights, toks)
    moved = toks[:]
    moved[far] = 7
    influence = float((plain_llama.forward(cfg, weights, moved)[-1] - ref[-1]).abs().max())
    assert influence > 10 * TOL[dtype] * float(ref[-1].abs().max()), "the far key must matter, or a lost page hides"
    for steps in (ru.trace_portions(reqs, sizes=(100, 2, 60, 7, 64, 3, 2, 2)), ru.trace_tail_one_by_one(reqs)):
        got = ru.run_in_process(d, dtype, steps, 256)
        ru.compare(steps, got, reqs, ru.Oracle(d), TOL[dtype])


@pytest.mark.parametrize("which", ["B", "D"])
def test_fp32_a_row_beside_neighbours_equals_the_row_alone_to_the_bit(models, which):
    """The exactness contract at the step level (the reference's `check_batched`,
    src/provider/local/model/cpu.rs:4072-4141): three requests over five steps, mixing a joint prefill, single
    tokens, a request that sits a step out and a four-token portion beside single tokens. In 32-bit every logit of
    every step equals, bit for bit, what the same request gives when it runs alone and whole."""
    import numpy as np
    vocab = tiny.CONFIGS[which]["vocab_size"]
    reqs = {"a": tiny.random_tokens(9, vocab, seed=41), "b": tiny.random_tokens(14, vocab, seed=42),
            "c": tiny.random_tokens(8, vocab, seed=43)}

    def ent(rid, lo, hi):
        return {"id": rid, "tokens": reqs[rid][lo:hi], "want": list(range(hi - lo))}

    steps = [
        {"step": 0, "entries": [ent("a", 0, 5), ent("b", 0, 9), ent("c", 0, 2)], "end": []},
        {"step": 1, "entries": [ent("a", 5, 6), ent("b", 9, 10), ent("c", 2, 3)], "end": []},
        {"step": 2, "entries": [ent("a", 6, 7), ent("c", 3, 7)], "end": []},            # b sits out
        {"step": 3, "entries": [ent("c", 7, 8), ent("b", 10, 11), ent("a", 7, 8)], "end": ["c"]},
        {"step": 4, "entries": [ent("b", 11, 14), ent("a", 8, 9)], "end": ["a", "b"]},
    ]
    got = ru.run_in_process(models[which], "float32", steps, ru.peak_tokens(steps))
    alone = {}
    for rid, toks in reqs.items():
        whole = ru.trace_whole({rid: toks})
        alone[rid] = ru.run_in_process(models[which], "float32", whole, 64)[0]
    pos = {rid: 0 for rid in reqs}
    for s in steps:
        row = 0
        for e in s["entries"]:
            for w in e["want"]:
                p = pos[e["id"]] + w
                assert np.array_equal(got[s["step"]][row], alone[e["id"]][p]), \
                    f"step {s['step']}, request {e['id']}, position {p}: not the bits of the request alone"
                row += 1
            pos[e["id"]] += len(e["tokens"])

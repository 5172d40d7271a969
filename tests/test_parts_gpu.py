"""Parts alone, and the generality of the layer assembly: a toy architecture defined here, in the test, with a
mixer that keeps state of its own per request, a routed feed-forward, a position encoding without fused tables,
a windowed attention layer, a layer that reads another layer's cache and a layer named twice in the run order.
Nothing in the framework's files knows these parts; they are registered, built, loaded with random weights and
stepped through the ordinary step function, and compared with a plain whole-sequence reference."""
import math

import numpy as np
import pytest
import torch

import plain_llama
import tiny

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------ toy parts
def _register_toy_parts():
    from cuca_b200.config.registry import register_architecture
    from cuca_b200.models.spec import LayerSpec, ModelSpec, Run
    from cuca_b200.parts.base import (CacheNeeds, FeedForward, Mixer, PartSpec, PositionEncoding, StateNeeds,
                                      TensorNeed, MIXERS, register_feed_forward, register_mixer, register_position)
    if "toy_cumsum" in MIXERS:
        return

    @register_mixer("toy_cumsum")
    class CumSumMixer(Mixer):
        """y_t = W (sum of h_s for s <= t): a recurrent mixer whose state (the running sum) lives in the
        request's slot."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.width = spec.params["width"]

        def tensors(self):
            return {self.spec.tensors["w"]: TensorNeed((self.width, self.width))}

        def load(self, get):
            self.w = get(self.spec.tensors["w"])

        def cache_needs(self):
            return CacheNeeds(state=StateNeeds((self.width,), "float32"))

        def forward(self, h, stream, step, cache):
            r = 0
            for slot, count in zip(step.host["slots"], step.host["counts"]):
                cs = torch.cumsum(h[r:r + count].float(), 0) + cache.state[slot]
                cache.state[slot] = cs[-1]
                # 64-bit products: torch's 32-bit matmul may run in a reduced-precision tensor-core mode
                stream.data[r:r + count] += (cs.double() @ self.w.double().T).float()
                r += count

    @register_feed_forward("toy_routed")
    class RoutedFF(FeedForward):
        """Top-1 of a few experts by 32-bit router logits; each expert is relu(x U^T) D^T."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.p = spec.params

        def tensors(self):
            t, p = self.spec.tensors, self.p
            out = {t["router"]: TensorNeed((p["experts"], p["width"]))}
            for e in range(p["experts"]):
                out[t["up"].format(e)] = TensorNeed((p["inner"], p["width"]))
                out[t["down"].format(e)] = TensorNeed((p["width"], p["inner"]))
            return out

        def load(self, get):
            t = self.spec.tensors
            self.router = get(t["router"])
            self.up = [get(t["up"].format(e)) for e in range(self.p["experts"])]
            self.down = [get(t["down"].format(e)) for e in range(self.p["experts"])]

        def forward(self, h, stream, step):
            x = h.double()
            choice = (x @ self.router.double().T).argmax(-1)
            for e in range(self.p["experts"]):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(x[rows] @ self.up[e].double().T) @ self.down[e].double().T
                    stream.data.index_add_(0, rows, y.float())

    @register_position("toy_adjacent_rope")
    class AdjacentRope(PositionEncoding):
        """Rotates adjacent pairs (2i, 2i+1); offers no fused tables, so the mixer calls apply()."""

        def prepare(self, context_length):
            d, theta = self.spec.params["head_dim"], self.spec.params["theta"]
            inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
            ang = torch.arange(context_length, dtype=torch.float64)[:, None] * inv[None, :]
            self.cos = torch.cos(ang).float().to(self.rt.device)
            self.sin = torch.sin(ang).float().to(self.rt.device)

        def apply(self, qkv, n_heads, n_kv_heads, head_dim, positions):
            T = qkv.shape[0]
            heads = qkv[:, :(n_heads + n_kv_heads) * head_dim].view(T, n_heads + n_kv_heads, head_dim // 2, 2)
            c = self.cos[positions.long()][:, None, :]
            s = self.sin[positions.long()][:, None, :]
            a, b = heads[..., 0].float().clone(), heads[..., 1].float().clone()  # .float() of 32-bit is a view
            heads[..., 0] = (a * c - b * s).to(qkv.dtype)
            heads[..., 1] = (a * s + b * c).to(qkv.dtype)

    @register_architecture("ToyForCausalLM")
    def build_toy(cfg):
        E, d, nh, nkv, V = cfg["width"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"], cfg["vocab"]
        eps = cfg["eps"]

        def norm(name):
            return PartSpec("rmsnorm", {"width": E, "eps": eps}, {"weight": name})

        def attn(i, window=None, position=None, shares=False):
            names = {"q": f"l{i}.q", "o": f"l{i}.o", "k": f"l{i}.k", "v": f"l{i}.v"}
            return PartSpec("attention", {"width": E, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d,
                                          "window": window, "scale": None, "position": position,
                                          "shares_cache": shares}, names)

        def swiglu(i):
            return PartSpec("swiglu", {"width": E, "inner": cfg["inner"]},
                            {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})

        rope = PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": 10000.0, "scaling": {"kind": "default"}})
        adj = PartSpec("toy_adjacent_rope", {"head_dim": d, "theta": 777.0})
        layers = [
            LayerSpec(PartSpec("pre_norm"), attn(0, None, rope), norm("l0.n1"), swiglu(0), norm("l0.n2")),
            LayerSpec(PartSpec("pre_norm"), PartSpec("toy_cumsum", {"width": E}, {"w": "l1.w"}), norm("l1.n1"),
                      PartSpec("toy_routed", {"width": E, "inner": 24, "experts": 3},
                               {"router": "l1.router", "up": "l1.up{}", "down": "l1.down{}"}), norm("l1.n2")),
            LayerSpec(PartSpec("pre_norm"), attn(2, cfg["window"], adj), norm("l2.n1"), swiglu(2), norm("l2.n2")),
            LayerSpec(PartSpec("pre_norm"), attn(3, None, rope, shares=True), norm("l3.n1"), swiglu(3), norm("l3.n2")),
        ]
        schedule = [Run(0, 0), Run(1, 1), Run(2, 2), Run(3, 0, owns=False), Run(1, 3)]
        return ModelSpec("ToyForCausalLM", V, E, cfg["max_positions"],
                         PartSpec("embedding", {"vocab": V, "width": E}, {"weight": "embed"}), layers, schedule,
                         norm("final"), PartSpec("head", {"vocab": V, "width": E}, {"weight": "embed"}))


TOY = {"architectures": ["ToyForCausalLM"], "width": 48, "head_dim": 16, "heads": 3, "kv_heads": 1, "vocab": 97,
       "inner": 40, "eps": 2e-5, "window": 9, "max_positions": 256}


def _toy_reference(w, tokens):
    """The toy model on a whole sequence, plainly (CPU, 32-bit)."""
    c = TOY
    E, d, nh, nkv = c["width"], c["head_dim"], c["heads"], c["kv_heads"]
    t = len(tokens)
    f = {k: v.float() for k, v in w.items()}
    cos, sin = plain_llama.rope_tables(t, d, 10000.0, None)
    inv = 777.0 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
    ang = torch.arange(t, dtype=torch.float64)[:, None] * inv[None, :]
    acos, asin = torch.cos(ang).float(), torch.sin(ang).float()

    def adjacent(x):  # [t, heads, d]
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * acos[:, None, :] - b * asin[:, None, :]
        out[..., 1::2] = a * asin[:, None, :] + b * acos[:, None, :]
        return out

    def ffn(i, x):
        return plain_llama.swiglu(x, f[f"l{i}.gate"], f[f"l{i}.up"], f[f"l{i}.down"])

    x = f["embed"][torch.tensor(tokens)]
    kv0 = None
    for layer, cache in [(0, 0), (1, 1), (2, 2), (3, 0), (1, 3)]:
        h = plain_llama.rms_norm(x, f[f"l{layer}.n1"], c["eps"])
        if layer == 1:
            x = x + torch.cumsum(h, 0) @ f["l1.w"].T
            g = plain_llama.rms_norm(x, f["l1.n2"], c["eps"])
            choice = (g @ f["l1.router"].T).argmax(-1)
            y = torch.zeros_like(x)
            for e in range(3):
                rows = (choice == e).nonzero().flatten()
                y[rows] = torch.relu(g[rows] @ f[f"l1.up{e}"].T) @ f[f"l1.down{e}"].T
            x = x + y
            continue
        q = (h @ f[f"l{layer}.q"].T).view(t, nh, d)
        if layer == 3:
            q = plain_llama.rotate_half_split(q, cos, sin)
            k, v = kv0
            window = None
        else:
            k = (h @ f[f"l{layer}.k"].T).view(t, nkv, d)
            v = (h @ f[f"l{layer}.v"].T).view(t, nkv, d)
            if layer == 0:
                q, k = plain_llama.rotate_half_split(q, cos, sin), plain_llama.rotate_half_split(k, cos, sin)
                kv0, window = (k, v), None
            else:
                q, k, window = adjacent(q), adjacent(k), c["window"]
        a = plain_llama.causal_attention(q, k, v, 1.0 / math.sqrt(d), window).reshape(t, nh * d)
        x = x + a @ f[f"l{layer}.o"].T
        x = x + ffn(layer, plain_llama.rms_norm(x, f[f"l{layer}.n2"], c["eps"]))
    return plain_llama.rms_norm(x, f["final"], c["eps"]) @ f["embed"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_registered_built_and_stepped(dtype):
    _register_toy_parts()
    from cuca_b200.config.registry import build_spec
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.step import StepEntry
    from cuca_b200.models.model import Model
    from cuca_b200.weights.loader import RandomSource

    spec = build_spec(TOY)
    needs = Model(spec).tensor_needs()
    assert "l3.k" not in needs and "l3.q" in needs  # the layer that reads another's cache has no keys of its own
    source = RandomSource(needs, seed=11, std=0.08, device="cpu", dtype=torch.bfloat16)
    weights = {n: source.read(n) for n in source.shapes()}
    core = EngineCore(spec, source, dtype=dtype, kv_tokens=192, max_sequences=4, block_size=8, window_pools="full")
    # groups: full attention (caches 0) and the windowed layer (cache 2); the two runs of layer 1 own state each
    assert {(g.window, g.cache_ids) for g in core.groups} == {(None, (0,)), (9, (2,))}
    assert sorted(core.cache.state) == [1, 3]
    assert not core.model.graph_safe()

    rs = np.random.default_rng(5)
    reqs = {name: rs.integers(0, TOY["vocab"], size=n).tolist() for name, n in (("a", 70), ("b", 33), ("c", 90))}
    ref = {k: _toy_reference(weights, v) for k, v in reqs.items()}
    tol = 3e-5 if dtype == "float32" else 4e-2

    def check(logits, name, positions):
        got = logits.float().cpu()
        want = ref[name][positions]
        err = float((got - want).abs().max() / want.abs().max())
        assert err < tol, (name, positions[:3], err)

    live = {}

    def entry(name, n, want):
        if name not in live:
            slot = core.slots.alloc()
            core.cache.clear_slot(slot)
            live[name] = [core.pools.new_seq(), slot, 0]
        blocks, slot, pos = live[name]
        core.pools.reserve(blocks, pos + n)
        live[name][2] = pos + n
        return StepEntry(blocks, slot, reqs[name][pos:pos + n], want), list(range(pos, pos + n))

    def finish(name):
        blocks, slot, _ = live.pop(name)
        core.pools.release(blocks)
        core.slots.release(slot)

    # request a whole; then b and c in portions beside each other (state, window pages and shared cache all cut)
    e, pos = entry("a", 70, list(range(70)))
    check(core.stepper.step([e]), "a", pos)
    finish("a")
    cuts_b, cuts_c = [5, 2, 17, 1, 8], [30, 1, 1, 40, 2, 16]
    ib = ic = 0
    while ib < len(cuts_b) or ic < len(cuts_c):
        entries, meta = [], []
        if ib < len(cuts_b):
            e, pos = entry("b", cuts_b[ib], [cuts_b[ib] - 1])
            entries.append(e)
            meta.append(("b", [pos[-1]]))
            ib += 1
        if ic < len(cuts_c):
            e, pos = entry("c", cuts_c[ic], [0, cuts_c[ic] - 1] if cuts_c[ic] > 1 else [0])
            entries.append(e)
            meta.append(("c", [pos[0], pos[-1]] if cuts_c[ic] > 1 else [pos[0]]))
            ic += 1
        logits = core.stepper.step(entries)
        row = 0
        for name, positions in meta:
            check(logits[row:row + len(positions)], name, positions)
            row += len(positions)
    core.rt.check_device_errors()
    # the windowed group gave pages back while c was still running
    blocks_c = live["c"][0]
    win = [i for i, g in enumerate(core.groups) if g.window][0]
    assert blocks_c.tables[win][0] == -1 and blocks_c.tables[1 - win][0] != -1
    finish("b")
    finish("c")
    core.pools.check()
    assert all(p.free == p.n_blocks for p in core.pools.pools)


def test_the_state_mixer_through_the_entry_point_and_the_prefix_cache_refusal():
    """The toy architecture through `LocalModel.generate`: requests with state in their slots run under the
    scheduler (graphs off by the parts' own declaration) and give the tokens of the plain reference. With
    `prefix_cache` the engine refuses to load: cached pages do not bring a mixer's running state back, and a
    request that started from them would compute with empty state (the reference snapshots such state,
    src/provider/local/engine/scheduler.rs:813-830; this engine says no)."""
    _register_toy_parts()
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig, RandomWeights
    from cuca_b200.cache.pages import StatefulCacheError
    from cuca_b200.config.registry import build_spec
    from cuca_b200.models.model import Model
    from cuca_b200.weights.loader import RandomSource

    def config(prefix_cache):
        return LocalModelConfig(model_config=TOY, random_weights=RandomWeights(seed=11, std=0.08), dtype="float32",
                                kv_block_size=8, batching=BatchingConfig(max_sequences=3, prefix_cache=prefix_cache,
                                                                         max_step_tokens=32, prefill_chunk=16))

    with pytest.raises(StatefulCacheError, match="prefix_cache"):
        LocalModel.load(config(True))
    m = LocalModel.load(config(False))
    assert not m.backend.use_graphs
    source = RandomSource(Model(build_spec(TOY)).tensor_needs(), seed=11, std=0.08, device="cpu", dtype=torch.bfloat16)
    weights = {n: source.read(n) for n in source.shapes()}
    prompts = [tiny.random_tokens(n, TOY["vocab"], seed=70 + n) for n in (5, 40, 23)]
    outs = m.generate(prompts, max_tokens=10, temperature=0.0)
    for prompt, out in zip(prompts, outs):
        ref = _toy_reference(weights, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) <= 2e-5 * float(row.abs().max()), f"token {i} is not the maximum"
    with pytest.raises(StatefulCacheError, match="rolled back"):
        m.core.pools.truncate(m.core.pools.new_seq(), 0)


# ------------------------------------------------------------------------------------------ other arrangements
def _register_parallel_parts():
    from cuca_b200.config.registry import register_architecture
    from cuca_b200.models.spec import LayerSpec, ModelSpec, default_schedule
    from cuca_b200.parts.base import BLOCKS, Block, Mixer, PartSpec, TensorNeed, register_block, register_mixer
    if "toy_parallel" in BLOCKS:
        return

    @register_block("toy_parallel")
    class ParallelBlock(Block):
        """x += mixer(n) + ffn(n) with one norm n = norm(x): both branches add into the stream one after the other,
        neither reads what the other added."""

        def forward(self, stream, step, cache):
            h = self.mixer_norm.forward(stream)
            self.mixer.forward(h, stream, step, cache)
            self.feed_forward.forward(h, stream, step)

    @register_mixer("toy_stream_reader")
    class StreamReader(Mixer):
        """y = (h W^T) * mean|x| of the row's residual stream: a mixer that reads the stream itself."""

        def tensors(self):
            E = self.spec.params["width"]
            return {self.spec.tensors["w"]: TensorNeed((E, E))}

        def load(self, get):
            self.w = get(self.spec.tensors["w"])

        def forward(self, h, stream, step, cache):
            x = stream.data
            y = (h.double() @ self.w.double().T) * x.double().abs().mean(-1, keepdim=True)
            stream.add(y.float())

    @register_architecture("ToyParallelForCausalLM")
    def build(cfg):
        E, d, nh, nkv, V = cfg["width"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"], cfg["vocab"]
        rope = PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": 10000.0, "scaling": {"kind": "default"}})

        def norm(name):
            return PartSpec("rmsnorm", {"width": E, "eps": cfg["eps"]}, {"weight": name})

        def attn(i):
            return PartSpec("attention", {"width": E, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "window": None,
                                          "scale": None, "position": rope},
                            {"q": f"l{i}.q", "o": f"l{i}.o", "k": f"l{i}.k", "v": f"l{i}.v"})

        def swiglu(i):
            return PartSpec("swiglu", {"width": E, "inner": cfg["inner"]},
                            {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})

        layers = [LayerSpec(PartSpec("pre_norm"), attn(0), norm("l0.n1"), swiglu(0), norm("l0.n2")),
                  LayerSpec(PartSpec("toy_parallel"), attn(1), norm("l1.n1"), swiglu(1), None),
                  LayerSpec(PartSpec("pre_norm"), PartSpec("toy_stream_reader", {"width": E}, {"w": "l2.w"}),
                            norm("l2.n1"), swiglu(2), norm("l2.n2"))]
        return ModelSpec("ToyParallelForCausalLM", V, E, cfg["max_positions"],
                         PartSpec("embedding", {"vocab": V, "width": E}, {"weight": "embed"}), layers,
                         default_schedule(3), norm("final"), PartSpec("head", {"vocab": V, "width": E}, {"weight": "out"}))


PAR = {"architectures": ["ToyParallelForCausalLM"], "width": 128, "head_dim": 64, "heads": 2, "kv_heads": 1,
       "vocab": 211, "inner": 192, "eps": 1e-5, "max_positions": 256}


def _parallel_reference(w, tokens):
    c = PAR
    E, d, nh, nkv = c["width"], c["head_dim"], c["heads"], c["kv_heads"]
    t = len(tokens)
    f = {k: v.float() for k, v in w.items()}
    cos, sin = plain_llama.rope_tables(t, d, 10000.0, None)

    def attn(i, h):
        q = plain_llama.rotate_half_split((h @ f[f"l{i}.q"].T).view(t, nh, d), cos, sin)
        k = plain_llama.rotate_half_split((h @ f[f"l{i}.k"].T).view(t, nkv, d), cos, sin)
        v = (h @ f[f"l{i}.v"].T).view(t, nkv, d)
        return plain_llama.causal_attention(q, k, v, 1.0 / math.sqrt(d)).reshape(t, nh * d) @ f[f"l{i}.o"].T

    def ffn(i, h):
        return plain_llama.swiglu(h, f[f"l{i}.gate"], f[f"l{i}.up"], f[f"l{i}.down"])

    x = f["embed"][torch.tensor(tokens)]
    x = x + attn(0, plain_llama.rms_norm(x, f["l0.n1"], c["eps"]))
    x = x + ffn(0, plain_llama.rms_norm(x, f["l0.n2"], c["eps"]))
    h = plain_llama.rms_norm(x, f["l1.n1"], c["eps"])
    x = x + attn(1, h) + ffn(1, h)
    h = plain_llama.rms_norm(x, f["l2.n1"], c["eps"])
    x = x + (h @ f["l2.w"].T) * x.abs().mean(-1, keepdim=True)
    x = x + ffn(2, plain_llama.rms_norm(x, f["l2.n2"], c["eps"]))
    return plain_llama.rms_norm(x, f["final"], c["eps"]) @ f["out"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_parallel_block_and_a_mixer_that_reads_the_stream(dtype):
    """Other arrangements written against the documented interface only: a parallel-residual block (two
    contractions add into the stream back to back) and a mixer that reads the stream itself. In bfloat16 with up to
    64 rows a contraction into the stream leaves its K slices unadded; the stream object hands them to whoever
    reads next, so these parts see the full sum without knowing about slices."""
    _register_parallel_parts()
    from cuca_b200.config.registry import build_spec
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.step import StepEntry
    from cuca_b200.models.model import Model
    from cuca_b200.weights.loader import RandomSource
    spec = build_spec(PAR)
    needs = Model(spec).tensor_needs()
    assert "l1.n2" not in needs
    source = RandomSource(needs, seed=3, std=0.06, device="cpu", dtype=torch.bfloat16, norm_std=0.2)
    weights = {n: source.read(n) for n in source.shapes()}
    core = EngineCore(spec, source, dtype=dtype, kv_tokens=256, max_sequences=2, block_size=16)
    if dtype == "bfloat16":
        from cuca_b200.kernels import ops
        probe = torch.zeros(8, PAR["width"], dtype=torch.bfloat16, device="cuda:0")
        assert ops.gemm_partial_supported(probe, core.model.blocks[0].mixer.w_o), "the case must leave slices unadded"
    tokens = tiny.random_tokens(60, PAR["vocab"], seed=8)
    ref = _parallel_reference(weights, tokens)
    tol = 3e-5 if dtype == "float32" else 4e-2
    blocks, slot, pos = core.pools.new_seq(), core.slots.alloc(), 0
    for n in (40, 1, 1, 5, 1, 12):
        core.pools.reserve(blocks, pos + n)
        logits = core.stepper.step([StepEntry(blocks, slot, tokens[pos:pos + n], list(range(n)))]).float().cpu()
        want = ref[pos:pos + n]
        err = float((logits - want).abs().max() / want.abs().max())
        assert err < tol, (pos, n, err)
        pos += n
    core.rt.check_device_errors()


# ------------------------------------------------------------------------------------------ built-in parts alone
@pytest.fixture(scope="module")
def rt32():
    from cuca_b200.runtime import Runtime
    return Runtime("cuda:0", torch.float32)


def test_rmsnorm_part_alone(rt32):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.norm import RMSNorm
    part = RMSNorm(PartSpec("rmsnorm", {"width": 50, "eps": 1e-3}, {"weight": "w"}), rt32)
    assert part.tensors()["w"].shape == (50,)
    w = torch.randn(50, device=rt32.device)
    part.load(lambda name: w)
    x = torch.randn(9, 50, device=rt32.device) * 2
    assert torch.allclose(part.forward(x).cpu(), plain_llama.rms_norm(x.cpu(), w.cpu(), 1e-3), atol=1e-5)


def test_rotary_part_tables_and_scalings(rt32):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.rope import RotaryEncoding
    for cfg in (tiny.TINY_A, tiny.TINY_B, tiny.TINY_C):
        d = cfg["head_dim"]
        rs = cfg.get("rope_scaling") or {}
        scaling = {"kind": rs.get("rope_type", "default"), **{k: v for k, v in rs.items() if k != "rope_type"}}
        part = RotaryEncoding(PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": cfg["rope_theta"],
                                                "scaling": scaling}), rt32)
        part.prepare(77)
        cos, sin, rot = part.fused_tables()
        pc, ps = plain_llama.rope_tables(77, d, cfg["rope_theta"], plain_llama.llama3_factors(cfg, d),
                                         plain_llama.linear_freq_scale(cfg))
        assert rot == d and torch.equal(cos.cpu(), pc) and torch.equal(sin.cpu(), ps)
    f = plain_llama.llama3_factors(tiny.TINY_B, 32)
    assert f[0] == 1.0 and f[-1] == 8.0 and any(1.0 < x < 8.0 for x in f)  # all three regimes occur


def test_swiglu_part_alone(rt32):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.mlp import SwiGLU
    part = SwiGLU(PartSpec("swiglu", {"width": 24, "inner": 56}, {"gate": "g", "up": "u", "down": "d"}), rt32)
    ws = {"g": torch.randn(56, 24), "u": torch.randn(56, 24), "d": torch.randn(24, 56)}
    part.load(lambda n: ws[n].to(rt32.device))
    h = torch.randn(7, 24)
    stream = torch.randn(7, 24)
    out = stream.clone().to(rt32.device)
    part.forward(h.to(rt32.device), out, None)
    assert torch.allclose(out.cpu(), stream + plain_llama.swiglu(h, ws["g"], ws["u"], ws["d"]), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("window", [None, 7])
def test_attention_part_alone_whole_and_cut(rt32, window):
    """The attention mixer with a page pool of its own: a whole sequence, then the same sequence in two
    portions; the keys of the second portion's early rows lie in pages written by the first step."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.engine.step import StepBatch
    from cuca_b200.parts.attention import PagedAttention
    from cuca_b200.parts.base import PartSpec
    dev = rt32.device
    E, nh, nkv, d, bs, t = 40, 4, 2, 16, 8, 29
    rope = PartSpec("rope", {"head_dim": d, "rotary_dim": d, "theta": 5000.0, "scaling": {"kind": "default"}})
    part = PagedAttention(PartSpec("attention", {"width": E, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d,
                                                 "window": window, "scale": None, "position": rope},
                                   {"q": "q", "k": "k", "v": "v", "o": "o"}), rt32)
    ws = {"q": torch.randn(nh * d, E) * 0.3, "k": torch.randn(nkv * d, E) * 0.3, "v": torch.randn(nkv * d, E) * 0.3,
          "o": torch.randn(E, nh * d) * 0.3}
    part.load(lambda n: ws[n].to(dev))
    part.prepare(64)
    h = torch.randn(t, E)
    cos, sin = plain_llama.rope_tables(t, d, 5000.0, None)
    q = plain_llama.rotate_half_split((h @ ws["q"].T).view(t, nh, d), cos, sin)
    k = plain_llama.rotate_half_split((h @ ws["k"].T).view(t, nkv, d), cos, sin)
    v = (h @ ws["v"].T).view(t, nkv, d)
    want = plain_llama.causal_attention(q, k, v, 1 / math.sqrt(d), window).reshape(t, nh * d) @ ws["o"].T

    def run(cuts):
        kpool = torch.zeros(6, nkv, bs, d, device=dev)
        vpool = torch.zeros_like(kpool)
        tables = torch.tensor([[-1] * 8, [5, 0, 3, 1, -1, -1, -1, -1]], dtype=torch.int32, device=dev)  # slot 1
        out, pos = [], 0
        for n in cuts:
            positions = torch.arange(pos, pos + n, dtype=torch.int32, device=dev)
            slot_of_row = torch.full((n,), 1, dtype=torch.int32, device=dev)
            step = StepBatch(n, 1, None, positions, slot_of_row, None, None, 0)
            stream = torch.zeros(n, E, device=dev)
            part.forward(h[pos:pos + n].to(dev), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, None))
            out.append(stream.cpu())
            pos += n
        return torch.cat(out)

    assert torch.allclose(run([t]), want, atol=2e-5, rtol=1e-4)
    assert torch.allclose(run([13, 2, 14]), want, atol=2e-5, rtol=1e-4)
    assert int(rt32.err.item()) == 0

"""Plain, slow implementation of the Llama dense decoder, used as the oracle of the tests.

It rests on the formulas of nassor/cuca's local engine (each function cites the
file and lines it restates). The reference is Rust on candle and cannot be
compiled or imported here, so nothing below was checked against its binaries:
the formulas are the anchor. Whole sequences only, no cache, one function per
part, and no code shared with the product path (`cuca_b200`): this file reads
`config.json` as a plain dict and safetensors through its own few lines.

Weights keep Hugging Face row order, so rotary pairs are (i, i + d/2); the
reference permutes q/k rows at conversion and rotates adjacent pairs, which is
the same rotation (src/provider/local/model/cpu.rs:4247-4275).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ----------------------------------------------------------------------------
# reading a model folder (own reader: the product's loader is not imported)
# ----------------------------------------------------------------------------
_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I32": np.int32, "I64": np.int64}


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data
    (src/provider/local/convert/safetensors.rs:1-24)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(raw, dtype=_NP[meta["dtype"]], count=(hi - lo) // np.dtype(_NP[meta["dtype"]]).itemsize,
                            offset=base + lo).reshape(meta["shape"])
        t = torch.from_numpy(arr.copy())
        if meta["dtype"] == "BF16":
            t = t.view(torch.bfloat16)
        out[name] = t
    return out


def load_model_dir(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = read_safetensors(model_dir / "model.safetensors")
    return cfg, weights


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """x[r] = E[token[r]] with scale 1 for Llama
    (src/provider/local/model/cpu.rs:2193-2198, model/quant.rs:391-411)."""
    if int(tokens.max()) >= table.shape[0] or int(tokens.min()) < 0:
        raise ValueError("token id outside the vocabulary")
    return table[tokens.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """h = x * rsqrt(mean(x^2) + eps) * w, the weight multiplies directly
    (src/provider/local/model/cpu.rs:3651-3654, model/gpu.rs:5883-5896)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * weight


def llama3_factors(cfg: dict, head_dim: int) -> list[float] | None:
    """Per-pair divisors of llama3 frequency scaling
    (src/provider/local/convert/config.rs:525-565): the frequency is computed in
    f32, the rest in f64, the factor stored as f32."""
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters")
    if not rs:
        return None
    kind = (rs.get("rope_type") or rs.get("type") or "default").lower()
    if kind == "default":
        return None
    if kind == "linear":
        return None  # handled by linear_freq_scale()
    if kind != "llama3":
        raise ValueError(f"rope scaling `{kind}` is not part of this oracle")
    base = float(rs.get("rope_theta", cfg.get("rope_theta", 10000.0)))
    factor = float(rs.get("factor", 8.0))
    low = float(rs.get("low_freq_factor", 1.0))
    high = float(rs.get("high_freq_factor", 4.0))
    old = float(rs.get("original_max_position_embeddings", 8192.0))
    out = []
    for i in range(head_dim // 2):
        freq = np.float32(1.0) / np.power(np.float32(base), np.float32(2 * i) / np.float32(head_dim), dtype=np.float32)
        wavelen = 2.0 * math.pi / float(freq)
        if wavelen < old / high:
            r = 1.0
        elif wavelen > old / low:
            r = factor
        else:
            smooth = (old / wavelen - low) / (high - low)
            r = 1.0 / ((1.0 - smooth) / factor + smooth)
        out.append(float(np.float32(r)))
    return out


def linear_freq_scale(cfg: dict) -> float:
    """`linear` scaling multiplies every angle by 1/factor
    (src/provider/local/model/params.rs:535-572, model/rope.rs:118-130)."""
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or {}
    kind = (rs.get("rope_type") or rs.get("type") or "default").lower()
    return 1.0 / float(rs.get("factor", 1.0)) if kind == "linear" else 1.0


def rope_tables(positions: int, n_dims: int, base: float, factors, freq_scale: float = 1.0):
    """theta = freq_scale * pos * base^(-2i/n_dims) / factor_i in f64, stored as f32
    (src/provider/local/model/rope.rs:118-152)."""
    half = n_dims // 2
    cos = torch.empty(positions, half, dtype=torch.float32)
    sin = torch.empty(positions, half, dtype=torch.float32)
    for i in range(half):
        f = 1.0 if factors is None else float(factors[i])
        inv = base ** (-(2 * i) / n_dims) / f
        for p in range(positions):
            theta = freq_scale * (p * inv)
            cos[p, i] = math.cos(theta)
            sin[p, i] = math.sin(theta)
    return cos, sin


def rotate_half_split(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [t, heads, d]; pair i is (i, i + half): out_a = a cos - b sin,
    out_b = a sin + b cos (src/provider/local/model/rope.rs:158-169, kind Neox
    on Hugging Face row order = kind Norm on the reference's permuted rows)."""
    half = cos.shape[-1]
    a, b = x[..., :half], x[..., half : 2 * half]
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    out[..., :half] = a * c - b * s
    out[..., half : 2 * half] = a * s + b * c
    return out


def causal_attention(q, k, v, scale: float, window: int | None = None) -> torch.Tensor:
    """q: [t, nh, d], k, v: [t, nkv, d] (whole sequence from position 0).
    Query at position P sees keys lo..P, lo = max(0, P - (window-1)); scores are
    scaled before the mask; head h reads KV head h // (nh/nkv)
    (src/provider/local/model/cpu.rs:3699-3728, model/mod.rs:356-383)."""
    t, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    out = torch.empty_like(q)
    pos = torch.arange(t)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(nh):
        kv = h // group
        s = (q[:, h, :] @ k[:, kv, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kv, :]
    return out


def swiglu(x, w_gate, w_up, w_down) -> torch.Tensor:
    """down(silu(gate x) * up x) (src/provider/local/model/cpu.rs:3554-3565)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (torch.nn.functional.silu(g) * u) @ w_down.T


# ----------------------------------------------------------------------------
# the whole model
# ----------------------------------------------------------------------------
def _get(weights, name, dtype):
    return weights[name].to(dtype)


def forward(cfg: dict, weights: dict[str, torch.Tensor], tokens, dtype=torch.float32) -> torch.Tensor:
    """Logits [t, vocab] of one whole sequence from position 0
    (order of operations: src/provider/local/model/cpu.rs:2650-2704, 2495-2583)."""
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    E = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    d = cfg.get("head_dim") or E // nh
    eps = float(cfg["rms_norm_eps"])
    base = float(cfg.get("rope_theta", 10000.0))
    t = tokens.shape[0]
    cos, sin = rope_tables(t, d, base, llama3_factors(cfg, d), linear_freq_scale(cfg))
    cos, sin = cos.to(dtype), sin.to(dtype)
    scale = 1.0 / math.sqrt(d)

    x = embed(_get(weights, "model.embed_tokens.weight", dtype), tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rms_norm(x, _get(weights, p + "input_layernorm.weight", dtype), eps)
        q = h @ _get(weights, p + "self_attn.q_proj.weight", dtype).T
        k = h @ _get(weights, p + "self_attn.k_proj.weight", dtype).T
        v = h @ _get(weights, p + "self_attn.v_proj.weight", dtype).T
        if p + "self_attn.q_proj.bias" in weights:
            q = q + _get(weights, p + "self_attn.q_proj.bias", dtype)
            k = k + _get(weights, p + "self_attn.k_proj.bias", dtype)
            v = v + _get(weights, p + "self_attn.v_proj.bias", dtype)
        q = rotate_half_split(q.view(t, nh, d), cos, sin)
        k = rotate_half_split(k.view(t, nkv, d), cos, sin)
        a = causal_attention(q, k, v.view(t, nkv, d), scale).reshape(t, nh * d)
        a = a @ _get(weights, p + "self_attn.o_proj.weight", dtype).T
        if p + "self_attn.o_proj.bias" in weights:
            a = a + _get(weights, p + "self_attn.o_proj.bias", dtype)
        x = x + a
        f = rms_norm(x, _get(weights, p + "post_attention_layernorm.weight", dtype), eps)
        x = x + swiglu(f, _get(weights, p + "mlp.gate_proj.weight", dtype),
                       _get(weights, p + "mlp.up_proj.weight", dtype),
                       _get(weights, p + "mlp.down_proj.weight", dtype))
    n = rms_norm(x, _get(weights, "model.norm.weight", dtype), eps)
    head = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in weights \
        else "lm_head.weight"
    return n @ _get(weights, head, dtype).T


# ----------------------------------------------------------------------------
# sampling (src/provider/local/sampler.rs)
# ----------------------------------------------------------------------------
_M64 = (1 << 64) - 1


class SplitMix64:
    """src/provider/local/sampler.rs:18-34."""

    def __init__(self, seed: int):
        self.state = seed & _M64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        return float(np.float32(self.next_u64() >> 40) / np.float32(16777216.0))


def greedy(logits) -> int:
    """First maximum wins (src/provider/local/sampler.rs:44-54)."""
    best, best_v = 0, -math.inf
    for i, v in enumerate(np.asarray(logits, dtype=np.float32)):
        if v > best_v:
            best, best_v = i, float(v)
    return best


def sample(logits, temperature: float, top_k: int, top_p: float, rng: SplitMix64) -> int:
    """temperature -> top-k by (logit desc, id asc) -> softmax -> top-p prefix ->
    draw with target = u * total, first acc > target
    (src/provider/local/sampler.rs:159-331). All arithmetic in f32."""
    logits = np.asarray(logits, dtype=np.float32)
    if temperature <= 0.0 or logits.shape[0] <= 1:
        return greedy(logits)
    f32 = np.float32
    scaled = (logits / f32(temperature)).astype(np.float32)
    ids = [i for i in range(len(scaled)) if np.isfinite(scaled[i])]
    if not ids:
        return greedy(logits)
    ranked = top_k > 0 and top_k < len(scaled)
    if ranked or top_p < 1.0:
        ids.sort(key=lambda i: (-float(scaled[i]), i))
    if ranked:
        ids = ids[:top_k]
    mx = max(scaled[i] for i in ids)
    probs = [np.exp(scaled[i] - mx, dtype=np.float32) for i in ids]
    total = f32(0.0)
    for p in probs:
        total = f32(total + p)
    probs = [f32(p / total) for p in probs]
    cand = [(p, i) for p, i in zip(probs, ids) if p > 0.0]
    if not cand:
        return greedy(logits)
    if ranked or top_p < 1.0:
        cum, keep = f32(0.0), len(cand)
        for j, (p, _) in enumerate(cand):
            cum = f32(cum + p)
            if cum >= f32(top_p):
                keep = j + 1
                break
        cand = cand[:keep]
    total = f32(0.0)
    for p, _ in cand:
        total = f32(total + p)
    target = f32(f32(rng.next_f32()) * total)
    acc = f32(0.0)
    for p, i in cand:
        acc = f32(acc + p)
        if target < acc:
            return i
    return cand[-1][1]


def generate_greedy(cfg, weights, prompt, n_tokens: int, dtype=torch.float32) -> list[int]:
    """Greedy continuation by re-running the whole sequence for each token."""
    ids = list(prompt)
    out = []
    for _ in range(n_tokens):
        logits = forward(cfg, weights, ids, dtype)[-1]
        nxt = greedy(logits.float().numpy())
        out.append(nxt)
        ids.append(nxt)
    return out

"""A second plain implementation of the Llama decoder, written another way than `plain_llama.py`, so that the
two can be checked against each other (the reference anchors its own numerics by computing every model twice:
src/provider/local/convert/oracle.rs:1-12, convert/oracle_local.rs:1-14; its Rust cannot be compiled here, and
model code of installed packages is not a source for this build, so the second computation is this file).

Where `plain_llama.py` keeps Hugging Face row order, whole-sequence matrices and masks in 32-bit torch, this file
follows the reference's own route in 64-bit numpy:

* conversion first: Q/K rows (and biases) are permuted from the half-split layout to adjacent pairs, row
  `j * half + i -> 2 i + j` per head (src/provider/local/convert/tensors.rs:250-271);
* then one token at a time against a growing list of keys and values, the way decoding runs
  (src/provider/local/model/cpu.rs:2822-2991): no mask exists, a token simply sees what has been appended;
* rotation of adjacent pairs `(2i, 2i + 1)` (`RopeKind::Norm`, src/provider/local/model/rope.rs:158-169) with the
  angle `pos * base^(-2i/n) / factor_i * freq_scale` (rope.rs:118-130);
* per-head loops and a hand-written softmax.

It shares no code with `plain_llama.py` or with the product.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


def read_folder(model_dir):
    """config.json as a dict; tensors as float64 arrays (bf16 widened by hand)."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    raw = (model_dir / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        blob = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            bits = np.frombuffer(blob, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(blob, dtype="<f4")
        elif meta["dtype"] == "F16":
            arr = np.frombuffer(blob, dtype="<f2")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        tensors[name] = arr.astype(np.float64).reshape(meta["shape"])
    return cfg, tensors


def permute_rows(w: np.ndarray, n_head: int) -> np.ndarray:
    """`LlamaModel.permute` as the reference applies it (convert/tensors.rs:250-271)."""
    rows = w.shape[0]
    per_head = rows // n_head
    half = per_head // 2
    out = np.empty_like(w)
    for h in range(n_head):
        for i in range(half):
            for j in range(2):
                out[h * per_head + 2 * i + j] = w[h * per_head + j * half + i]
    return out


def pair_divisors(cfg: dict, n_dims: int):
    """llama3 divisors (convert/config.rs:525-565): frequency in 32-bit, the rest in 64-bit, stored 32-bit."""
    rs = cfg.get("rope_scaling") or {}
    kind = str(rs.get("rope_type") or rs.get("type") or "default").lower()
    if kind != "llama3":
        return [1.0] * (n_dims // 2), (1.0 / float(rs["factor"]) if kind == "linear" else 1.0)
    base = np.float32(cfg.get("rope_theta", 10000.0))
    factor, low, high = float(rs.get("factor", 8.0)), float(rs.get("low_freq_factor", 1.0)), \
        float(rs.get("high_freq_factor", 4.0))
    original = float(rs.get("original_max_position_embeddings", 8192))
    out = []
    for i in range(n_dims // 2):
        exponent = np.float32(np.float32(2 * i) / np.float32(n_dims))
        freq = np.float32(1.0) / np.float32(np.power(base, exponent))
        wavelength = 2.0 * math.pi / float(freq)
        if wavelength < original / high:
            div = 1.0
        elif wavelength > original / low:
            div = factor
        else:
            smooth = (original / wavelength - low) / (high - low)
            div = 1.0 / ((1.0 - smooth) / factor + smooth)
        out.append(float(np.float32(div)))
    return out, 1.0


def logits_token_by_token(cfg: dict, t: dict, tokens) -> np.ndarray:
    """[len(tokens), vocab] in 64-bit, one token at a time."""
    E, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    d = cfg.get("head_dim") or E // nh
    L, eps = cfg["num_hidden_layers"], float(cfg["rms_norm_eps"])
    base = float(cfg.get("rope_theta", 10000.0))
    divisors, freq_scale = pair_divisors(cfg, d)
    group = nh // nkv

    layers = []
    for i in range(L):
        p = f"model.layers.{i}."
        layer = {
            "attn_norm": t[p + "input_layernorm.weight"], "ffn_norm": t[p + "post_attention_layernorm.weight"],
            "wq": permute_rows(t[p + "self_attn.q_proj.weight"], nh),
            "wk": permute_rows(t[p + "self_attn.k_proj.weight"], nkv),
            "wv": t[p + "self_attn.v_proj.weight"], "wo": t[p + "self_attn.o_proj.weight"],
            "gate": t[p + "mlp.gate_proj.weight"], "up": t[p + "mlp.up_proj.weight"], "down": t[p + "mlp.down_proj.weight"],
            "keys": [], "values": [],
        }
        if p + "self_attn.q_proj.bias" in t:
            layer["bq"] = permute_rows(t[p + "self_attn.q_proj.bias"][:, None], nh)[:, 0]
            layer["bk"] = permute_rows(t[p + "self_attn.k_proj.bias"][:, None], nkv)[:, 0]
            layer["bv"] = t[p + "self_attn.v_proj.bias"]
        if p + "self_attn.o_proj.bias" in t:
            layer["bo"] = t[p + "self_attn.o_proj.bias"]
        layers.append(layer)
    tied = cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in t
    head = t["model.embed_tokens.weight"] if tied else t["lm_head.weight"]

    def norm(x, w):
        return x / math.sqrt(float(np.dot(x, x)) / x.shape[0] + eps) * w

    def rotate(vec, pos):
        out = vec.copy()
        for i in range(d // 2):
            theta = freq_scale * (pos * base ** (-(2 * i) / d) / divisors[i])
            c, s = math.cos(theta), math.sin(theta)
            a, b = vec[2 * i], vec[2 * i + 1]
            out[2 * i], out[2 * i + 1] = a * c - b * s, a * s + b * c
        return out

    rows = []
    for pos, tok in enumerate(tokens):
        x = t["model.embed_tokens.weight"][tok].copy()
        for layer in layers:
            h = norm(x, layer["attn_norm"])
            q, k, v = layer["wq"] @ h, layer["wk"] @ h, layer["wv"] @ h
            if "bq" in layer:
                q, k, v = q + layer["bq"], k + layer["bk"], v + layer["bv"]
            layer["keys"].append([rotate(k[g * d:(g + 1) * d], pos) for g in range(nkv)])
            layer["values"].append([v[g * d:(g + 1) * d] for g in range(nkv)])
            attn = np.empty(nh * d)
            for hd in range(nh):
                qh = rotate(q[hd * d:(hd + 1) * d], pos)
                g = hd // group
                scores = [float(np.dot(qh, past[g])) / math.sqrt(d) for past in layer["keys"]]
                top = max(scores)
                weights = [math.exp(s - top) for s in scores]
                total = sum(weights)
                acc = np.zeros(d)
                for w_, past in zip(weights, layer["values"]):
                    acc += (w_ / total) * past[g]
                attn[hd * d:(hd + 1) * d] = acc
            o = layer["wo"] @ attn
            if "bo" in layer:
                o = o + layer["bo"]
            x = x + o
            f = norm(x, layer["ffn_norm"])
            gate, up = layer["gate"] @ f, layer["up"] @ f
            x = x + layer["down"] @ (gate / (1.0 + np.exp(-gate)) * up)
        rows.append(head @ norm(x, t["model.norm.weight"]))
    return np.stack(rows)

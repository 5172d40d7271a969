"""Weights made so that a lost key shows: random weights give nearly flat attention, under which one missing
page moves the logits by less than a bfloat16 tolerance."""
from __future__ import annotations

import torch

import plain_llama


def plant_far_key(folder, last: int, far: int, key_token: int, query_token: int, qk_scale: float = 8.0) -> None:
    """Rewrites the model folder: layer 0's query and key projections are scaled so that scores are sharp, and
    the embedding row of `query_token` is built so that, at position `last`, its query (head 0) points at the
    key that `key_token` leaves at position `far`. A sequence with `key_token` at `far` and `query_token` at
    `last` then has last-position logits that hang on that one far key."""
    from cuca_b200.weights import safetensors_io as st
    cfg, w = plain_llama.load_model_dir(folder)
    pre = "model.layers.0.self_attn."
    for name, scale in (("q_proj", qk_scale), ("k_proj", qk_scale), ("v_proj", 4.0), ("o_proj", 4.0)):
        w[pre + name + ".weight"] = (w[pre + name + ".weight"].float() * scale).to(torch.bfloat16)
    dh = cfg["head_dim"]
    pos = torch.tensor([far, last])
    cos, sin = tables_at(cfg, dh, pos)
    E = w["model.embed_tokens.weight"].float()
    wq, wk = w[pre + "q_proj.weight"].float()[:dh], w[pre + "k_proj.weight"].float()[:dh]
    norm_w = w["model.layers.0.input_layernorm.weight"].float()
    n_key = plain_llama.rms_norm(E[key_token:key_token + 1], norm_w, cfg["rms_norm_eps"])
    k_far = plain_llama.rotate_half_split((n_key @ wk.T).view(1, 1, dh), cos[0:1], sin[0:1])
    target = plain_llama.rotate_half_split(k_far, cos[1:2], -sin[1:2])[0, 0]  # rotated back from position `last`
    n_query = torch.linalg.pinv(wq) @ target  # the normed input whose query is `target`
    row = n_query / norm_w  # undo the norm's weight; its scale is free (the norm divides it out)
    E[query_token] = row / row.norm() * E[key_token].norm()
    w["model.embed_tokens.weight"] = E.to(torch.bfloat16)
    st.write_safetensors(folder / "model.safetensors", w)


def tables_at(cfg, dh, positions):
    """cos/sin rows of the plain implementation at a few positions (its table builder walks every position)."""
    import math
    factors = plain_llama.llama3_factors(cfg, dh)
    scale = plain_llama.linear_freq_scale(cfg)
    base = float(cfg.get("rope_theta", 10000.0))
    cos = torch.empty(len(positions), dh // 2)
    sin = torch.empty(len(positions), dh // 2)
    for r, p in enumerate(positions.tolist()):
        for i in range(dh // 2):
            f = 1.0 if factors is None else float(factors[i])
            theta = scale * (p * (base ** (-(2 * i) / dh) / f))
            cos[r, i], sin[r, i] = math.cos(theta), math.sin(theta)
    return cos, sin

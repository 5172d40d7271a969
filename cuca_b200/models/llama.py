"""The Llama dense decoder as a `ModelSpec`: RMSNorm, rotary positions with
optional llama3 / linear scaling, grouped-query attention, SwiGLU, optionally
tied embeddings (the `DEFAULT` behaviour row of src/provider/local/model/arch.rs:
283-319; `MistralForCausalLM` is the same class there, convert/arch.rs:71-73).
Tensor names are the Hugging Face ones the reference's converter maps from
(src/provider/local/convert/tensors.rs:819-833,990-1014)."""
from __future__ import annotations

import re

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, default_schedule

_IGNORABLE = re.compile(r".*rotary_emb\.inv_freq$")


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    E, d = cfg.hidden_size, cfg.head_dim
    s = cfg.rope_scaling
    position = PartSpec("rope", {
        "head_dim": d, "rotary_dim": d, "theta": cfg.rope_theta,
        "scaling": {"kind": s.kind, "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                    "high_freq_factor": s.high_freq_factor,
                    "original_max_position_embeddings": s.original_max_position_embeddings}})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        names = {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                 "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}
        if cfg.attention_bias:
            names.update({"q_bias": p + "self_attn.q_proj.bias", "k_bias": p + "self_attn.k_proj.bias",
                          "v_bias": p + "self_attn.v_proj.bias", "o_bias": p + "self_attn.o_proj.bias"})
        layers.append(LayerSpec(
            block=PartSpec("pre_norm"),
            mixer=PartSpec("attention", {"width": E, "n_heads": cfg.num_attention_heads,
                                         "n_kv_heads": cfg.num_key_value_heads, "head_dim": d, "window": None,
                                         "scale": None, "position": position}, names),
            mixer_norm=PartSpec("rmsnorm", {"width": E, "eps": cfg.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            feed_forward=PartSpec("swiglu", {"width": E, "inner": cfg.intermediate_size},
                                  {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                                   "down": p + "mlp.down_proj.weight"}),
            ffn_norm=PartSpec("rmsnorm", {"width": E, "eps": cfg.rms_norm_eps},
                              {"weight": p + "post_attention_layernorm.weight"}),
        ))
    embed_name = "model.embed_tokens.weight"
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    tied = cfg.tie_word_embeddings

    def ignorable(name: str) -> bool:
        # a tied checkpoint may still carry lm_head.weight; the reference skips it
        # (src/provider/local/convert/tensors.rs:828-833) as it skips inv_freq (:614)
        return bool(_IGNORABLE.match(name)) or (tied and name == "lm_head.weight")

    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, width=E,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab_size, "width": E}, {"weight": embed_name}),
        layers=layers, schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"width": E, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("head", {"vocab": cfg.vocab_size, "width": E}, {"weight": head_name}),
        eos_token_ids=cfg.eos_token_ids, ignorable_tensor=ignorable)


@register_architecture("LlamaForCausalLM", "MistralForCausalLM")
def build_llama(config_json: dict) -> ModelSpec:
    return llama_spec(LlamaConfig.from_json(config_json))

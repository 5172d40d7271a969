"""Configuration: config.json keys, defaults, range checks, the architecture registry."""
import copy

import pytest

import tiny
from cuca_b200.config.model_config import ConfigError, LlamaConfig, RopeScaling
from cuca_b200.config.registry import architectures, build_spec


def test_reads_every_key_of_both_tiny_configs():
    a = LlamaConfig.from_json(tiny.TINY_A)
    b = LlamaConfig.from_json(tiny.TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.max_position_embeddings) == (2, 64, 4, 2, 16, 176, 256, 128)
    assert a.rms_norm_eps == 1e-5 and a.rope_theta == 10000.0 and a.rope_scaling.kind == "default"
    assert not a.tie_word_embeddings
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size) == (3, 96, 3, 1, 32, 320, 512)
    assert b.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64) and b.tie_word_embeddings


def test_defaults_follow_the_reference():
    cfg = {k: v for k, v in tiny.TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta",
                                                            "rms_norm_eps", "rope_scaling")}
    c = LlamaConfig.from_json(cfg)
    assert c.num_key_value_heads == c.num_attention_heads
    assert c.head_dim == c.hidden_size // c.num_attention_heads
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    llama3 = RopeScaling.from_json({"rope_type": "llama3"})
    assert (llama3.factor, llama3.low_freq_factor, llama3.high_freq_factor,
            llama3.original_max_position_embeddings) == (8.0, 1.0, 4.0, 8192)


def test_round_trip_through_config_json():
    for cfg in (tiny.TINY_A, tiny.TINY_B, tiny.TINY_C):
        c = LlamaConfig.from_json(cfg)
        assert LlamaConfig.from_json(c.to_json()) == c


@pytest.mark.parametrize("key,value,word", [
    ("num_key_value_heads", 3, "divide"), ("head_dim", 15, "even"), ("num_hidden_layers", 0, "positive"),
    ("rms_norm_eps", 0.0, "positive"), ("rope_scaling", {"rope_type": "yarn9"}, "yarn9"),
    ("mlp_bias", True, "mlp_bias"), ("hidden_size", "wide", "hidden_size"),
    ("hidden_act", "gelu", "SiLU"), ("hidden_activation", "gelu_pytorch_tanh", "SiLU"),
])
def test_bad_values_are_refused(key, value, word):
    cfg = copy.deepcopy(tiny.TINY_A)
    cfg[key] = value
    with pytest.raises(ConfigError, match=word):
        LlamaConfig.from_json(cfg)


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size",
                                 "vocab_size", "max_position_embeddings", "architectures"])
def test_missing_keys_are_named(key):
    cfg = {k: v for k, v in tiny.TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        build_spec(cfg)


def test_registry_names_and_unknown_architecture():
    assert {"LlamaForCausalLM", "MistralForCausalLM"} <= set(architectures())
    cfg = dict(tiny.TINY_A, architectures=["GptOssForCausalLM"])
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        build_spec(cfg)


def test_spec_is_data_chosen_layer_by_layer():
    spec = build_spec(tiny.TINY_B)
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "attention" and m.params["n_heads"] == 3 and m.params["n_kv_heads"] == 1
    assert m.params["position"].params["scaling"]["kind"] == "llama3"
    assert spec.layers[2].feed_forward.params == {"width": 96, "inner": 320}
    assert spec.head.tensors["weight"] == spec.embedding.tensors["weight"]  # tied
    assert build_spec(tiny.TINY_A).head.tensors["weight"] == "lm_head.weight"

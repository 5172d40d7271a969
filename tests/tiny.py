"""Two tiny Llama configurations that differ in every size and option, and helpers to write them."""
from __future__ import annotations

import numpy as np
import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 176, "vocab_size": 256, "max_position_embeddings": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 512, "max_position_embeddings": 256,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": True,
}
# a third shape for odd sizes: head size 48 (a multiple of 16, no power of two), 6/3 heads, odd vocabulary
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 331, "max_position_embeddings": 512,
    "rms_norm_eps": 3e-5, "rope_theta": 25000.0, "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "tie_word_embeddings": False, "attention_bias": True,
}
# two small shapes at the head sizes of real models, so that in bfloat16 the replays run the serving kernels
# (tensor-core attention over prompt portions, TMA-fed decode attention, contractions over more than 64 tokens):
# head size 128 with two query heads per key/value head, head size 64 with three
SMALL_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 384, "vocab_size": 1000, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "tie_word_embeddings": False,
}
SMALL_E = {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 456, "vocab_size": 777, "max_position_embeddings": 1024,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True,
}
SEEDS = {"A": 0, "B": 2, "C": 9, "D": 4, "E": 11}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": SMALL_D, "E": SMALL_E}


def write_tiny(folder, which: str, dtype=torch.bfloat16, std: float = 0.02, norm_std: float = 0.2):
    """Norm weights are 1 + N(0, 0.2), different in every layer: with all of them 1.0 a swapped, dropped or
    wrongly bound norm weight would change nothing."""
    from cuca_b200.weights.random_init import write_random_model
    return write_random_model(folder, CONFIGS[which], SEEDS[which], std=std, dtype=dtype, norm_std=norm_std)


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()

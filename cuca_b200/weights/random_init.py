"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed."""
from __future__ import annotations

from pathlib import Path

import torch

from ..config.registry import build_spec
from ..models.model import Model
from .loader import write_model_folder


def write_random_model(folder, config_json: dict, seed: int, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16, norm_std: float = 0.0, device="cpu") -> Path:
    """Every weight N(0, std) from (seed, tensor name, element), norm weights 1.0 (or 1 + N(0, norm_std)),
    stored as `dtype`.

    The architecture named in `config_json` decides which tensors exist; nothing
    but the registry is consulted, so a newly registered architecture gets its
    random folders for free.
    """
    spec = build_spec(config_json)
    needs = Model(spec, runtime=None).tensor_needs()
    return write_model_folder(folder, config_json, needs, seed, std, dtype, norm_std, device)

"""Putting model, cache and step function together for one device."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

from ..cache.device import DeviceCache, plan_groups
from ..cache.pages import KvPools, StateSlots
from ..config.model_config import read_config_json
from ..config.registry import build_spec
from ..models.model import Model
from ..runtime import Runtime
from ..weights.loader import FolderSource, RandomSource, WeightSource
from .step import Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype `{name}` is unknown; use bfloat16 or float32") from None


class EngineCore:
    """Model + page pools + device cache + step function.

    `kv_tokens` positions of cache are shared by all live requests (rounded up to
    whole pages); `context_length` bounds one request and sizes the position tables.
    """

    def __init__(self, spec, source: Optional[WeightSource], dtype=torch.bfloat16, device="cuda:0",
                 context_length: Optional[int] = None, kv_tokens: Optional[int] = None, max_sequences: int = 4,
                 block_size: int = 16, max_step_tokens: Optional[int] = None, window_pools: str = "sized",
                 random_seed: Optional[int] = None, random_std: float = 0.02):
        self.spec = spec
        self.rt = Runtime(device, parse_dtype(dtype))
        self.model = Model(spec, self.rt)
        if source is None:
            if random_seed is None:
                raise ValueError("neither a weight source nor a seed for random weights was given")
            source = RandomSource(self.model.tensor_needs(), random_seed, random_std, device=self.rt.device,
                                  dtype=torch.bfloat16)
        self.model.load(source)
        self.context_length = min(context_length or spec.max_positions, spec.max_positions)
        if context_length is not None and context_length > spec.max_positions:
            # the reference refuses a context above the model's maximum (src/provider/local/model/mod.rs:475-483)
            raise ValueError(f"context length {context_length} exceeds the model's maximum {spec.max_positions}")
        self.model.prepare(self.context_length)
        self.block_size = block_size
        self.max_sequences = max_sequences
        kv_tokens = kv_tokens or self.context_length
        self.max_step_tokens = max_step_tokens or max(max_sequences, 256)
        needs = self.model.cache_needs()
        self.groups = plan_groups(needs, kv_tokens, block_size, max_sequences, self.max_step_tokens, window_pools)
        self.pools = KvPools(self.groups, block_size)
        self.pools.stateful = any(n.state is not None for n in needs.values())
        self.slots = StateSlots(max_sequences)
        self.cache = DeviceCache(self.rt, self.groups, block_size, needs, max_sequences, self.context_length)
        self.stepper = Stepper(self.model, self.pools, self.cache, self.context_length)

    @classmethod
    def from_folder(cls, model_dir, **kw) -> "EngineCore":
        model_dir = Path(model_dir)
        spec = build_spec(read_config_json(model_dir))
        return cls(spec, FolderSource(model_dir), **kw)

    @classmethod
    def from_config(cls, config_json: dict, seed: int, **kw) -> "EngineCore":
        """Random weights drawn on the device (nothing is written to disk)."""
        return cls(build_spec(config_json), None, random_seed=seed, **kw)

    def kv_tokens(self) -> int:
        return min(g.n_blocks for g in self.groups) * self.block_size if self.groups else 0

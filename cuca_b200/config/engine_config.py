"""Engine configuration with the reference's field names and rules.

`LocalModelConfig` mirrors the subset of the reference's struct that an engine
on one GPU needs (src/provider/local/mod.rs:1762-1915): `source`,
`context_length`, `sampling` (`SamplingConfig`, :1018-1039) and `batching`
(`BatchingConfig`, :2234-2277), validated as there (:2587-2608,2741-2757).
Ours: `dtype`, `kv_block_size` and `random_weights`.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional


class EngineConfigError(ValueError):
    pass


@dataclass
class SamplingConfig:
    """None means: take the checkpoint's generation_config.json, else the built-in default."""

    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: Optional[int] = None
    suppress_tokens: Optional[list] = None  # token ids that are never sampled (the reference takes them from the
    # tokenizer's metadata; here: this list, else generation_config.json's `suppress_tokens`)

    DEFAULT_TEMPERATURE = 1.0
    DEFAULT_TOP_K = 64
    DEFAULT_TOP_P = 0.95


@dataclass
class BatchingConfig:
    max_sequences: int = 4  # 1..=64
    kv_tokens: Optional[int] = None  # positions in the shared page pool; default context + min(context, 4096)
    max_step_tokens: Optional[int] = None  # rows of one step; default the prefill chunk of the context
    prefix_cache: bool = False  # requests reuse the cached pages of a prompt prefix they share with earlier ones
    prefill_chunk: Optional[int] = None  # ours: most tokens of one prompt per step; default: the reference's
    # clamp(2^21 / context, 16, 256), or max_step_tokens when that is given (a B200 takes a 2048-token portion whole)


@dataclass
class RandomWeights:
    seed: int = 0
    std: float = 0.02


@dataclass
class LocalModelConfig:
    source: Optional[str] = None  # a model folder (config.json + safetensors)
    context_length: Optional[int] = None  # default min(8192, the model's maximum)
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    batching: BatchingConfig = field(default_factory=BatchingConfig)
    dtype: str = "bfloat16"
    kv_block_size: int = 16
    random_weights: Optional[RandomWeights] = None  # with `model_config`: weights drawn on the device
    model_config: Optional[dict] = None  # a config.json given inline (random weights only)
    device: str = "cuda:0"

    def validate(self) -> None:
        b, s = self.batching, self.sampling
        if self.context_length is not None and self.context_length < 1:
            raise EngineConfigError("context_length must be at least 1")
        if not 1 <= b.max_sequences <= 64:
            raise EngineConfigError(f"batching.max_sequences must lie in 1..=64, found {b.max_sequences}")
        if b.max_step_tokens is not None and not b.max_sequences <= b.max_step_tokens <= 8192:
            raise EngineConfigError(
                f"batching.max_step_tokens must lie in max_sequences..=8192, found {b.max_step_tokens}")
        if s.temperature is not None and not (s.temperature >= 0.0 and s.temperature == s.temperature
                                              and s.temperature != float("inf")):
            raise EngineConfigError("sampling.temperature must be a finite number >= 0")
        if s.top_p is not None and not 0.0 < s.top_p <= 1.0:
            raise EngineConfigError("sampling.top_p must lie in (0, 1]")
        if s.top_k is not None and s.top_k < 0:
            raise EngineConfigError("sampling.top_k must be >= 0 (0 disables it)")
        if self.dtype not in ("bfloat16", "float32"):
            raise EngineConfigError(f"dtype must be bfloat16 or float32, found {self.dtype}")
        if self.kv_block_size < 1 or self.kv_block_size & (self.kv_block_size - 1):
            raise EngineConfigError("kv_block_size must be a power of two")
        if (self.source is None) == (self.model_config is None):
            raise EngineConfigError("give either `source` (a model folder) or `model_config` with `random_weights`")
        if self.model_config is not None and self.random_weights is None:
            raise EngineConfigError("`model_config` without a folder needs `random_weights`")

    def resolve(self, model_max_positions: int) -> dict:
        """Derived sizes (src/provider/local/mod.rs:293-299, model/mod.rs:387-389, engine/mod.rs:998-1060)."""
        ctx = self.context_length or min(8192, model_max_positions)
        if ctx > model_max_positions:
            raise EngineConfigError(f"context_length {ctx} exceeds the model's maximum {model_max_positions}")
        chunk = max(16, min(256, (1 << 21) // ctx))
        b = self.batching
        step = b.max_step_tokens or max(chunk, b.max_sequences)
        if b.kv_tokens is None:
            kv = ctx + min(ctx, 4096)
        else:
            if b.kv_tokens < ctx + 16:
                raise EngineConfigError(f"batching.kv_tokens must be at least context_length + 16 = {ctx + 16}")
            kv = b.kv_tokens
        bs = self.kv_block_size
        kv = -(-kv // bs) * bs
        if b.prefill_chunk is not None:
            if b.prefill_chunk < 1:
                raise EngineConfigError("batching.prefill_chunk must be at least 1")
            chunk = b.prefill_chunk
        elif b.max_step_tokens is not None:
            chunk = step
        return {"context_length": ctx, "prefill_chunk": min(chunk, step), "max_step_tokens": step, "kv_tokens": kv}

    @staticmethod
    def from_json(obj: dict) -> "LocalModelConfig":
        """Unknown keys are an error, as the reference's `deny_unknown_fields`."""
        def take(cls, d, where):
            known = cls.__dataclass_fields__
            bad = [k for k in d if k not in known]
            if bad:
                raise EngineConfigError(f"unknown key(s) in {where}: {', '.join(bad)}")
            return d
        d = dict(take(LocalModelConfig, obj, "the engine configuration"))
        if isinstance(d.get("sampling"), dict):
            d["sampling"] = SamplingConfig(**take(SamplingConfig, d["sampling"], "sampling"))
        if isinstance(d.get("batching"), dict):
            d["batching"] = BatchingConfig(**take(BatchingConfig, d["batching"], "batching"))
        if isinstance(d.get("random_weights"), dict):
            d["random_weights"] = RandomWeights(**take(RandomWeights, d["random_weights"], "random_weights"))
        return LocalModelConfig(**d)

    @staticmethod
    def from_file(path) -> "LocalModelConfig":
        return LocalModelConfig.from_json(json.loads(Path(path).read_text()))

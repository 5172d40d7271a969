"""Typed model configuration read from a checkpoint's own `config.json` keys.

Key names, defaults and range checks follow the reference's converter and
hyper-parameter reader (src/provider/local/convert/config.rs:106-134,328-448,
520-565; src/provider/local/model/params.rs:417-857): `num_key_value_heads`
defaults to `num_attention_heads` and must divide it, `head_dim` defaults to
`hidden_size / num_attention_heads` and must be even, `rope_theta` defaults to
10000, `rms_norm_eps` to 1e-6, rope scaling knows `default`, `llama3` and
`linear`. No size stands in code: everything a part needs comes from here.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or is out of range."""


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` / `rope_parameters` of config.json."""

    kind: str = "default"  # default | llama3 | linear
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_json(obj: Optional[dict], where: str = "rope_scaling") -> "RopeScaling":
        if not obj:
            return RopeScaling()
        if not isinstance(obj, dict):
            raise ConfigError(f"config.json `{where}` must be an object, found {type(obj).__name__}")
        kind = str(obj.get("rope_type") or obj.get("type") or "default").lower()
        if kind == "default":
            return RopeScaling()
        if kind == "llama3":
            # defaults of src/provider/local/convert/config.rs:540-544
            return RopeScaling(
                kind="llama3",
                factor=float(obj.get("factor", 8.0)),
                low_freq_factor=float(obj.get("low_freq_factor", 1.0)),
                high_freq_factor=float(obj.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(obj.get("original_max_position_embeddings", 8192)),
            )
        if kind == "linear":
            factor = float(obj.get("factor", 1.0))
            if not factor > 0.0:
                raise ConfigError(f"config.json `{where}.factor` must be positive, found {factor}")
            return RopeScaling(kind="linear", factor=factor)
        raise ConfigError(
            f"config.json `{where}` has rope type `{kind}`; this engine knows: default, llama3, linear")


def _req(cfg: dict, key: str, kind=int):
    if key not in cfg or cfg[key] is None:
        raise ConfigError(f"config.json is missing `{key}`")
    try:
        return kind(cfg[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json `{key}` = {cfg[key]!r} is not {kind.__name__}") from e


def _opt(cfg: dict, key: str, default, kind=int):
    v = cfg.get(key)
    if v is None:
        return default
    try:
        return kind(v)
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json `{key}` = {v!r} is not {kind.__name__}") from e


def _eos_ids(v: Any) -> tuple[int, ...]:
    if v is None:
        return ()
    if isinstance(v, (list, tuple)):
        return tuple(int(x) for x in v)
    return (int(v),)


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama dense decoder's hyper-parameters, one field per config.json key."""

    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    @staticmethod
    def from_json(cfg: dict) -> "LlamaConfig":
        archs = cfg.get("architectures") or []
        if not archs:
            raise ConfigError("config.json is missing `architectures`")
        n_head = _req(cfg, "num_attention_heads")
        hidden = _req(cfg, "hidden_size")
        n_kv = _opt(cfg, "num_key_value_heads", n_head)
        if n_head <= 0 or hidden <= 0:
            raise ConfigError("config.json `num_attention_heads` and `hidden_size` must be positive")
        head_dim = _opt(cfg, "head_dim", None)
        if head_dim is None:
            if hidden % n_head:
                raise ConfigError(
                    f"config.json has no `head_dim` and `hidden_size` {hidden} is not a multiple of "
                    f"`num_attention_heads` {n_head}")
            head_dim = hidden // n_head
        if n_kv <= 0 or n_head % n_kv:
            raise ConfigError(
                f"config.json `num_key_value_heads` {n_kv} must divide `num_attention_heads` {n_head}")
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"config.json `head_dim` {head_dim} must be even")
        scaling_obj = cfg.get("rope_scaling")
        rope_theta = _opt(cfg, "rope_theta", None, float)
        params = cfg.get("rope_parameters")
        if isinstance(params, dict):
            # newer checkpoints keep theta and the scaling in one object
            if rope_theta is None and params.get("rope_theta") is not None:
                rope_theta = float(params["rope_theta"])
            if scaling_obj is None:
                scaling_obj = params
        layers = _req(cfg, "num_hidden_layers")
        if layers <= 0:
            raise ConfigError("config.json `num_hidden_layers` must be positive")
        if cfg.get("mlp_bias"):
            # the reference has no name for an mlp bias tensor
            # (src/provider/local/convert/tensors.rs:899-904)
            raise ConfigError("config.json `mlp_bias` = true: feed-forward biases are not part of this architecture")
        for key in ("hidden_act", "hidden_activation"):
            act = cfg.get(key)
            if act is not None and str(act).lower() not in ("silu", "swish"):
                # the reference fixes the activation by the architecture's row: SiLU for this one
                # (src/provider/local/model/arch.rs:283-319); another one here would run SiLU without a word
                raise ConfigError(f"config.json `{key}` = {act!r}: this architecture's feed-forward is SiLU-gated")
        eps = _opt(cfg, "rms_norm_eps", 1e-6, float)
        if not eps > 0.0:
            raise ConfigError(f"config.json `rms_norm_eps` must be positive, found {eps}")
        return LlamaConfig(
            architecture=str(archs[0]),
            num_hidden_layers=layers,
            hidden_size=hidden,
            num_attention_heads=n_head,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            intermediate_size=_req(cfg, "intermediate_size"),
            vocab_size=_req(cfg, "vocab_size"),
            max_position_embeddings=_req(cfg, "max_position_embeddings"),
            rms_norm_eps=eps,
            rope_theta=10000.0 if rope_theta is None else rope_theta,
            rope_scaling=RopeScaling.from_json(scaling_obj),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            attention_bias=bool(cfg.get("attention_bias", False)),
            eos_token_ids=_eos_ids(cfg.get("eos_token_id")),
            bos_token_id=_opt(cfg, "bos_token_id", None),
        )

    def to_json(self) -> dict:
        """The config.json a model folder of this configuration carries."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": "silu",
        }
        s = self.rope_scaling
        if s.kind == "llama3":
            out["rope_scaling"] = {
                "rope_type": "llama3", "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        elif s.kind == "linear":
            out["rope_scaling"] = {"rope_type": "linear", "factor": s.factor}
        else:
            out["rope_scaling"] = None
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        return out


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e

"""One registry from an architecture's name (config.json `architectures[0]`) to its model builder.

A builder takes the parsed config.json and returns a `ModelSpec` (see
`models/spec.py`). An unknown name is an error that lists the registered
names, as the reference's `Arch::from_name` does
(src/provider/local/model/arch.rs:375-385).
"""
from __future__ import annotations

from typing import Callable

from .model_config import ConfigError

_BUILDERS: dict[str, Callable] = {}


def register_architecture(*names: str):
    def deco(fn):
        for n in names:
            _BUILDERS[n] = fn
        return fn
    return deco


def architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_BUILDERS)


def _ensure_builtin() -> None:
    from ..models import llama  # noqa: F401  (registers itself)


def build_spec(config_json: dict):
    """config.json (a dict) -> ModelSpec, through the registered builder of its architecture."""
    _ensure_builtin()
    archs = config_json.get("architectures") or []
    if not archs:
        raise ConfigError("config.json is missing `architectures`")
    name = str(archs[0])
    if name not in _BUILDERS:
        raise ConfigError(f"architecture `{name}` is not registered; registered: {', '.join(sorted(_BUILDERS))}")
    spec = _BUILDERS[name](config_json)
    spec.validate()
    return spec

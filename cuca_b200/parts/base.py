"""Interfaces of the parts a model is put together from, and their registries.

A model is data: a list of layers, each naming a block arrangement, a mixer, a
feed-forward and its norms by registry key with their sizes and constants
(`PartSpec`), plus a run order (`models/spec.py`). A part never learns which
model it sits in: it gets its own parameters, the names of its tensors and,
at step time, the batch description and its cache view.

Interfaces (all tensors live on the runtime's device):

* `Norm.forward(x, rows=None) -> h`: x is the 32-bit residual stream
  `[T, E]`; h has the compute dtype. `rows` (int32 device tensor) gathers rows.
* `PositionEncoding.prepare(context_length)`; `fused_tables()` returns
  `(cos, sin, rotary_dim)` for the fused rotate-and-store kernel, or None, in
  which case `apply(qkv, ...)` must rotate q and k in place.
* `Mixer.forward(h, stream, step, cache)`: adds the mixer's output to the
  32-bit residual stream in place. `cache_needs()` declares paged keys/values
  (`KvNeeds`) and/or fixed-size per-request state (`StateNeeds`).
* `FeedForward.forward(h, stream, step)`: adds its output to the stream.
* `Block.forward(stream, step, cache)`: arranges norms, mixer, feed-forward.

Every part also has `tensors()` (name -> expected shape, for the loader's one
error) and `load(get)` (`get(name)` returns the checked tensor on the device).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by the configuration: registry key, constants, tensor names."""

    kind: str
    params: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)  # role -> tensor name in the checkpoint


@dataclass(frozen=True)
class TensorNeed:
    """What a part expects of one checkpoint tensor."""

    shape: tuple
    optional: bool = False
    keep_fp32: bool = False  # small vectors (norm weights) stay 32-bit in every mode
    init: str = "normal"  # random-weights mode: "normal" N(0, std) or "ones"


@dataclass(frozen=True)
class KvNeeds:
    """Paged keys and values: layers with equal needs share a group of pages."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: all keys; w: the last w keys


@dataclass(frozen=True)
class StateNeeds:
    """Per-request state of fixed size, kept in the request's slot."""

    shape: tuple
    dtype: str = "float32"


@dataclass
class CacheNeeds:
    kv: Optional[KvNeeds] = None
    state: Optional[StateNeeds] = None


class Part:
    """Base of every part. `spec.params` holds its sizes and constants."""

    def __init__(self, spec: PartSpec, runtime):
        self.spec = spec
        self.rt = runtime

    def tensors(self) -> dict[str, TensorNeed]:
        return {}

    def load(self, get: Callable[[str], Any]) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of parameters a step reads from this part."""
        return 0


class Norm(Part):
    def forward(self, x, rows=None):  # pragma: no cover - interface
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, context_length: int) -> None:
        pass

    def fused_tables(self):
        return None

    def apply(self, qkv, n_heads: int, n_kv_heads: int, head_dim: int, positions) -> None:
        raise NotImplementedError


class Mixer(Part):
    graph_safe = False  # True when forward() only launches kernels on static buffers

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def prepare(self, context_length: int) -> None:
        pass

    def forward(self, h, stream, step, cache) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    graph_safe = False

    def forward(self, h, stream, step) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream."""

    def __init__(self, spec: PartSpec, runtime, mixer: Mixer, feed_forward: FeedForward,
                 mixer_norm: Norm, ffn_norm: Norm):
        super().__init__(spec, runtime)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None]

    def forward(self, stream, step, cache) -> None:  # pragma: no cover - interface
        raise NotImplementedError


# ----------------------------------------------------------------------------
# registries
# ----------------------------------------------------------------------------
class Registry:
    """Name -> class, with an error that lists what is registered."""

    def __init__(self, what: str):
        self.what = what
        self._items: dict[str, Any] = {}

    def register(self, name: str):
        def deco(obj):
            self._items[name] = obj
            return obj
        return deco

    def get(self, name: str):
        if name not in self._items:
            known = ", ".join(sorted(self._items)) or "(none)"
            raise KeyError(f"unknown {self.what} `{name}`; registered: {known}")
        return self._items[name]

    def names(self) -> list[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register

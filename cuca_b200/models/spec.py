"""A model as data: parts chosen layer by layer, and the order they run in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its block arrangement and the parts inside it."""

    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class Run:
    """One entry of the run order: which layer runs and which cache it uses.

    `cache` names a cache (keys/values and state) by number. The entry that
    `owns` it writes it; an entry with `owns=False` reads what an earlier entry
    wrote (its mixer must be built with `shares_cache`). A layer named twice
    runs twice, each run with a cache of its own unless it names a shared one.
    """

    layer: int
    cache: int
    owns: bool = True


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple = ()
    ignorable_tensor: Callable[[str], bool] = field(default=lambda name: False)

    def validate(self) -> None:
        owners = {}
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {run.layer}; the model has {len(self.layers)}")
            if run.owns:
                if run.cache in owners:
                    raise ValueError(f"cache {run.cache} is written by run entries {owners[run.cache]} and {i}")
                owners[run.cache] = i
            elif run.cache not in owners:
                raise ValueError(f"run order entry {i} reads cache {run.cache} before any entry writes it")


def default_schedule(n_layers: int) -> list:
    return [Run(layer=i, cache=i, owns=True) for i in range(n_layers)]

"""Rotary position encoding: tables of cos/sin per position and pair.

theta(pos, i) = pos * base^(-2i/n) / factor_i * freq_scale, computed in 64-bit
and stored as 32-bit tables [positions, n/2] (src/provider/local/model/rope.rs:
118-152). `llama3` scaling gives per-pair divisors computed as the reference's
converter does, with the frequency in 32-bit
(src/provider/local/convert/config.rs:525-565); `linear` scales every frequency
by 1/factor (src/provider/local/model/params.rs:535-572). Pairs are (i, i + n/2)
in Hugging Face row order, which equals the reference's adjacent pairs on its
permuted rows (src/provider/local/model/cpu.rs:4247-4275).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding, register_position


def llama3_factors(n_dims: int, base: float, factor: float, low: float, high: float, original: int) -> np.ndarray:
    out = np.empty(n_dims // 2, dtype=np.float32)
    low_wavelen, high_wavelen = original / low, original / high
    for i in range(n_dims // 2):
        freq = np.float32(1.0) / np.power(np.float32(base), np.float32(2 * i) / np.float32(n_dims), dtype=np.float32)
        wavelen = 2.0 * math.pi / float(freq)
        if wavelen < high_wavelen:
            r = 1.0
        elif wavelen > low_wavelen:
            r = factor
        else:
            smooth = (original / wavelen - low) / (high - low)
            r = 1.0 / ((1.0 - smooth) / factor + smooth)
        out[i] = np.float32(r)
    return out


def rope_tables(positions: int, n_dims: int, base: float, factors=None, freq_scale: float = 1.0):
    """cos, sin as float32 CPU tensors [positions, n_dims // 2], angles in float64."""
    i = np.arange(n_dims // 2, dtype=np.float64)
    inv = np.power(np.float64(base), -(2.0 * i) / n_dims)
    if factors is not None:
        inv = inv / np.asarray(factors, dtype=np.float64)
    inv = inv * freq_scale
    theta = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return (torch.from_numpy(np.cos(theta).astype(np.float32)), torch.from_numpy(np.sin(theta).astype(np.float32)))


@register_position("rope")
class RotaryEncoding(PositionEncoding):
    """params: head_dim, rotary_dim, theta, scaling {kind, factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings}."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.theta = float(p["theta"])
        self.scaling = dict(p.get("scaling") or {"kind": "default"})
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and at most the head size {self.head_dim}")
        self.cos = self.sin = None

    def host_tables(self, context_length: int):
        kind = self.scaling.get("kind", "default")
        factors, freq_scale = None, 1.0
        if kind == "llama3":
            factors = llama3_factors(self.rotary_dim, self.theta, float(self.scaling["factor"]),
                                     float(self.scaling["low_freq_factor"]), float(self.scaling["high_freq_factor"]),
                                     int(self.scaling["original_max_position_embeddings"]))
        elif kind == "linear":
            freq_scale = 1.0 / float(self.scaling["factor"])
        elif kind != "default":
            raise ValueError(f"rope scaling `{kind}` is unknown; known: default, llama3, linear")
        return rope_tables(context_length, self.rotary_dim, self.theta, factors, freq_scale)

    def prepare(self, context_length: int) -> None:
        cos, sin = self.host_tables(context_length)
        self.cos = cos.to(self.rt.device)
        self.sin = sin.to(self.rt.device)

    def fused_tables(self):
        return self.cos, self.sin, self.rotary_dim

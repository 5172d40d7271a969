"""Token embedding and output head.

x[r] = E[token[r]] into the 32-bit stream (src/provider/local/model/cpu.rs:2193-2198);
logits = n W_head^T in 32-bit, W_head = lm_head or the embedding table when tied
(src/provider/local/model/cpu.rs:1614-1622,2586-2621).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, TensorNeed


class TokenEmbedding(Part):
    """params: vocab, width. tensors: weight [vocab, width]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.weight = None

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width))}

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])

    def forward(self, tokens, out) -> None:
        ops.embed(self.weight, tokens, out, self.rt.err)


class OutputHead(Part):
    """params: vocab, width. tensors: weight [vocab, width] (the embedding's name when tied)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.weight = None

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.vocab, self.width))}

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, h) -> torch.Tensor:
        return self.rt.linear(h, self.weight, out_dtype=torch.float32)

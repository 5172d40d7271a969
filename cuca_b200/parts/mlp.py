"""Dense SwiGLU feed-forward: y = down(silu(gate f) * (up f))
(src/provider/local/model/cpu.rs:3554-3565). gate and up are stacked into one
weight at load so one contraction with a SwiGLU epilogue yields the activation
(the reference accepts the stacked form too: model/cpu.rs:3131-3136)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorNeed, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: width, inner. tensors: gate [inner, width], up [inner, width], down [width, inner]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.w_gate_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        return {t["gate"]: TensorNeed((self.inner, self.width)), t["up"]: TensorNeed((self.inner, self.width)),
                t["down"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_gate_up = torch.cat([get(t["gate"]), get(t["up"])], dim=0).contiguous()
        self.w_down = get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        act = self.rt.linear(h, self.w_gate_up, epilogue=ops.EPI_SWIGLU)
        self.rt.stream(stream).add_linear(act, self.w_down)

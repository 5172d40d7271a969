"""RMSNorm: h = x * rsqrt(mean(x^2) + eps) * w, the weight multiplies directly
(src/provider/local/model/cpu.rs:3651-3654; formula in model/gpu.rs:5883-5896)."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, TensorNeed, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: width, eps. tensors: weight [width]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensors(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.width,), keep_fp32=True, init="ones")}

    def load(self, get):
        self.weight = get(self.spec.tensors["weight"])

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, stream, rows=None):
        # this kernel adds the K slices a contraction left on the stream while it reads the stream
        x, pending = self.rt.stream(stream).take()
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty(n, self.width)
        if pending is not None:
            ops.add_partials_rmsnorm(x, pending, self.weight, out, self.eps, rows)
        else:
            ops.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

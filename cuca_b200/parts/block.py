"""Block arrangements. `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x))
(src/provider/local/model/cpu.rs:2650-2704 with pre_norms on, post_norms off)."""
from __future__ import annotations

from .base import Block, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def _norm(self, norm, stream):
        # a contraction may have left unadded K slices on the stream; a norm that cannot add them gets them added
        if not getattr(norm, "consumes_partials", False):
            self.rt.flush(stream)
        return norm.forward(stream)

    def forward(self, stream, step, cache) -> None:
        h = self._norm(self.mixer_norm, stream)
        self.mixer.forward(h, stream, step, cache)
        if self.feed_forward is not None:
            f = self._norm(self.ffn_norm, stream)
            self.feed_forward.forward(f, stream, step)

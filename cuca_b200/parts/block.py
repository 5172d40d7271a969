"""Block arrangements. `pre_norm`: x += mixer(norm(x)); x += ffn(norm(x))
(src/provider/local/model/cpu.rs:2650-2704 with pre_norms on, post_norms off)."""
from __future__ import annotations

from .base import Block, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    def forward(self, stream, step, cache) -> None:
        h = self.mixer_norm.forward(stream)
        self.mixer.forward(h, stream, step, cache)
        if self.feed_forward is not None:
            f = self.ffn_norm.forward(stream)
            self.feed_forward.forward(f, stream, step)

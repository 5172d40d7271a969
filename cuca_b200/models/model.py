"""The generic model: parts built from a `ModelSpec`, run in the order its schedule gives."""
from __future__ import annotations

import torch

from ..parts import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from ..parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, TensorNeed
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights import loader
from .spec import ModelSpec


class Model:
    """Embedding, the layers' blocks, final norm and head; `runtime=None` builds a model that can only
    describe itself (tensor names and shapes), which is what the weight checks need on a machine without GPU."""

    def __init__(self, spec: ModelSpec, runtime=None):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = TokenEmbedding(spec.embedding, runtime)
        self.blocks = []
        for ls in spec.layers:
            mixer = MIXERS.get(ls.mixer.kind)(ls.mixer, runtime)
            ffn = FEED_FORWARDS.get(ls.feed_forward.kind)(ls.feed_forward, runtime) if ls.feed_forward else None
            mixer_norm = NORMS.get(ls.mixer_norm.kind)(ls.mixer_norm, runtime) if ls.mixer_norm else None
            ffn_norm = NORMS.get(ls.ffn_norm.kind)(ls.ffn_norm, runtime) if ls.ffn_norm else None
            self.blocks.append(BLOCKS.get(ls.block.kind)(ls.block, runtime, mixer, ffn, mixer_norm, ffn_norm))
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, runtime)
        self.head = OutputHead(spec.head, runtime)
        self.loaded = False

    # ------------------------------------------------------------ description
    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def tensor_needs(self) -> dict:
        needs: dict[str, TensorNeed] = {}
        for part in self.parts():
            for name, need in part.tensors().items():
                if name in needs and tuple(needs[name].shape) != tuple(need.shape):
                    raise ValueError(f"tensor `{name}` is wanted as {needs[name].shape} and as {need.shape}")
                needs.setdefault(name, need)
        return needs

    def cache_needs(self) -> dict:
        """cache number -> what its owning layer's mixer keeps there."""
        out = {}
        for run in self.spec.schedule:
            if run.owns:
                out[run.cache] = self.blocks[run.layer].mixer.cache_needs()
        return out

    def graph_safe(self) -> bool:
        return all(b.mixer.graph_safe and (b.feed_forward is None or b.feed_forward.graph_safe) for b in self.blocks)

    # ------------------------------------------------------------ weights
    def check_weights(self, source: loader.WeightSource) -> None:
        loader.check_tensors(self.tensor_needs(), source.shapes(), self.spec.ignorable_tensor, source.describe())

    def load(self, source: loader.WeightSource) -> None:
        if self.rt is None:
            raise RuntimeError("a model built without a runtime cannot hold weights")
        needs = self.tensor_needs()
        self.check_weights(source)
        raw = loader.binder(needs, source, self.rt.device, self.rt.dtype)
        seen: dict = {}

        def get(name):
            if name not in seen:
                seen[name] = raw(name)
            return seen[name]

        for part in self.parts():
            part.load(get)
        self.loaded = True

    def prepare(self, context_length: int) -> None:
        for b in self.blocks:
            b.mixer.prepare(context_length)

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads (every layer's parts once per run, the head, no embedding table)."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for run in self.spec.schedule:
            total += sum(p.weight_bytes() for p in self.blocks[run.layer].parts())
        return total

    # ------------------------------------------------------------ step
    def forward(self, step, cache) -> torch.Tensor | None:
        """Run the step's rows through the model; logits [wanted rows, vocab] in 32-bit, or None."""
        x = torch.empty(step.n_rows, self.spec.width, dtype=torch.float32, device=self.rt.device)
        self.embedding.forward(step.tokens, x)
        stream = self.rt.stream(x)
        for run in self.spec.schedule:
            self.blocks[run.layer].forward(stream, step, cache.view(run.cache, step))
        if step.logit_rows is None or step.n_logit_rows == 0:
            stream.drop_pending()
            return None
        h = self.final_norm.forward(stream, rows=step.logit_rows)
        return self.head.forward(h)

"""How a layer's parts are arranged.  "prenorm_residual" is the reference's block:
x += mixer(norm(x)); x += feed_forward(norm(x)), pre-norms only
(imparo-model/src/lfm2/workflow_cpu.rs:8-18,172-319)."""
from __future__ import annotations

from .base import Part, make_part


class PreNormResidualBlock(Part):
    """params: layer (LayerSpec)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        spec = params["layer"]
        self.mixer_norm = make_part("norm", spec.mixer_norm, prefix, rt)
        self.mixer = make_part("mixer", spec.mixer, prefix, rt)
        self.ff_norm = make_part("norm", spec.feed_forward_norm, prefix, rt)
        self.ff = make_part("feed_forward", spec.feed_forward, prefix, rt)
        self.parts = (self.mixer_norm, self.mixer, self.ff_norm, self.ff)
        self.graph_safe = all(p.graph_safe for p in self.parts)

    def weight_specs(self):
        return [w for p in self.parts for w in p.weight_specs()]

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, x, batch, caches):
        """x: the 32-bit residual stream [tokens, width], updated in place."""
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x), batch, caches, x)
        self.ff.forward(self._normed(self.ff_norm, self.ff, x), batch, x)

    @staticmethod
    def _normed(norm, consumer, x):
        if consumer.accepts_lazy_input and hasattr(norm, "lazy"):
            return norm.lazy(x)
        return norm.forward(x)

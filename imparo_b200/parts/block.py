"""How a layer's parts are arranged.  "prenorm_residual" is the reference's block:
x += mixer(norm(x)); x += feed_forward(norm(x)), pre-norms only
(imparo-model/src/lfm2/workflow_cpu.rs:8-18,172-319)."""
from __future__ import annotations

from .base import Block, make_part


class PreNormResidualBlock(Block):
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
        self.picks_rows = True         # forward(only_rows=...) is implemented

    def weight_specs(self):
        return [w for p in self.parts for w in p.weight_specs()]

    def bind(self, tensors):
        for p in self.parts:
            p.bind(tensors)

    def cache_specs(self):
        return self.mixer.cache_specs()

    def forward(self, x, batch, caches, only_rows=None):
        """x: the 32-bit residual stream [tokens, width], updated in place.
        only_rows = (rows, n): the caller needs the block's output at these n rows only (the
        model's last block, whose output feeds nothing but the wanted logits; the reference skips
        the same work, imparo-model/src/lfm2/workflow_gpu.rs:990-992,1201-1203).  The mixer still
        runs on every row (its cache and state advance); the feed-forward runs on the picked rows,
        and their stream [n, width] is returned instead (None when n is 0)."""
        from ..kernels import ops
        if self.rt.probe_now:
            return self._forward_probed(x, batch, caches, only_rows)
        h = self.mixer_norm.forward(x, tag="normed_mixer")
        self._run(self.mixer, x, lambda: self.mixer.forward(h, batch, caches, x))
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                ops.settle(x)
                return None
            xs = self.rt.workspace.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            picked_in = self.ff_norm.forward(xs, tag="normed_ff")
            self._run(self.ff, xs, lambda: self.ff.forward(picked_in, batch, xs))
            return xs
        ff_in = self.ff_norm.forward(x, tag="normed_ff")
        self._run(self.ff, x, lambda: self.ff.forward(ff_in, batch, x))
        return None

    def _forward_probed(self, x, batch, caches, only_rows):
        """The same block with every stage evaluated and shown to the runtime's probe: the stream
        going in, the mixer's normed input, the stream after the mixer, the feed-forward's normed
        input, the stream going out.  Nothing is deferred here."""
        from ..kernels import ops
        probe = self.rt.probe
        ops.settle(x)
        probe("stream_in", x)
        h = self.mixer_norm.forward(x, tag="normed_mixer")
        probe("mixer_norm", h)
        ops.settle(x)
        self.mixer.forward(h, batch, caches, x)
        ops.settle(x)
        probe("stream_mixer", x)
        if only_rows is not None:
            rows, n = only_rows
            if n == 0:
                return None
            xs = self.rt.workspace.get("stream_picked", (n, x.shape[1]), x.dtype, first="rows")
            ops.gather_rows(x, rows, xs)
            x = xs
        ff_in = self.ff_norm.forward(x, tag="normed_ff")
        probe("ff_norm", ff_in)
        self.ff.forward(ff_in, batch, x)
        ops.settle(x)
        probe("stream_out", x)
        return x if only_rows is not None else None

    @staticmethod
    def _run(part, x, call) -> None:
        """A part whose last write to the stream is an accumulate-product may leave that add as
        split partials for the next norm to fold (ops.allow_deferred_add); any other part gets
        and leaves a stream that is whole."""
        from ..kernels import ops
        if part.adds_with_linear:
            ops.allow_deferred_add(x)
            try:
                call()
            finally:
                ops.disallow_deferred_add(x)
        else:
            ops.settle(x)
            call()

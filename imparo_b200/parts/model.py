"""A model put together from a ModelSpec: embedding, the layers, the order they run in,
final norm and head.  It holds no architecture-specific code."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .base import Part, Runtime, make_part
from .spec import ModelSpec, PartSpec, WeightSpec


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = make_part("embedding", spec.embedding, "", rt)
        self.layers: List[Part] = [make_part("block", PartSpec(ls.block, {"layer": ls}), ls.prefix, rt)
                                   for ls in spec.layers]
        self.final_norm = make_part("norm", spec.final_norm, "", rt)
        self.head = make_part("head", spec.head, "", rt)
        self.schedule = spec.schedule
        self.graph_safe = all(p.graph_safe for p in self.parts())
        for i, e in enumerate(self.schedule):
            if e.cache_from is not None:
                mine = self.layers[e.layer].cache_specs()
                theirs = self.layers[self.schedule[e.cache_from].layer].cache_specs()
                if mine != theirs:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                                     f"but their cache needs differ: {mine} vs {theirs}")

    # -- weights -----------------------------------------------------------------------
    def parts(self) -> Sequence[Part]:
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def weight_specs(self) -> List[WeightSpec]:
        """Every tensor the model reads, once per name (a tied head names the embedding's)."""
        seen: Dict[str, WeightSpec] = {}
        for p in self.parts():
            for w in p.weight_specs():
                old = seen.get(w.name)
                if old is None:
                    seen[w.name] = w
                elif old.shapes != w.shapes or old.role != w.role:
                    raise ValueError(f"tensor '{w.name}' is declared twice with different shapes or roles")
        return list(seen.values())

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.bind(tensors)

    # -- cache needs -------------------------------------------------------------------
    def cache_requirements(self) -> List[Tuple[int, Tuple]]:
        """For every schedule entry that OWNS a cache: (entry index, its cache specs)."""
        out = []
        for i, e in enumerate(self.schedule):
            if e.cache_from is None:
                specs = self.layers[e.layer].cache_specs()
                if specs:
                    out.append((i, tuple(specs)))
        return out

    # -- running -----------------------------------------------------------------------
    def forward(self, batch, cache_views, wanted=None):
        """Runs the batch's tokens through every schedule entry.  cache_views(entry) gives
        the tuple of bound cache views for that entry.  Returns the residual stream.

        wanted = (rows, n): only these n rows of the result will be read (the logits' rows).  When
        they are fewer than the batch's tokens and the last entry is a block that can run its
        feed-forward on picked rows, the result is (stream of the picked rows [n, width] or None
        for n = 0, True); else (the whole stream, False)."""
        x = self.embedding.forward(batch)
        last = len(self.schedule) - 1
        for i, e in enumerate(self.schedule):
            layer = self.layers[e.layer]
            self.rt.probe_now = self.rt.probe is not None and self.rt.probe_entry == i
            if i == last and wanted is not None and wanted[1] < batch.n_tokens and layer.picks_rows:
                out = layer.forward(x, batch, cache_views(i), only_rows=wanted)
                self.rt.probe_now = False
                return out, True
            layer.forward(x, batch, cache_views(i))
        self.rt.probe_now = False
        return (x, False) if wanted is not None else x

    def settle(self, x: torch.Tensor) -> None:
        """Make the stream whole (fold split partials a product may have left) for a reader that
        does not go through the ops launchers."""
        from ..kernels import ops
        ops.settle(x)

    def logits(self, x: torch.Tensor, rows: Optional[torch.Tensor], n_rows: int) -> torch.Tensor:
        """Final norm and head at the wanted rows only: [n_rows, vocab] in 32-bit.  rows None: x
        holds exactly the wanted rows."""
        h = self.final_norm.forward(x, rows=rows, n_rows=n_rows, tag="final_normed")
        return self.head.forward(h)

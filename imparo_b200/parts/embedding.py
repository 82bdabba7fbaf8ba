"""Token embedding and output head as parts.

Embedding: rows of the table, unscaled, into the 32-bit residual stream
(imparo-model/src/cpu_support.rs:327-342; lfm2/plan.rs:147-151).  Head: logits = h * E^T
in 32-bit, E the embedding table when tied, no softcap and no scale for this
architecture (cpu_support.rs:451-466; lfm2/plan.rs:163-169)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class TokenEmbedding(Part):
    """params: vocab, width, name."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab"])
        self.width = int(params["width"])
        self.name = prefix + params["name"]
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name, ((self.vocab, self.width),))]

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, batch) -> torch.Tensor:
        """batch: the step's batch (token_ids, positions, item_of_token, ... on the device).  This part reads
        the token ids only; an embedding that adds learned positions or segment rows reads the rest."""
        out = self.rt.workspace.get("residual", (batch.n_tokens, self.width), torch.float32, first="tokens")
        ops.embed_gather(self.table, batch.token_ids, out, self.rt.status)
        return out


class LinearHead(Part):
    """params: vocab, width, name (the table's own tensor, or the embedding's when tied)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab"])
        self.width = int(params["width"])
        self.name = prefix + params["name"]
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name, ((self.vocab, self.width),))]

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.rt.workspace.get("logits", (h.shape[0], self.vocab), torch.float32, first="rows")
        ops.linear(h, self.table, logits, status=self.rt.status)
        return logits

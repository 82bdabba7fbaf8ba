"""RMS norm as a part: y = x * 1/sqrt(mean(x^2) + eps) * w, sums in 32-bit
(imparo-cpu/src/ops.rs:6-22)."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class RMSNorm(Part):
    """params: width, eps, name (tensor name after the prefix, e.g. "operator_norm.weight")."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = prefix + params["name"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self):
        return [WeightSpec(self.name, ((self.width,),), role="vector", init=("norm",))]

    def bind(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                tag: str = "normed") -> torch.Tensor:
        """x: 32-bit [tokens, width].  rows (int32, device) picks input rows; n_rows is how
        many of them.  Returns activations in the path's dtype."""
        n = x.shape[0] if rows is None else int(n_rows if n_rows is not None else rows.numel())
        out = self.rt.workspace.get(tag, (n, self.width), self.rt.act_dtype, first="tokens" if rows is None else "rows")
        ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

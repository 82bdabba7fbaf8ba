"""Position encodings.  An attention mixer asks its position part for the table of
per-pair inverse frequencies that its fused norm+rotation kernel applies (rotary()); a
part that returns None adds no position information.  Any half-split rotation — scaled
or per-pair adjusted frequencies, a rotation of only the first n_rot dimensions — is a
part that returns its own table.

RotaryNeox: pairs (i, i + n_rot/2); angle = position * theta^(-2i/n_rot), the product
rounded to 32 bits, then sin and cos (imparo-cpu/src/ops.rs:551-569).  The per-pair
inverse frequency is computed in 64-bit on the host and kept as a 32-bit table."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import Part


class PositionEncoding(Part):
    def rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        """(inv_freq float32 [n_rot/2] on the device, n_rot): dimension i < n_rot/2 pairs
        with i + n_rot/2 and turns by position * inv_freq[i].  None: no rotation."""
        return None


class NoPosition(PositionEncoding):
    pass


class RotaryNeox(PositionEncoding):
    """params: head_dim, theta, n_rot (default head_dim)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.head_dim = int(params["head_dim"])
        self.n_rot = int(params.get("n_rot", self.head_dim))
        self.theta = float(params["theta"])
        if self.n_rot % 2 or self.n_rot > self.head_dim:
            raise ValueError(f"rotary: n_rot {self.n_rot} must be even and at most the head size {self.head_dim}")
        i = torch.arange(self.n_rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.n_rot).to(torch.float32)
        self.inv_freq = inv.to(rt.device)

    def rotary(self):
        return self.inv_freq, self.n_rot

"""SwiGLU feed-forward as a part: down(silu(gate(x)) * up(x)), SiLU on the gate
(imparo-model/src/lfm2/workflow_cpu.rs:307-313; imparo-cpu/src/ops.rs:73-78).
gate = w1, up = w3, down = w2."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class SwiGLU(Part):
    """params: hidden, ff, names (optional)."""
    adds_with_linear = True


    NAMES = {"gate": "feed_forward.w1.weight", "up": "feed_forward.w3.weight", "down": "feed_forward.w2.weight"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden"])
        self.ff = int(params["ff"])
        self.names = {k: prefix + v for k, v in {**self.NAMES, **params.get("names", {})}.items()}
        self.w_gu = self.w_down = None

    def weight_specs(self):
        n, H, F = self.names, self.hidden, self.ff
        return [WeightSpec(n["gate"], ((F, H),)), WeightSpec(n["up"], ((F, H),)), WeightSpec(n["down"], ((H, F),))]

    def bind(self, tensors):
        n = self.names
        # one fused projection [gate | up]
        self.w_gu = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]]

    def forward(self, x, batch, residual):
        rt, T, F = self.rt, x.shape[0], self.ff
        h = rt.workspace.get("ffn_h", (T, F), rt.act_dtype, first="tokens")
        # [T, 2F] is made only where no kernel has silu(gate) * up in its epilogue
        ops.linear_swiglu(x, self.w_gu, h, rt.status, tmp=lambda: rt.workspace.get("ffn_gu", (T, 2 * F), rt.act_dtype, first="tokens"))
        ops.linear(h, self.w_down, residual, accumulate=True, status=rt.status)

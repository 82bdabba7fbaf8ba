"""Gated short convolution as a part: in_proj to [b | c | x], depthwise causal
convolution over b*x with a rolling per-request state of taps-1 values, gate by c,
out_proj (imparo-model/src/lfm2/workflow_cpu.rs:260-277; imparo-cpu/src/ops.rs:109-167).
The reference has no bias; with bias=True a per-channel bias is added before the gate,
and in_proj/out_proj biases are added when the file carries them."""
from __future__ import annotations

from ..kernels import ops
from .base import Part
from .spec import SlotState, WeightSpec


class ShortConvMixer(Part):
    """params: hidden, taps, bias (bool), names (optional)."""
    adds_with_linear = True


    NAMES = {"in": "conv.in_proj.weight", "conv": "conv.conv.weight", "out": "conv.out_proj.weight",
             "conv_bias": "conv.conv.bias", "in_bias": "conv.in_proj.bias", "out_bias": "conv.out_proj.bias"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden"])
        self.taps = int(params["taps"])
        self.bias = bool(params.get("bias", False))
        if not 2 <= self.taps <= 16:
            raise ValueError(f"short conv: {self.taps} taps; the kernel takes 2 to 16 (one tap carries no state)")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **params.get("names", {})}.items()}
        self.w_in = self.w_out = self.w_conv = self.b_conv = self.b_in = self.b_out = None

    def weight_specs(self):
        n, H, L = self.names, self.hidden, self.taps
        specs = [WeightSpec(n["in"], ((3 * H, H),)),
                 WeightSpec(n["conv"], ((H, 1, L), (H, L)), role="vector", init=("conv_taps",)),
                 WeightSpec(n["out"], ((H, H),))]
        if self.bias:
            specs += [WeightSpec(n["conv_bias"], ((H,),), role="vector", init=("bias",)),
                      WeightSpec(n["in_bias"], ((3 * H,),), role="vector", init=("skip",), optional=True),
                      WeightSpec(n["out_bias"], ((H,),), role="vector", init=("skip",), optional=True)]
        return specs

    def bind(self, tensors):
        n = self.names
        self.w_in = tensors[n["in"]]
        self.w_out = tensors[n["out"]]
        self.w_conv = tensors[n["conv"]].reshape(self.hidden, self.taps).contiguous()   # tap fastest, tap 0 oldest
        self.b_conv = tensors.get(n["conv_bias"])
        self.b_in = tensors.get(n["in_bias"])
        self.b_out = tensors.get(n["out_bias"])

    def cache_specs(self):
        return (SlotState((self.taps - 1, self.hidden)),)

    def forward(self, x, batch, caches, residual):
        st = caches[0]
        rt, T, H = self.rt, x.shape[0], self.hidden
        bcx = rt.workspace.get("conv_bcx", (T, 3 * H), rt.act_dtype, first="tokens")
        if self.b_in is None:
            bcx = ops.linear_unfolded(x, self.w_in, bcx, status=rt.status)     # the conv kernel can add split partials itself
        else:
            ops.linear(x, self.w_in, bcx, status=rt.status)
            ops.add_bias(bcx, self.b_in)
        y = rt.workspace.get("conv_y", (T, H), rt.act_dtype, first="tokens")
        ops.gated_conv(bcx, self.w_conv, self.b_conv, st.state, batch.item_row_start, batch.item_of_token,
                       batch.item_slot, y, self.taps, rt.status)
        ops.linear(y, self.w_out, residual, accumulate=True, status=rt.status)
        if self.b_out is not None:
            ops.add_bias(residual, self.b_out)

"""SwiGLU feed-forward as a part: down(silu(gate(x)) * up(x)), SiLU on the gate
(imparo-model/src/lfm2/workflow_cpu.rs:307-313; imparo-cpu/src/ops.rs:73-78).
gate = w1, up = w3, down = w2."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class SwiGLU(Part):
    """The gated feed-forward down(act(gate(x)) * up(x)).  params: hidden, ff, names (optional), act ("silu" by default, or
    "gelu_tanh"), bias (bool, default False: True declares a bias for each of the three products, names "gate_bias",
    "up_bias", "down_bias"; they are 32-bit and added to the products' results before the activation / after the down
    product).  forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer) instead of
    adding into it."""
    adds_with_linear = True


    NAMES = {"gate": "feed_forward.w1.weight", "up": "feed_forward.w3.weight", "down": "feed_forward.w2.weight",
             "gate_bias": "feed_forward.w1.bias", "up_bias": "feed_forward.w3.bias", "down_bias": "feed_forward.w2.bias"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden"])
        self.ff = int(params["ff"])
        self.act = params.get("act", "silu")
        if self.act not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: unknown activation '{self.act}' (silu, gelu_tanh)")
        self.bias = bool(params.get("bias", False))
        self.names = {k: prefix + v for k, v in {**self.NAMES, **params.get("names", {})}.items()}
        self.w_gu = self.w_down = self.b_gu = self.b_down = None

    def weight_specs(self):
        n, H, F = self.names, self.hidden, self.ff
        specs = [WeightSpec(n["gate"], ((F, H),)), WeightSpec(n["up"], ((F, H),)), WeightSpec(n["down"], ((H, F),))]
        if self.bias:
            specs += [WeightSpec(n["gate_bias"], ((F,),), role="vector", init=("bias",)),
                      WeightSpec(n["up_bias"], ((F,),), role="vector", init=("bias",)),
                      WeightSpec(n["down_bias"], ((H,),), role="vector", init=("bias",))]
        return specs

    def bind(self, tensors):
        n = self.names
        # one fused projection [gate | up]
        self.w_gu = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]]
        if self.bias:
            self.b_gu = torch.cat([tensors[n["gate_bias"]].float(), tensors[n["up_bias"]].float()]).contiguous()
            self.b_down = tensors[n["down_bias"]]

    def forward(self, x, batch, residual, accumulate=True):
        rt, T, F = self.rt, x.shape[0], self.ff
        h = rt.workspace.get("ffn_h", (T, F), rt.act_dtype, first="tokens")
        if self.act == "silu" and not self.bias:
            # [T, 2F] is made only where no kernel has silu(gate) * up in its epilogue
            ops.linear_swiglu(x, self.w_gu, h, rt.status, tmp=lambda: rt.workspace.get("ffn_gu", (T, 2 * F), rt.act_dtype, first="tokens"))
        else:
            ops.linear_gated(x, self.w_gu, h, self.act, bias=self.b_gu, status=rt.status,
                             tmp=lambda: rt.workspace.get("ffn_gu", (T, 2 * F), rt.act_dtype, first="tokens"))
        ops.linear(h, self.w_down, residual, accumulate=accumulate, status=rt.status)
        if self.b_down is not None:
            ops.add_bias(residual, self.b_down)


class DenseFeedForward(Part):
    """down(act(up(x))) with one activation on its own: params hidden, ff, act ("relu2": relu(z)^2, "gelu_tanh",
    "silu"), names (optional).

    forward(x, batch, residual, scale=1.0) adds scale * output into the stream; forward_into(x, out) writes the
    output into a float32 buffer instead (for an arrangement that adds several sublayers in one pass)."""
    takes_scale = True

    NAMES = {"up": "up", "down": "down"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.hidden = int(params["hidden"])
        self.ff = int(params["ff"])
        self.act = params.get("act", "relu2")
        if self.act not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward: unknown activation '{self.act}'; known: {', '.join(sorted(ops.ACTIVATIONS))}")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **params.get("names", {})}.items()}
        self.w_up = self.w_down = None

    def weight_specs(self):
        n, H, F = self.names, self.hidden, self.ff
        return [WeightSpec(n["up"], ((F, H),)), WeightSpec(n["down"], ((H, F),))]

    def bind(self, tensors):
        self.w_up = tensors[self.names["up"]]
        self.w_down = tensors[self.names["down"]]

    def input_rows(self) -> int:
        return self.ff

    def input_weight(self):
        return self.w_up

    def adopt_input_weight(self, view) -> None:
        self.w_up = view

    def forward_into(self, x, out, projected=None):
        rt, T = self.rt, x.shape[0]
        h = rt.workspace.get("ffn_h", (T, self.ff), rt.act_dtype, first="tokens")
        if projected is not None:
            ops.activation(projected, h, self.act)          # from the shared product's columns into a dense tensor
        else:
            ops.linear(x, self.w_up, h, status=rt.status)
            ops.activation(h, h, self.act)
        ops.linear(h, self.w_down, out, status=rt.status)

    def forward(self, x, batch, residual, scale: float = 1.0):
        if scale == 1.0:
            rt, T = self.rt, x.shape[0]
            h = rt.workspace.get("ffn_h", (T, self.ff), rt.act_dtype, first="tokens")
            ops.linear(x, self.w_up, h, status=rt.status)
            ops.activation(h, h, self.act)
            ops.linear(h, self.w_down, residual, accumulate=True, status=rt.status)
            return
        out = self.rt.workspace.get("ffn_out", (x.shape[0], self.hidden), torch.float32, first="tokens")
        self.forward_into(x, out)
        ops.add_scaled(residual, out, scale)

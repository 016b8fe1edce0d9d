"""The gated delta rule with one decay per head and key channel, as a part (mixer "gated_delta_rule").

With h the mixer's input: q, k (kv_heads x dim) and v (heads x vdim) are projections that pass a short causal convolution
per channel and silu; q and k are made unit vectors per head (q also times dim^-1/2); beta = sigmoid(W_b h) per head;
g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias)) per head and key channel.  Value head h (query/key head
h // (heads / kv_heads)) keeps a state S [dim, vdim] per request:

    S <- g * S (row d times g[d]);   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q

Each head's o is divided by its root mean square over vdim, times a weight [vdim] shared by the heads, times
sigmoid(W_g2 (W_g1 h)); then W_o.  The state starts at zero for a new request, is 32-bit and lives in the request's state
slot beside the convolution's last taps-1 inputs; unit norms, beta, decays, the recurrence, the output norm and the gate
are 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import SlotState, WeightSpec


class GatedDeltaRule(Part):
    """params: hidden, heads, kv_heads, dim, vdim, conv (taps), decay_rank and gate_rank (inner sizes of the two-step
    projections), eps (of the output norm), unit_eps (inside the unit norms' root, default 1e-6), names (optional dict of
    tensor names after the prefix).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "A_log": "A_log",
             "norm": "norm", "a1": "a1", "a2": "a2", "dt_bias": "dt_bias", "g1": "g1", "g2": "g2", "o": "o"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.taps = int(p["conv"])
        self.decay_rank = int(p["decay_rank"])
        self.gate_rank = int(p["gate_rank"])
        self.eps = float(p["eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        if self.heads % self.kv_heads:
            raise ValueError(f"delta rule: kv_heads {self.kv_heads} must divide heads {self.heads}")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"delta rule: key size {self.dim} is not supported by the kernel (1 to 256)")
        if not 1 <= self.taps <= 17:
            raise ValueError(f"delta rule: {self.taps} conv taps are not supported by the kernel (1 to 17)")
        self.qk = self.kv_heads * self.dim
        self.vv = self.heads * self.vdim
        self.channels = 2 * self.qk + self.vv
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_low = self.w_a2 = self.w_g2 = self.w_o = None
        self.conv_w = self.A_log = self.dt_bias = self.w_norm = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        return [WeightSpec(n["q"], ((self.qk, H),)), WeightSpec(n["k"], ((self.qk, H),)), WeightSpec(n["v"], ((self.vv, H),)),
                WeightSpec(n["q_conv"], ((self.qk, self.taps),), role="vector", init=("conv_taps",)),
                WeightSpec(n["k_conv"], ((self.qk, self.taps),), role="vector", init=("conv_taps",)),
                WeightSpec(n["v_conv"], ((self.vv, self.taps),), role="vector", init=("conv_taps",)),
                WeightSpec(n["b"], ((self.heads, H),)),
                WeightSpec(n["A_log"], ((self.heads,),), role="vector", init=("uniform", -3.0, 0.0)),
                WeightSpec(n["norm"], ((self.vdim,),), role="vector", init=("norm",)),
                WeightSpec(n["a1"], ((self.decay_rank, H),)), WeightSpec(n["a2"], ((self.heads * self.dim, self.decay_rank),)),
                WeightSpec(n["dt_bias"], ((self.heads * self.dim,),), role="vector", init=("uniform", -4.0, -1.0)),
                WeightSpec(n["g1"], ((self.gate_rank, H),)), WeightSpec(n["g2"], ((self.vv, self.gate_rank),)),
                WeightSpec(n["o"], ((H, self.vv),))]

    def bind(self, tensors):
        n = self.names
        # one 32-bit product [q | k | v | beta] and one product [decay | gate] into the two inner spaces (layout choices)
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["b"]]], dim=0).contiguous()
        low = torch.cat([tensors[n["a1"]], tensors[n["g1"]]], dim=0)
        # the second inner space starts on a 16-byte boundary so that its rows can feed the tensor-core products
        self.g_at = (self.decay_rank + 7) // 8 * 8
        self.w_low = torch.zeros(((self.g_at + self.gate_rank + 7) // 8 * 8, low.shape[1]), dtype=low.dtype, device=low.device)
        self.w_low[:self.decay_rank] = tensors[n["a1"]]
        self.w_low[self.g_at:self.g_at + self.gate_rank] = tensors[n["g1"]]
        self.w_a2, self.w_g2, self.w_o = tensors[n["a2"]], tensors[n["g2"]], tensors[n["o"]]
        self.conv_w = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        self.A_log, self.dt_bias, self.w_norm = tensors[n["A_log"]], tensors[n["dt_bias"]], tensors[n["norm"]]

    def cache_specs(self):
        return (SlotState((self.heads, self.dim, self.vdim)), SlotState((max(self.taps - 1, 1), self.channels)))

    def forward(self, x, batch, caches, residual, accumulate=True):
        st, conv = caches
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        H, D, V = self.heads, self.dim, self.vdim
        # the projections stay 32-bit: what enters the recurrence is rounded nowhere
        proj = ws.get("delta_in", (T, self.channels + H), torch.float32, first="tokens")
        ops.linear(x, self.w_in, proj, status=rt.status)
        low = ws.get("delta_low", (T, self.w_low.shape[0]), rt.act_dtype, first="tokens")
        ops.linear(x, self.w_low, low, status=rt.status)
        a = ws.get("delta_decay", (T, H * D), torch.float32, first="tokens")
        ops.linear(low[:, :self.decay_rank], self.w_a2, a, status=rt.status)
        gate = ws.get("delta_gate", (T, self.vv), torch.float32, first="tokens")
        ops.linear(low[:, self.g_at:self.g_at + self.gate_rank], self.w_g2, gate, status=rt.status)
        qkv = ws.get("delta_qkv", (T, self.channels), torch.float32, first="tokens")
        ops.channel_conv(proj, 0, self.channels, self.taps, self.conv_w, None, conv.state, batch.item_row_start, batch.item_of_token,
                         batch.item_slot, batch.n_items, qkv, rt.status, act="silu")
        beta = ws.get("delta_beta", (T, H), torch.float32, first="tokens")
        ops.delta_prepare(qkv, 0, self.qk, proj, self.channels, a, self.A_log, self.dt_bias, beta, H, self.kv_heads, D,
                          self.unit_eps, float(D) ** -0.5)
        o = ws.get("delta_o", (T, self.vv), torch.float32, first="tokens")
        ops.delta_scan(qkv, 0, self.qk, 2 * self.qk, a, beta, st.state, batch.item_row_start, batch.item_slot, batch.n_items, o,
                       H, self.kv_heads, D, V, rt.status)
        y = ws.get("delta_y", (T, self.vv), rt.act_dtype, first="tokens")
        ops.head_norm_gate(o, self.w_norm, self.eps, gate, y, H, V)
        ops.linear(y, self.w_o, residual, accumulate=accumulate, status=rt.status)

"""A matrix memory with exponential gates (the mLSTM cell of xLSTM), as a part (mixer "matrix_memory").

With q = W_q h * dim^(-1/2), k = W_k h (heads x dim) and v = W_v h (heads x vdim), every head has a log input gate
a = cap * tanh((W_i h + b_i) / cap) and a log forget gate f = log sigmoid(cap * tanh((W_f h + b_f) / cap)), and keeps per
request a matrix S [dim, vdim], a vector n [dim] and a running maximum m (all zero at the start):

    m' = max(f + m, a);   S' = exp(f + m - m') S + exp(a - m') k v^T;   n' = exp(f + m - m') n + exp(a - m') k
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

Each head's o is divided by its root mean square, the heads side by side are multiplied by a weight (heads * vdim) and by
sigmoid(W_g h), and projected by W_o.  The state is 32-bit and lives in the request's state slot; the gates, the
recurrence, the norm and the output gate are 32-bit in both precisions: the one product [q | k | v | g | i | f] is written in
32-bit, so what enters the recurrence is not rounded.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import SlotState, WeightSpec


class MatrixMemory(Part):
    """params: hidden, heads, dim, vdim, gate_cap, eps (of the per-head output norm), names (optional dict of tensor names
    after the prefix: q, k, v, g, o, norm, i, f, i_bias, f_bias).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True
    CHUNK_FROM = 128          # portions from this many tokens on run in chunks side by side
    CHUNK = 64

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.cap = float(p["gate_cap"])
        self.eps = float(p["eps"])
        if not 1 <= self.dim <= 256:
            raise ValueError(f"matrix memory: key size {self.dim} is not supported by the kernel (1 to 256)")
        if not self.cap > 0.0:
            raise ValueError("matrix memory: the gate cap must be positive")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_o = self.w_norm = self.b_i = self.b_f = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        qk, vv = self.heads * self.dim, self.heads * self.vdim
        return [WeightSpec(n["q"], ((qk, H),)), WeightSpec(n["k"], ((qk, H),)), WeightSpec(n["v"], ((vv, H),)),
                WeightSpec(n["g"], ((vv, H),)), WeightSpec(n["o"], ((H, vv),)),
                WeightSpec(n["norm"], ((vv,),), role="vector", init=("norm",)),
                WeightSpec(n["i"], ((self.heads, H),)), WeightSpec(n["f"], ((self.heads, H),)),
                WeightSpec(n["i_bias"], ((self.heads,),), role="vector", init=("uniform", -2.0, 1.0)),
                WeightSpec(n["f_bias"], ((self.heads,),), role="vector", init=("uniform", 1.0, 4.0))]

    def bind(self, tensors):
        n = self.names
        # one fused projection [q | k | v | g | i | f]: a layout choice, the arithmetic is unchanged
        self.w_in = torch.cat([tensors[n[k]] for k in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.w_norm = tensors[n["norm"]]
        self.b_i, self.b_f = tensors[n["i_bias"]], tensors[n["f_bias"]]

    def cache_specs(self):
        vb = ops.mlstm_value_blocks(self.vdim)
        return (SlotState((self.heads, self.dim, self.vdim)), SlotState((self.heads, vb, self.dim)), SlotState((self.heads, vb)))

    # the 32-bit first product may be made by an arrangement that stacks several parts' matrices (SideBySideMixer)
    def wide_input_rows(self) -> int:
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim + 2 * self.heads

    def wide_input_weight(self):
        return self.w_in

    def adopt_wide_input_weight(self, view) -> None:
        self.w_in = view

    def forward(self, x, batch, caches, residual, accumulate=True, projected=None):
        S, n, m = caches
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        H = self.heads
        qk, vv = H * self.dim, H * self.vdim
        # the product stays 32-bit: gates, keys, values and queries enter the recurrence unrounded
        if projected is not None:
            proj = projected
        else:
            proj = ws.get("mlstm_in", (T, self.w_in.shape[0]), torch.float32, first="tokens")
            ops.linear(x, self.w_in, proj, status=rt.status)
        o = ws.get("mlstm_o", (T, vv), torch.float32, first="tokens")
        chunk, scratch = 0, None
        if batch.max_tokens_per_item >= self.CHUNK_FROM:
            # long portions: chunks of rows side by side.  A chunk's CTA walks its rows one after the other, so the chunks are
            # halved while they would leave SMs without a CTA (with several CTAs on an SM the walks share its issue slots
            # and shorter chunks only add to the scan: 123 against 134 us per layer at 2,048 tokens, 8 heads); the length
            # follows the step's totals alone (tokens, requests), which are part of its shape
            vb = ops.mlstm_value_blocks(self.vdim)
            chunk = self.CHUNK
            per_cta = 128 if self.dim <= 64 else 64          # value columns a CTA of the recurrence covers
            if (T // chunk + batch.n_items) * H * -(-self.vdim // per_cta) < ops.sm_count():
                chunk //= 2
            most = T // chunk + batch.n_items
            scratch = (ws.get("mlstm_chunk_S", (most * H * self.dim * self.vdim,), torch.float32),
                       ws.get("mlstm_chunk_n", (most * H * vb * self.dim,), torch.float32),
                       ws.get("mlstm_chunk_mb", (most * H * vb * 3,), torch.float32))
        ops.mlstm_scan(proj, 0, qk, 2 * qk, 2 * qk + 2 * vv, 2 * qk + 2 * vv + H, self.b_i, self.b_f, self.cap, self.dim ** -0.5,
                       S.state, n.state, m.state, batch.item_row_start, batch.item_slot, batch.n_items, o, H, self.dim, self.vdim,
                       rt.status, chunk=chunk, scratch=scratch)
        y = ws.get("mlstm_y", (T, vv), rt.act_dtype, first="tokens")
        ops.head_norm_gate(o, self.w_norm, self.eps, proj[:, 2 * qk + vv:2 * qk + 2 * vv], y, H, self.vdim)
        ops.linear(y, self.w_o, residual, accumulate=accumulate, status=rt.status)

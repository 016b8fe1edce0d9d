"""RMS norm as a part: y = x * 1/sqrt(mean(x^2) + eps) * w, sums in 32-bit
(imparo-cpu/src/ops.rs:6-22).  With `offset` the stored tensor is the weight's distance from that number
(offset 1: the file keeps w - 1, y = x / rms * (1 + stored)).  With `streams` the input rows hold n copies of the
stream side by side and the norm reads their weighted sum."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class RMSNorm(Part):
    """params: width, eps, name (tensor name after the prefix, e.g. "operator_norm.weight"), offset (default 0: the
    stored tensor is the weight; c: the weight is c + the stored tensor, added once in 32-bit when the tensor is bound),
    streams (default 1; n > 1: x is [tokens, n * width] and the norm reads u = sum_s a[s] x_s), stream_weights (the tensor
    name of a [n], after the prefix; absent: every copy counts once)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = prefix + params["name"]
        self.offset = float(params.get("offset", 0.0))
        self.streams = int(params.get("streams") or 1)
        self.by_copies = params.get("streams") is not None       # the stream is laid out in copies (even one): the copies' kernel reads it
        self.coef_name = prefix + params["stream_weights"] if params.get("stream_weights") else None
        self.weight: Optional[torch.Tensor] = None
        self.coef: Optional[torch.Tensor] = None

    def weight_specs(self):
        init = ("norm",) if self.offset == 0.0 else ("norm_offset", self.offset)
        specs = [WeightSpec(self.name, ((self.width,),), role="vector", init=init)]
        if self.coef_name is not None:
            specs.append(WeightSpec(self.coef_name, ((self.streams,),), role="vector", init=("uniform", 0.2, 0.6)))
        return specs

    def bind(self, tensors):
        self.weight = tensors[self.name]
        if self.offset != 0.0:
            self.weight = (self.weight.float() + self.offset).contiguous()
        if self.coef_name is not None:
            self.coef = tensors[self.coef_name]

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                tag: str = "normed") -> torch.Tensor:
        """x: 32-bit [tokens, width].  rows (int32, device) picks input rows; n_rows is how
        many of them.  Returns activations in the path's dtype."""
        n = x.shape[0] if rows is None else int(n_rows if n_rows is not None else rows.numel())
        out = self.rt.workspace.get(tag, (n, self.width), self.rt.act_dtype, first="tokens" if rows is None else "rows")
        if self.by_copies:
            ops.streams_norm(x, self.streams, self.coef, self.weight, self.eps, out, rows)
        else:
            ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

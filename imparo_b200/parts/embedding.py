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
    """params: vocab, width, name, scale (optional factor on the rows, applied in 32-bit), copies (optional n > 1: the
    stream holds n copies of every row side by side, [tokens, n * width], for arrangements that keep several), position_table
    (optional {"name": tensor, "rows": n}: a learned vector per position, [n, width], added unscaled to the scaled row; a
    token at a position beyond the table is reported through the status word)."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab"])
        self.width = int(params["width"])
        self.name = prefix + params["name"]
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0
        self.copies = int(params.get("copies") or 1)
        pos = params.get("position_table")
        self.pos_name = prefix + pos["name"] if pos else None
        self.pos_rows = int(pos["rows"]) if pos else 0
        self.table = self.pos_table = None

    def weight_specs(self):
        specs = [WeightSpec(self.name, ((self.vocab, self.width),))]
        if self.pos_name is not None:
            specs.append(WeightSpec(self.pos_name, ((self.pos_rows, self.width),)))
        return specs

    def bind(self, tensors):
        self.table = tensors[self.name]
        if self.pos_name is not None:
            self.pos_table = tensors[self.pos_name].contiguous()

    def forward(self, batch) -> torch.Tensor:
        """batch: the step's batch (token_ids, positions, item_of_token, ... on the device).  This part reads
        the token ids only; an embedding that adds learned positions or segment rows reads the rest."""
        out = self.rt.workspace.get("residual", (batch.n_tokens, self.copies * self.width), torch.float32, first="tokens")
        if self.scale != 1.0 or self.copies != 1 or self.pos_table is not None:
            ops.embed_copies(self.table, batch.token_ids, out, self.rt.status, scale=self.scale, copies=self.copies,
                             pos_table=self.pos_table, positions=batch.positions if self.pos_table is not None else None)
        else:
            ops.embed_gather(self.table, batch.token_ids, out, self.rt.status)
        return out


class LinearHead(Part):
    """params: vocab, width, name (the table's own tensor, or the embedding's when tied), scale (optional factor on
    the logits, applied in 32-bit before any cap), softcap (optional c > 0: logits become c * tanh(logits / c))."""

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        self.vocab = int(params["vocab"])
        self.width = int(params["width"])
        self.name = prefix + params["name"]
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name, ((self.vocab, self.width),))]

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.rt.workspace.get("logits", (h.shape[0], self.vocab), torch.float32, first="rows")
        ops.linear(h, self.table, logits, status=self.rt.status)
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits

"""A routed feed-forward (mixture of experts) as a part (feed_forward "routed_experts").

Router logits z = W_r h in 32-bit; scores sigmoid(z) (or a softmax over the experts); each row uses the `top` experts
with the largest scores, weighted by those scores (optionally renormalised to sum 1, and times a factor).  The experts may
form equal groups of neighbours of which only the groups with the best single scores can be chosen from.  An expert is a
gated feed-forward without biases, W_down act(W_gate u, W_up u) with act(g, u) = silu(g) u, or, with a limit c,
g' = min(g, c), u' = clamp(u, -c, c): g' sigmoid(1.702 g') (u' + 1); the weight multiplies the expert's input u = w h
(weight_on "input") or its output (weight_on "output").  The row's result is the sum over its experts, in the order of
their scores.  A shared expert of the same form runs for every row and is added.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import WeightSpec


class RoutedExperts(Part):
    """params: hidden, ff (per expert), experts, top, score ("sigmoid" | "softmax", default sigmoid), renormalise (bool,
    default False), weight_on ("input" | "output", default "output"), names (optional: router, and gate / up / down as
    patterns with {e} for the expert's number), groups and keep (the experts in `groups` equal groups of neighbours, a
    group's score its largest; only the `keep` best groups' experts can be chosen; default: no groups), renorm_eps (added
    to the sum the chosen scores are divided by), weight_scale (a factor on the weights), act ("silu" | "clamped_swish")
    with limit, shared ({"ff", "limit", "names": {gate, up, down}}: an expert of the same form that every row uses with
    weight 1; with the experts' own size and limit it is stacked behind them and runs in the same launches).

    forward(x, batch, residual, accumulate=False) overwrites `residual` (a float32 [rows, hidden] buffer); with
    accumulate=True the result is added into it (through a buffer of the part's own), times `scale`."""
    takes_scale = True
    GROUP_FROM = 65           # steps with at least this many (row, expert) pairs run sorted by expert, in tiles
    TILES_FROM = 256          # and from this many on (bfloat16, aligned sizes) on the tensor-memory product, tiles of 128 rows

    NAMES = {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.ff = int(p["ff"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.score = p.get("score", "sigmoid")
        self.renormalise = bool(p.get("renormalise", False))
        self.weight_on = p.get("weight_on", "output")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed experts: unknown score '{self.score}' (sigmoid, softmax)")
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: weight_on is 'input' or 'output', found '{self.weight_on}'")
        if not 1 <= self.top <= min(self.experts, 32):
            raise ValueError(f"routed experts: top {self.top} must be between 1 and min(experts, 32) = {min(self.experts, 32)}")
        self.groups = int(p.get("groups") or 1)
        self.keep = int(p.get("keep") or self.groups)
        if self.experts % self.groups or not 1 <= self.keep <= self.groups or self.keep * (self.experts // self.groups) < self.top:
            raise ValueError(f"routed experts: {self.groups} groups (keep {self.keep}) do not fit {self.experts} experts, top {self.top}")
        self.renorm_eps = float(p.get("renorm_eps", 0.0))
        self.weight_scale = float(p.get("weight_scale", 1.0))
        self.act = p.get("act", "silu")
        self.limit = float(p.get("limit", 0.0))
        if self.act not in ("silu", "clamped_swish"):
            raise ValueError(f"routed experts: unknown activation '{self.act}' (silu, clamped_swish)")
        self.shared = dict(p["shared"]) if p.get("shared") else None
        # a shared expert of the experts' own form is one more expert that every row chooses with weight 1
        self.shared_stacked = (self.shared is not None and int(self.shared["ff"]) == self.ff and self.weight_on == "output"
                               and float(self.shared.get("limit", self.limit)) == self.limit)
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_router = self.w_gu = self.w_down = None
        self.w_shared_gu = self.w_shared_down = None

    def weight_specs(self):
        n, H, F = self.names, self.hidden, self.ff
        specs = [WeightSpec(n["router"], ((self.experts, H),), role="vector", init=("normal", 0.5))]
        for e in range(self.experts):
            specs += [WeightSpec(n["gate"].format(e=e), ((F, H),)), WeightSpec(n["up"].format(e=e), ((F, H),)),
                      WeightSpec(n["down"].format(e=e), ((H, F),))]
        if self.shared is not None:
            sn, sf = self._shared_names(), int(self.shared["ff"])
            specs += [WeightSpec(sn["gate"], ((sf, H),)), WeightSpec(sn["up"], ((sf, H),)), WeightSpec(sn["down"], ((H, sf),))]
        return specs

    def _shared_names(self):
        names = {"gate": "shared.gate", "up": "shared.up", "down": "shared.down", **self.shared.get("names", {})}
        return {k: self.prefix + v for k, v in names.items()}

    def bind(self, tensors):
        n = self.names
        self.w_router = tensors[n["router"]]
        # For bfloat16 rows the router's logits come from the tensor-core product: the 32-bit matrix cut into three
        # bfloat16 pieces that add up to it to its last bit, so every product is exact and the sums are 32-bit.
        self.w_router_pieces = None
        if self.rt.act_dtype == torch.bfloat16:
            rest, pieces = self.w_router.float(), []
            for _ in range(3):
                piece = rest.to(torch.bfloat16)
                pieces.append(piece)
                rest = rest - piece.float()
                if not bool(rest.any()):          # a router stored in bfloat16 is its own first piece
                    break
            self.router_parts = len(pieces)
            self.w_router_pieces = torch.cat(pieces, dim=0).contiguous()
        # experts stacked: [experts, 2 ff, hidden] = [gate; up] and [experts, hidden, ff]
        gu = [torch.cat([tensors[n["gate"].format(e=e)], tensors[n["up"].format(e=e)]], dim=0) for e in range(self.experts)]
        down = [tensors[n["down"].format(e=e)] for e in range(self.experts)]
        if self.shared is not None:
            sn = self._shared_names()
            s_gu, s_down = torch.cat([tensors[sn["gate"]], tensors[sn["up"]]], dim=0), tensors[sn["down"]]
            if self.shared_stacked:
                gu.append(s_gu)
                down.append(s_down)
            else:
                self.w_shared_gu, self.w_shared_down = s_gu.unsqueeze(0).contiguous(), s_down.unsqueeze(0).contiguous()
        self.w_gu = torch.stack(gu).contiguous()
        self.w_down = torch.stack(down).contiguous()

    def _experts(self, x, w_gu, w_down, ids, wts, top, weight_input, limit, out, tag):
        """One pass of the expert kernels: pair by pair, sorted into small tiles, or on the tensor-memory product."""
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        n_experts, ff = w_gu.shape[0], w_gu.shape[1] // 2
        pairs = T * top
        if pairs >= self.TILES_FROM and ops.moe_tiles_usable(x, w_gu):
            # many rows in bfloat16: sorted into tiles of 128 rows per expert, both products on the tensor-memory kernel
            rows = (pairs // 128 + n_experts) * 128
            ops.moe_experts_tiles(x, w_gu, w_down, ids, wts, top, weight_input,
                                  ws.get(tag + "sorted_in", (rows, self.hidden), rt.act_dtype),
                                  ws.get(tag + "sorted_mid", (rows, ff), rt.act_dtype),
                                  ws.get(tag + "sorted_out", (rows, self.hidden), torch.float32),
                                  ws.get(tag + "tile_plan", (pairs + rows // 128,), torch.int32), out, rt.status,
                                  act=self.act, limit=limit)
            return
        mid = ws.get(tag + "mid", (pairs, ff), rt.act_dtype, first="tokens")
        scratch = None
        if pairs >= self.GROUP_FROM:
            scratch = (ws.get(tag + "pair_out", (pairs, self.hidden), torch.float32, first="tokens"),
                       ws.get(tag + "plan", (pairs + n_experts + 2 + 3 * (pairs // 32 + n_experts),), torch.int32))
        ops.moe_experts(x, w_gu, w_down, ids, wts, top, weight_input, mid, out, scratch=scratch, act=self.act, limit=limit)

    def forward(self, x, batch, residual, accumulate=False, scale: float = 1.0):
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        always = 1 if self.shared_stacked else 0
        chosen = self.top + always
        ids = ws.get("moe_ids", (T, chosen), torch.int32, first="tokens")
        wts = ws.get("moe_wts", (T, chosen), torch.float32, first="tokens")
        how = dict(softmax=self.score == "softmax", renormalise=self.renormalise, groups=self.groups, keep=self.keep,
                   renorm_eps=self.renorm_eps, weight_scale=self.weight_scale, always=always)
        if self.w_router_pieces is not None and x.dtype == torch.bfloat16:
            logits = ws.get("moe_logits", (T, self.router_parts * self.experts), torch.float32, first="tokens")
            ops.linear(x, self.w_router_pieces, logits, status=rt.status)
            ops.moe_pick(logits, self.experts, self.router_parts, self.top, ids, wts, **how)
        else:
            ops.moe_route(x, self.w_router, self.top, ids, wts, logits=ws.get("moe_logits", (T, self.experts), torch.float32, first="tokens"),
                          **how)
        out = residual if not accumulate else ws.get("moe_out", tuple(residual.shape), torch.float32, first="tokens")
        self._experts(x, self.w_gu, self.w_down, ids, wts, chosen, self.weight_on == "input", self.limit, out, "moe_")
        if self.w_shared_gu is not None:
            # a shared expert of another size: the same kernels with one expert that every row chooses with weight 1
            one_i = ws.get("moe_shared_ids", (T, 1), torch.int32, first="tokens")
            one_w = ws.get("moe_shared_wts", (T, 1), torch.float32, first="tokens")
            one_i.zero_()
            one_w.fill_(1.0)
            extra = ws.get("moe_shared_out", tuple(residual.shape), torch.float32, first="tokens")
            self._experts(x, self.w_shared_gu, self.w_shared_down, one_i, one_w, 1, False,
                          float(self.shared.get("limit", self.limit)), extra, "moe_shared_")
            ops.add_scaled(out, extra, 1.0)
        if accumulate:
            ops.add_scaled(residual, out, scale)
        elif scale != 1.0:
            ops.scale_rows(out, scale)

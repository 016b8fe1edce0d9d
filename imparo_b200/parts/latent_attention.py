"""Attention whose keys and values are made from one small latent vector per token, as a part (mixer "latent_attention").

With h the mixer's input:  cq = rms(W_dq h) * n_q,  q = W_uq cq  (heads x dim);  c = rms(W_dkv h) * n_kv  (rank);  per head
k = U_k c, v = U_v c;  score = scale * q . k;  causal;  optionally one more term exp(sink_h) in the softmax's denominator
that has no value;  the heads' outputs times sigmoid(W_g h) when gated;  W_o.  There is no position encoding.

Two variants, by parameters: the queries may come straight from the input (no query latent: q = W_q h), and beside the
latent there may be a ROTATED part: every head's query is [dim plain | rot_dim rotated], W_dkv h has kv_rank + rot_dim rows
of which the last rot_dim, not normed, are one key part kr that all heads share; the rotated parts of q and kr are turned
by the position (half-split pairs) and score = scale * (q_plain . k + q_rot . kr).  The cached row is then [c | kr], and
the latent-space query [U_k^T q_plain | q_rot], so the attention over the cached rows is unchanged; of its result only
the first kv_rank entries (the weighted sum of the latents) go on to U_v.  The output gate is a number per output element
or one per head.

Only c (and kr) is cached (one row per position that is key and value at once, PagedKV.values_are_keys).  Because
q . (U_k c) = (U_k^T q) . c and sum_j p_j U_v c_j = U_v sum_j p_j c_j, the queries are taken into the latent space before
the attention and its result out of it afterwards; the attention itself sees one key/value head of size rank that all
heads share, over prompts and decoded tokens alike.  Norms, scores, the sink and the softmax are 32-bit in both precisions.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part
from .spec import PagedKV, WeightSpec


class LatentAttention(Part):
    """params: hidden, heads, dim, vdim, q_rank (None: queries straight from the input, tensor "q"), kv_rank, scale, eps (of
    the latent norms), sink (bool: a learned number per head in the softmax's denominator), gate (False; True: output gate
    sigmoid(W_g h) per output element; "head": one gate per head), rot_dim (default 0: rotated dimensions per head and of
    the shared key part; needs q_rank None), position (PartSpec of the rotation over the rot_dim part), names (optional dict
    of tensor names after the prefix).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True

    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "sink": "sink", "g": "g", "o": "o", "q": "q"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else None
        self.kv_rank = int(p["kv_rank"])
        self.rot_dim = int(p.get("rot_dim") or 0)
        self.row = self.kv_rank + self.rot_dim          # what the cache keeps per position
        if self.rot_dim and self.q_rank is not None:
            raise ValueError("latent attention: a rotated part needs queries straight from the input (q_rank None)")
        from .base import make_part
        from .spec import PartSpec
        self.position = make_part("position", p.get("position", PartSpec("none")), prefix, rt)
        if self.position.interleaved or self.position.magnitude != 1.0:
            raise ValueError("latent attention: the rotated part takes a half-split rotation without a magnitude")
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.sink = bool(p.get("sink", False))
        self.gate = bool(p.get("gate", False))
        self.gate_per_head = p.get("gate") == "head"
        if not 1 <= self.row <= 640:
            raise ValueError(f"latent attention: cached row size {self.row} is not supported by the kernel (1 to 640)")
        if max(self.dim, self.kv_rank) > 1536:
            raise ValueError("latent attention: head and latent sizes up to 1536")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_uq = self.w_ukT = self.w_uv = self.w_o = self.n_q = self.n_kv = self.sinks = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        if self.q_rank is not None:
            specs = [WeightSpec(n["dq"], ((self.q_rank, H),)), WeightSpec(n["dq_norm"], ((self.q_rank,),), role="vector", init=("norm",)),
                     WeightSpec(n["uq"], ((hd, self.q_rank),))]
        else:
            specs = [WeightSpec(n["q"], ((self.heads * (self.dim + self.rot_dim), H),))]
        specs += [WeightSpec(n["dkv"], ((self.row, H),)),
                  WeightSpec(n["dkv_norm"], ((self.kv_rank,),), role="vector", init=("norm",)),
                  WeightSpec(n["uk"], ((hd, self.kv_rank),)), WeightSpec(n["uv"], ((hv, self.kv_rank),)),
                  WeightSpec(n["o"], ((H, hv),))]
        if self.sink:
            specs.append(WeightSpec(n["sink"], ((self.heads,),), role="vector", init=("uniform", -1.0, 2.0)))
        if self.gate:
            specs.append(WeightSpec(n["g"], ((self.heads if self.gate_per_head else hv, H),)))
        return specs + self.position.weight_specs()

    def bind(self, tensors):
        n = self.names
        # one product for everything that reads the input: [query latent (or the queries) | key/value latent (| key part) | gate]
        first = tensors[n["dq"]] if self.q_rank is not None else tensors[n["q"]]
        self.w_in = torch.cat([first, tensors[n["dkv"]]] + ([tensors[n["g"]]] if self.gate else []), dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.n_kv = tensors[n["dkv_norm"]]
        if self.q_rank is not None:
            self.w_uq, self.n_q = tensors[n["uq"]], tensors[n["dq_norm"]]
        self.position.bind(tensors)
        # per head: U_k^T [rank, dim] takes a query into the latent space, U_v [vdim, rank] takes the result out of it
        self.w_ukT = tensors[n["uk"]].view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.sinks = tensors[n["sink"]] if self.sink else None

    def cache_specs(self):
        return (PagedKV(1, self.row, None, None, values_are_keys=True),)

    def _partials_room(self, upper_context: int, groups: int) -> int:
        """Partial results (per head) that the split-key kernel leaves for this engine's largest step of one-token rows at
        the longest context it allows: the scratch is made for that at once, so it does not move (and void the captured
        graphs) when a few more requests decode."""
        most = self.rt.workspace.most
        rows = most.get("rows", 0)
        if not rows:
            return 0
        context = max(int(upper_context), min(most.get("context", 0), 1 << 17))
        return (8 * ops.sm_count() + rows * groups * (1 + -(-context // 512))) * -(-self.heads // groups)

    def forward(self, x, batch, caches, residual, accumulate=True):
        kv = caches[0]
        rt, T = self.rt, x.shape[0]
        ws = rt.workspace
        H, R = self.heads, self.row
        hv = H * self.vdim
        # the product stays 32-bit: the latents are normed (and the rotated parts turned) from unrounded rows, the gate's
        # sigmoid reads them too
        proj = ws.get("latent_in", (T, self.w_in.shape[0]), torch.float32, first="tokens")
        ops.linear(x, self.w_in, proj, status=rt.status)
        table = batch.tables[kv.group]
        q = ws.get("latent_q", (T, H * self.dim), rt.act_dtype, first="tokens")
        ql = ws.get("latent_ql", (T, H * R), rt.act_dtype, first="tokens")
        if self.q_rank is not None:
            cq = ws.get("latent_cq", (T, self.q_rank), rt.act_dtype, first="tokens")
            ops.latent_norm_store(proj, 0, self.q_rank, self.q_rank, R, self.n_q, self.n_kv, self.eps, batch.positions,
                                  batch.item_of_token, cq, kv.k, table, kv.page_size, kv.n_pages, rt.status)
            ops.linear(cq, self.w_uq, q, status=rt.status)
            gate_off = self.q_rank + R
        else:
            rot = self.position.rotary() if self.rot_dim else None
            inv_freq, n_rot = rot if rot is not None else (None, 0)
            ops.latent_rot_store(proj, H, self.dim, self.rot_dim, self.kv_rank, self.n_kv, self.eps, inv_freq, n_rot,
                                 batch.positions, batch.item_of_token, q, ql, kv.k, table, kv.page_size, kv.n_pages, rt.status)
            gate_off = H * (self.dim + self.rot_dim) + R
        ops.heads_linear(q, self.w_ukT, ql, out_head=R)
        ol = ws.get("latent_ol", (T, H * R), rt.act_dtype, first="tokens")
        done = False
        if rt.act_dtype == torch.bfloat16 and R in (64, 128) and T <= 65535:
            # latents of a tensor-core head size: prompt portions on the tcgen05 kernel (a tile is 128 / heads tokens times all
            # heads over the one cached row per position), rows of one token (and portions too short for a tile, or pages that
            # kernel does not take) on the split-key kernel with the heads in groups of at most 8
            n1 = getattr(batch, "n_single", 0)            # decode rows come first when the step also holds portions
            first_split = T
            if batch.max_tokens_per_item >= 8:
                a = n1 if 0 < n1 < batch.n_items else 0
                if ops.attention_prefill(ql, kv.k, kv.k, batch.item_row_start[a:], batch.item_start_pos[a:], batch.n_items - a,
                                         table[a:], kv.page_size, kv.n_pages, None, self.scale, ol, H, 1, R, rt.status,
                                         sink_values=self.sinks, max_group=128):
                    first_split = a
            done = first_split == 0
            if first_split:
                n = first_split
                groups = ops.head_groups(H, 1)
                upper = table.shape[1] * kv.page_size
                chunk, n_splits = ops.split_plan(n, groups, upper)
                room = self._partials_room(upper, groups)
                part_acc = ws.get("latent_part_acc", (n * H * n_splits * R,), torch.float32, reserve=room * R)
                part_ml = ws.get("latent_part_ml", (n * H * n_splits * 2,), torch.float32, reserve=room * 2)
                done = ops.paged_attention_split_shared(ql[:n], kv.k, kv.k, batch.positions[:n], batch.item_of_token[:n], table,
                                                        kv.page_size, kv.n_pages, None, self.scale, ol[:n], part_acc, part_ml,
                                                        chunk, n_splits, H, 1, R, rt.status, sink_values=self.sinks)
        if not done:
            ops.attention_any(ql, kv.k, kv.k, batch.positions, batch.item_of_token, table, kv.page_size, kv.n_pages, None,
                              self.scale, self.sink, ol, H, 1, R, R, rt.status, sink_values=self.sinks)
        o = ws.get("latent_o", (T, hv), rt.act_dtype, first="tokens")
        ops.heads_linear(ol, self.w_uv, o, gate=proj[:, gate_off:] if self.gate else None, x_head=R)
        ops.linear(o, self.w_o, residual, accumulate=accumulate, status=rt.status)

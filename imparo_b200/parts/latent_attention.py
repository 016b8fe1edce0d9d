"""Attention whose keys and values are made from one small latent vector per token, as a part (mixer "latent_attention").

With h the mixer's input:  cq = rms(W_dq h) * n_q,  q = W_uq cq  (heads x dim);  c = rms(W_dkv h) * n_kv  (rank);  per head
k = U_k c, v = U_v c;  score = scale * q . k;  causal;  optionally one more term exp(sink_h) in the softmax's denominator
that has no value;  the heads' outputs times sigmoid(W_g h) when gated;  W_o.  There is no position encoding.

Only c is cached (one row per position that is key and value at once, PagedKV.values_are_keys).  Because
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
    """params: hidden, heads, dim, vdim, q_rank, kv_rank, scale, eps (of the two latent norms), sink (bool: a learned
    number per head in the softmax's denominator), gate (bool: output gate sigmoid(W_g h)), names (optional dict of tensor
    names after the prefix).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer)."""
    adds_with_linear = True

    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "sink": "sink", "g": "g", "o": "o"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.q_rank = int(p["q_rank"])
        self.kv_rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.sink = bool(p.get("sink", False))
        self.gate = bool(p.get("gate", False))
        if not 1 <= self.kv_rank <= 512:
            raise ValueError(f"latent attention: latent size {self.kv_rank} is not supported by the kernel (1 to 512)")
        if max(self.dim, self.kv_rank) > 1536:
            raise ValueError("latent attention: head and latent sizes up to 1536")
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.w_in = self.w_uq = self.w_ukT = self.w_uv = self.w_o = self.n_q = self.n_kv = self.sinks = None

    def weight_specs(self):
        n, H = self.names, self.hidden
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        specs = [WeightSpec(n["dq"], ((self.q_rank, H),)), WeightSpec(n["dq_norm"], ((self.q_rank,),), role="vector", init=("norm",)),
                 WeightSpec(n["uq"], ((hd, self.q_rank),)), WeightSpec(n["dkv"], ((self.kv_rank, H),)),
                 WeightSpec(n["dkv_norm"], ((self.kv_rank,),), role="vector", init=("norm",)),
                 WeightSpec(n["uk"], ((hd, self.kv_rank),)), WeightSpec(n["uv"], ((hv, self.kv_rank),)),
                 WeightSpec(n["o"], ((H, hv),))]
        if self.sink:
            specs.append(WeightSpec(n["sink"], ((self.heads,),), role="vector", init=("uniform", -1.0, 2.0)))
        if self.gate:
            specs.append(WeightSpec(n["g"], ((hv, H),)))
        return specs

    def bind(self, tensors):
        n = self.names
        # one product for everything that reads the input: [query latent | key/value latent | gate]
        self.w_in = torch.cat([tensors[n["dq"]], tensors[n["dkv"]]] + ([tensors[n["g"]]] if self.gate else []), dim=0).contiguous()
        self.w_uq, self.w_o = tensors[n["uq"]], tensors[n["o"]]
        self.n_q, self.n_kv = tensors[n["dq_norm"]], tensors[n["dkv_norm"]]
        # per head: U_k^T [rank, dim] takes a query into the latent space, U_v [vdim, rank] takes the result out of it
        self.w_ukT = tensors[n["uk"]].view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.sinks = tensors[n["sink"]] if self.sink else None

    def cache_specs(self):
        return (PagedKV(1, self.kv_rank, None, None, values_are_keys=True),)

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
        H, R = self.heads, self.kv_rank
        hv = H * self.vdim
        # the product stays 32-bit: both latents are normed from unrounded rows, the gate's sigmoid reads them too
        proj = ws.get("latent_in", (T, self.w_in.shape[0]), torch.float32, first="tokens")
        ops.linear(x, self.w_in, proj, status=rt.status)
        cq = ws.get("latent_cq", (T, self.q_rank), rt.act_dtype, first="tokens")
        table = batch.tables[kv.group]
        ops.latent_norm_store(proj, 0, self.q_rank, self.q_rank, R, self.n_q, self.n_kv, self.eps, batch.positions,
                              batch.item_of_token, cq, kv.k, table, kv.page_size, kv.n_pages, rt.status)
        q = ws.get("latent_q", (T, H * self.dim), rt.act_dtype, first="tokens")
        ops.linear(cq, self.w_uq, q, status=rt.status)
        ql = ws.get("latent_ql", (T, H * R), rt.act_dtype, first="tokens")
        ops.heads_linear(q, self.w_ukT, ql)
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
        ops.heads_linear(ol, self.w_uv, o, gate=proj[:, self.q_rank + R:] if self.gate else None)
        ops.linear(o, self.w_o, residual, accumulate=accumulate, status=rt.status)

"""Grouped-query attention over the paged cache, as a part.

q/k/v projections, per-head RMS norm of q and k, position encoding, cache write,
causal attention scaled by 1/sqrt(head), output projection
(imparo-model/src/lfm2/workflow_cpu.rs:203-250; imparo-model/src/cpu_support.rs:361-445).
A window keeps only keys pos+1-window..pos (cpu_support.rs:387-388,423).  The part knows
heads, groups, head size, eps, window and its position part; nothing of the model.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import Part, make_part
from .spec import PagedKV, PartSpec, SlotState, WeightSpec


class AttentionMixer(Part):
    """params: hidden, n_heads, n_kv_heads, head_dim, eps, window (None or int), position
    (PartSpec), qk_norm (bool, default True: per-head RMS norm of q and k with a weight each; False: none, and
    no norm tensors are declared), bias (bool, default False: True declares optional q/k/v/out biases, used
    when the file carries them), names (optional dict of tensor names), v_head_dim (the value size per head, default
    head_dim), scale (the factor on q.k, default 1/sqrt(head_dim)), sink (bool, default False: the softmax's denominator
    counts one more term of score 0 that has no value, p_j = exp(s_j) / (1 + sum exp(s_j))), softcap (c > 0: the scaled
    score becomes c * tanh(score / c)), unit_norm (bool: after the rotation q and k are divided by their own root mean
    square per head, eps as given, no weight), bias "required" (q/k/v biases that the file must carry, added in 32-bit
    before the rotation), v_share ({"role": "source" | "blend", "lambda": tensor name}: the source layer leaves the values
    it made for the step's rows to later layers of the same step; a blending layer stores (1 - lambda) v + lambda v_source,
    lambda its own scalar tensor), qk_conv ({"taps": n, "q": tensor name, "k": tensor name}: a causal convolution over time on
    every channel of q and of k, taps [channels, n] with the last column on the current token, right after the projection
    and its bias; the last n - 1 projected rows of a request live in its state slot), v_from_k (bool: there is no value
    projection; a key head as it stands before the rotation is also the value head, so the value size is the head size),
    gate (bool: the heads' outputs, side by side, are multiplied element by element with sigmoid(W_g h), W_g the tensor
    "g" [n_heads * v_head_dim, hidden], before the output projection; with the 32-bit head preparation only), o_bias
    "required" (an output bias the file must carry, with the 32-bit head preparation).

    Shapes and variants the specialised kernels do not take (a value size of its own, a sink, a rotation of interleaved
    pairs or with a magnitude, a head size that is no multiple of 16) run on the general pair of kernels
    (ops.qkv_rotate_store, ops.attention_any).

    forward(..., accumulate=False) overwrites `residual` (then any float32 [tokens, hidden] buffer) instead of adding
    into it: a mixer that runs beside others hands its output to whoever combines them."""
    adds_with_linear = True


    NAMES = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
             "o": "self_attn.out_proj.weight", "q_norm": "self_attn.q_layernorm.weight",
             "k_norm": "self_attn.k_layernorm.weight", "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias",
             "v_bias": "self_attn.v_proj.bias", "o_bias": "self_attn.out_proj.bias", "g": "self_attn.gate.weight"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.nh = int(p["n_heads"])
        self.nkv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.sink = bool(p.get("sink", False))
        self.eps = float(p.get("eps", 0.0))
        self.window = int(p["window"]) if p.get("window") else None
        self.qk_norm = bool(p.get("qk_norm", True))
        self.bias = bool(p.get("bias", False))
        if self.nh % self.nkv:
            raise ValueError(f"attention: kv heads {self.nkv} must divide heads {self.nh}")
        if not 1 <= self.hd <= 256 or not 1 <= self.vd <= 256:
            raise ValueError(f"attention: head size {self.hd} / value size {self.vd} is not supported by the kernels (1 to 256)")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.position = make_part("position", p.get("position", PartSpec("none")), prefix, rt)
        # the general kernels take what the specialised ones (per-head norm + half-split rotation, equal sizes,
        # plain softmax) do not
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.unit_norm = bool(p.get("unit_norm", False))
        self.v_share = dict(p["v_share"]) if p.get("v_share") else None
        if self.v_share is not None and self.v_share.get("role") not in ("source", "blend"):
            raise ValueError("attention: v_share role must be 'source' or 'blend'")
        self.bias_required = p.get("bias") == "required"
        self.qk_conv = dict(p["qk_conv"]) if p.get("qk_conv") else None
        self.v_from_k = bool(p.get("v_from_k", False))
        self.gate = bool(p.get("gate", False))
        self.o_bias_required = p.get("o_bias") == "required"
        if self.v_from_k and (self.vd != self.hd or self.v_share is not None):
            raise ValueError("attention: keys that are their own values need value size = head size and no shared values")
        if self.qk_conv is not None and not 1 <= int(self.qk_conv["taps"]) <= 17:
            raise ValueError(f"attention: {self.qk_conv['taps']} conv taps are not supported by the kernel (1 to 17)")
        # whole heads in 32-bit before anything is rounded: biases, convolution, rotation, the norm without a weight, shared values
        self.prepared = (self.unit_norm or self.v_share is not None or self.bias_required or self.qk_conv is not None
                         or self.v_from_k or self.gate or self.o_bias_required)
        self.general = (self.sink or self.vd != self.hd or self.hd % 16 != 0 or self.position.interleaved
                        or self.position.magnitude != 1.0 or self.prepared or self.softcap > 0.0)
        if self.prepared and (self.qk_norm or self.position.interleaved or self.position.magnitude != 1.0):
            raise ValueError("attention: the 32-bit head preparation (unit_norm, v_share, required biases) takes a half-split "
                             "rotation and no weighted q/k norms")
        if self.general and not self.prepared and (self.qk_norm or self.bias):
            raise ValueError("attention: per-head q/k norms and biases are not available together with a sink, a value size "
                             "of its own, an interleaved or scaled rotation, or a head size that is no multiple of 16")
        self.v_lambda = None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None

    def weight_specs(self):
        n, H, hd, vd = self.names, self.hidden, self.hd, self.vd
        specs = [WeightSpec(n["q"], ((self.nh * hd, H),)), WeightSpec(n["k"], ((self.nkv * hd, H),)),
                 WeightSpec(n["v"], ((self.nkv * vd, H),)), WeightSpec(n["o"], ((H, self.nh * vd),))]
        if self.v_from_k:
            del specs[2]
        if self.qk_conv is not None:
            taps = int(self.qk_conv["taps"])
            specs += [WeightSpec(self.prefix + self.qk_conv["q"], ((self.nh * hd, taps),), role="vector", init=("conv_taps",)),
                      WeightSpec(self.prefix + self.qk_conv["k"], ((self.nkv * hd, taps),), role="vector", init=("conv_taps",))]
        if self.qk_norm:
            specs += [WeightSpec(n["q_norm"], ((hd,),), role="vector", init=("norm",)),
                      WeightSpec(n["k_norm"], ((hd,),), role="vector", init=("norm",))]
        if self.bias_required:
            specs += [WeightSpec(n["q_bias"], ((self.nh * hd,),), role="vector", init=("bias",)),
                      WeightSpec(n["k_bias"], ((self.nkv * hd,),), role="vector", init=("bias",))]
            if not self.v_from_k:
                specs.append(WeightSpec(n["v_bias"], ((self.nkv * vd,),), role="vector", init=("bias",)))
        elif self.bias:
            specs += [WeightSpec(n["q_bias"], ((self.nh * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["k_bias"], ((self.nkv * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["v_bias"], ((self.nkv * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["o_bias"], ((H,),), role="vector", init=("bias",), optional=True)]
        if self.v_share is not None:
            specs.append(WeightSpec(self.prefix + self.v_share["lambda"], ((),), role="vector", init=("uniform", 0.2, 0.8)))
        if self.gate:
            specs.append(WeightSpec(n["g"], ((self.nh * vd, H),)))
        if self.o_bias_required:
            specs.append(WeightSpec(n["o_bias"], ((H,),), role="vector", init=("bias",)))
        return specs + self.position.weight_specs()

    def bind(self, tensors):
        n = self.names
        # one fused projection [q | k | v]: a layout choice, the arithmetic is unchanged
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]]] + ([] if self.v_from_k else [tensors[n["v"]]])
                               + ([tensors[n["g"]]] if self.gate else []), dim=0).contiguous()
        if self.qk_conv is not None:
            self.conv_w = torch.cat([tensors[self.prefix + self.qk_conv["q"]], tensors[self.prefix + self.qk_conv["k"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.q_norm = tensors[n["q_norm"]] if self.qk_norm else None
        self.k_norm = tensors[n["k_norm"]] if self.qk_norm else None
        if self.v_share is not None:
            self.v_lambda = tensors[self.prefix + self.v_share["lambda"]].reshape(1).float().contiguous()
        if self.bias:
            parts = [(tensors.get(n["q_bias"]), self.nh * self.hd), (tensors.get(n["k_bias"]), self.nkv * self.hd)]
            if not self.v_from_k:
                parts.append((tensors.get(n["v_bias"]), self.nkv * self.vd))
            if any(t is not None for t, _ in parts):      # one vector [q | k | v], zeros where the file has none
                ref = self.w_o
                self.b_qkv = torch.cat([t.float() if t is not None else torch.zeros(w, dtype=torch.float32, device=ref.device)
                                        for t, w in parts]).contiguous()
            self.b_o = tensors.get(n["o_bias"])
        if self.o_bias_required:
            self.b_o = tensors[n["o_bias"]]
        self.position.bind(tensors)

    def cache_specs(self):
        paged = PagedKV(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd)
        if self.qk_conv is not None:
            return (paged, SlotState((max(int(self.qk_conv["taps"]) - 1, 1), (self.nh + self.nkv) * self.hd)))
        return (paged,)

    def _partials_room(self, upper_context: int) -> int:
        """Partial results (per head) that the split-key attention of this engine's largest step of one-token rows
        leaves at the longest context the engine allows (or this table width, if longer): with few rows the plan fills about eight CTAs per SM with short chunks, with
        many it cuts 512 keys per chunk.  The scratch is made for that at once, so it does not move (and void the
        captured graphs) each time a few more requests decode."""
        most = self.rt.workspace.most
        rows = most.get("rows", 0)
        if not rows:
            return 0
        context = max(int(upper_context), min(most.get("context", 0), 1 << 17))
        return (8 * ops.sm_count() + rows * self.nkv * (1 + -(-context // 512))) * (self.nh // self.nkv)

    def input_rows(self) -> int:
        return self.nh * self.hd + self.nkv * (self.hd + self.vd) if self.general and not self.prepared else 0

    def input_weight(self):
        return self.w_qkv

    def adopt_input_weight(self, view) -> None:
        self.w_qkv = view

    # with the 32-bit head preparation the first product [q | k | v | gate] is 32-bit: an arrangement that stacks several
    # parts' matrices may make it (SideBySideMixer)
    def wide_input_rows(self) -> int:
        if not self.prepared or self.qk_conv is not None or self.v_share is not None:
            return 0
        return self.nh * self.hd + self.nkv * (self.hd + (0 if self.v_from_k else self.vd)) + (self.nh * self.vd if self.gate else 0)

    def wide_input_weight(self):
        return self.w_qkv

    def adopt_wide_input_weight(self, view) -> None:
        self.w_qkv = view

    def _forward_general(self, x, batch, kv, residual, accumulate, projected=None, conv_state=None):
        """Product (unless the arrangement made it), rotation + cache write, attention, output product."""
        rt, T = self.rt, x.shape[0]
        nh, hd, vd = self.nh, self.hd, self.vd
        nkv = self.nkv if kv.writes else 0
        width = nh * hd + nkv * (hd + (0 if self.v_from_k else vd))
        q = rt.workspace.get("attn_q", (T, nh * hd), rt.act_dtype, first="tokens")
        rot = self.position.rotary()
        inv_freq, n_rot = rot if rot is not None else (None, 0)
        table = batch.tables[kv.group]
        if self.prepared:
            if not kv.writes:
                raise ValueError("attention: a layer that reads another entry's cache cannot prepare heads in 32-bit")
            # the product in 32-bit, so that biases, angles and the norm without a weight see unrounded heads
            wide = width + (nh * vd if self.gate else 0)          # the gate's pre-activations ride along, unrounded
            if projected is not None and projected.dtype == torch.float32 and projected.shape[1] == wide:
                qkv = projected
            else:
                qkv = rt.workspace.get("attn_qkv32", (T, wide), torch.float32, first="tokens")
                ops.linear(x, self.w_qkv[:wide], qkv, status=rt.status)
            gate = qkv[:, width:] if self.gate else None
            if self.gate:
                qkv = qkv[:, :width]
            bias = self.b_qkv
            if self.qk_conv is not None:
                # the convolution reads the biased product (the bias is the projection's) and leaves plain 32-bit rows
                conv = rt.workspace.get("attn_qk_conv32", (T, width), torch.float32, first="tokens")
                ops.channel_conv(qkv, 0, width, int(self.qk_conv["taps"]), self.conv_w, bias, conv_state.state, batch.item_row_start,
                                 batch.item_of_token, batch.item_slot, batch.n_items, conv, rt.status)
                qkv, bias = conv, None
            v_other = v_save = None
            if self.v_share is not None:
                notes = batch.notes
                key = ("v_share", nkv * vd)
                if self.v_share["role"] == "source":
                    v_save = notes[key] = rt.workspace.get("attn_v_shared", (T, nkv * vd), rt.act_dtype, first="tokens")
                else:
                    v_other = notes.get(key)
                    if v_other is None:
                        raise ValueError("attention: a layer blends shared values, but no earlier layer of the step left any")
            ops.qkv_prepare_store(qkv, bias, batch.positions, batch.item_of_token, inv_freq, n_rot,
                                  self.eps if self.unit_norm else None, v_other, self.v_lambda if v_other is not None else None,
                                  v_save, q, kv.k, kv.v, table, kv.page_size, kv.n_pages, nh, nkv, hd, vd, rt.status,
                                  v_from_k=self.v_from_k)
        else:
            if projected is not None and kv.writes:
                qkv = projected
            else:
                qkv = rt.workspace.get("attn_qkv", (T, width), rt.act_dtype, first="tokens")
                ops.linear(x, self.w_qkv[:width], qkv, status=rt.status)
            ops.qkv_rotate_store(qkv, batch.positions, batch.item_of_token, inv_freq, n_rot, self.position.interleaved,
                                 self.position.magnitude, q, kv.k, kv.v, table, kv.page_size, kv.n_pages, nh, nkv, hd, vd, rt.status)
        out = rt.workspace.get("attn_out", (T, nh * vd), rt.act_dtype, first="tokens")
        done = False
        if rt.act_dtype == torch.bfloat16 and hd == vd and hd in (64, 128) and nh // self.nkv <= 8 and T <= 65535:
            # the tensor-core kernels take these sizes (the sink as a flag): prompt portions on the tcgen05 kernel, rows
            # of one token (and portions too short for a tile, or pages it does not take) on the split-key kernel
            n1 = getattr(batch, "n_single", 0)
            first_split = 0              # rows from here on are left to the split-key kernel... none when the portions are done
            if batch.max_tokens_per_item >= 8 and 0 < n1 < batch.n_items:
                done = ops.attention_prefill(q, kv.k, kv.v, batch.item_row_start[n1:], batch.item_start_pos[n1:],
                                             batch.n_items - n1, table[n1:], kv.page_size, kv.n_pages, self.window, self.scale,
                                             out, nh, self.nkv, hd, rt.status, sink=self.sink, softcap=self.softcap)
                first_split = n1 if done else T
            elif batch.max_tokens_per_item >= 8:
                done = ops.attention_prefill(q, kv.k, kv.v, batch.item_row_start, batch.item_start_pos, batch.n_items, table,
                                             kv.page_size, kv.n_pages, self.window, self.scale, out, nh, self.nkv, hd, rt.status,
                                             sink=self.sink, softcap=self.softcap)
                first_split = 0 if done else T
            else:
                first_split = T
            if first_split:
                n = first_split
                chunk, n_splits = ops.split_plan(n, self.nkv, table.shape[1] * kv.page_size)
                room = self._partials_room(table.shape[1] * kv.page_size)
                part_acc = rt.workspace.get("attn_part_acc", (n * nh * n_splits * hd,), torch.float32, reserve=room * hd)
                part_ml = rt.workspace.get("attn_part_ml", (n * nh * n_splits * 2,), torch.float32, reserve=room * 2)
                done = ops.paged_attention_split(q[:n], kv.k, kv.v, batch.positions[:n], batch.item_of_token[:n], table,
                                                 kv.page_size, kv.n_pages, self.window, self.scale, out[:n], part_acc, part_ml,
                                                 chunk, n_splits, nh, self.nkv, hd, rt.status, sink=self.sink, softcap=self.softcap)
        if not done:
            ops.attention_any(q, kv.k, kv.v, batch.positions, batch.item_of_token, table, kv.page_size, kv.n_pages, self.window,
                              self.scale, self.sink, out, nh, self.nkv, hd, vd, rt.status, softcap=self.softcap)
        if self.prepared and self.gate:
            ops.sigmoid_gate(out, gate)
        ops.linear(out, self.w_o, residual, accumulate=accumulate, status=rt.status)
        if self.prepared and self.b_o is not None:
            ops.add_bias(residual, self.b_o)

    def forward(self, x, batch, caches, residual, accumulate=True, projected=None):
        kv = caches[0]
        if self.general:
            return self._forward_general(x, batch, kv, residual, accumulate, projected,
                                         conv_state=caches[1] if self.qk_conv is not None else None)
        if not accumulate:
            residual.zero_()              # the specialised path's products add; the caller's buffer starts from nothing
        rt, T = self.rt, x.shape[0]
        nh, hd = self.nh, self.hd
        nkv = self.nkv if kv.writes else 0          # a reader of another entry's cache computes q only
        width = (nh + 2 * nkv) * hd
        qkv = rt.workspace.get("attn_qkv", (T, width), rt.act_dtype, first="tokens")
        if self.b_qkv is None:
            qkv = ops.linear_unfolded(x, self.w_qkv[:width], qkv, status=rt.status)    # the kernel below can add split partials
        else:
            ops.linear(x, self.w_qkv[:width], qkv, status=rt.status)
            ops.add_bias(qkv, self.b_qkv[:width])
        q = rt.workspace.get("attn_q", (T, nh * hd), rt.act_dtype, first="tokens")
        rot = self.position.rotary()
        table = batch.tables[kv.group]
        inv_freq, n_rot = rot if rot is not None else (None, 0)
        out = rt.workspace.get("attn_out", (T, nh * hd), rt.act_dtype, first="tokens")
        if batch.decode_only and kv.writes and ops.switches().decode_from_qkv and T <= 65535 and isinstance(qkv, ops.PartialProduct):
            # Every request brings one token: the split-key kernel makes its queries from the product's partials
            # itself and writes the new key and value rows, so the q/k kernel does not run (bfloat16, head 64 / 128).
            chunk, n_splits = ops.split_plan(T, self.nkv, table.shape[1] * kv.page_size)
            room = self._partials_room(table.shape[1] * kv.page_size)
            part_acc = rt.workspace.get("attn_part_acc", (T * nh * n_splits * hd,), torch.float32, reserve=room * hd)
            part_ml = rt.workspace.get("attn_part_ml", (T * nh * n_splits * 2,), torch.float32, reserve=room * 2)
            in_product = n_splits <= 64 and ops.fuse_producers()          # the output product combines the partials while it makes its operand
            # every key chunk's CTA makes the group's queries again: worth the q/k kernel it saves up to 16 chunks or so
            # (batch 8: 0.846 against 0.851 ms per step at 2,560 positions, equal at 16 k, 1.44-1.52 against 1.34-1.36 at 32 k)
            if n_splits <= 16 and ops.attention_decode_from_qkv(qkv, batch.positions, batch.item_of_token, self.q_norm, self.k_norm, inv_freq,
                                             n_rot, self.eps, kv.k, kv.v, table, kv.page_size, kv.n_pages, self.window,
                                             self.scale, None if in_product else out, part_acc, part_ml, chunk, n_splits,
                                             nh, self.nkv, hd, rt.status):
                if not in_product or not ops.linear_of_attention_partials(part_acc, part_ml, T, nh, hd, n_splits, self.w_o,
                                                                          residual, rt.status):
                    if in_product:
                        ops.attention_split_combine(part_acc, part_ml, out, T * nh, hd, n_splits)
                    ops.linear(out, self.w_o, residual, accumulate=True, status=rt.status)
                if self.b_o is not None:
                    ops.add_bias(residual, self.b_o)
                return
        ops.qk_norm_rope_store(qkv, batch.positions, batch.item_of_token, self.q_norm, self.k_norm, inv_freq, n_rot,
                               self.eps, q, kv.k, kv.v, table, kv.page_size, kv.n_pages, nh, nkv, hd, rt.status)
        done = False
        n1 = getattr(batch, "n_single", 0)             # decode rows come first when the step also holds portions
        if batch.max_tokens_per_item >= 8 and 0 < n1 < batch.n_items and nh // self.nkv <= 8:
            # Portions beside decode rows: the prompt kernel walks a request's keys tile by tile in one
            # CTA per 128 query rows, which for a single query token is one CTA crawling over the whole
            # context.  So the portions (requests n1 onward) go to the prompt kernel and the decode rows
            # (the first n1 tokens, one per request) to the split-key kernel, which cuts their keys
            # over many CTAs.
            done = ops.attention_prefill(q, kv.k, kv.v, batch.item_row_start[n1:], batch.item_start_pos[n1:],
                                         batch.n_items - n1, table[n1:], kv.page_size, kv.n_pages, self.window, self.scale,
                                         out, nh, self.nkv, hd, rt.status, dependents_after_wait=ops.switches().attn_side_by_side)
            if done:
                chunk, n_splits = ops.split_plan(n1, self.nkv, table.shape[1] * kv.page_size)
                room = self._partials_room(table.shape[1] * kv.page_size)
                part_acc = rt.workspace.get("attn_part_acc", (n1 * nh * n_splits * hd,), torch.float32, reserve=room * hd)
                part_ml = rt.workspace.get("attn_part_ml", (n1 * nh * n_splits * 2,), torch.float32, reserve=room * 2)
                ops.paged_attention_split(q[:n1], kv.k, kv.v, batch.positions[:n1], batch.item_of_token[:n1], table,
                                          kv.page_size, kv.n_pages, self.window, self.scale, out[:n1], part_acc, part_ml,
                                          chunk, n_splits, nh, self.nkv, hd, rt.status, fresh=1, overlap_prev=done == 2)
        elif batch.max_tokens_per_item >= 8:
            # prompt portions: the tensor-core kernel (bfloat16, head size 64 or 128), tiles of one request each
            done = ops.attention_prefill(q, kv.k, kv.v, batch.item_row_start, batch.item_start_pos, batch.n_items, table,
                                         kv.page_size, kv.n_pages, self.window, self.scale, out, nh, self.nkv, hd, rt.status)
        if not done and nh // self.nkv <= 8 and T <= 65535:
            # keys cut into chunks; the cut depends on the launch's shape (tokens, table width) only
            chunk, n_splits = ops.split_plan(T, self.nkv, table.shape[1] * kv.page_size)
            room = self._partials_room(table.shape[1] * kv.page_size)
            part_acc = rt.workspace.get("attn_part_acc", (T * nh * n_splits * hd,), torch.float32, reserve=room * hd)
            part_ml = rt.workspace.get("attn_part_ml", (T * nh * n_splits * 2,), torch.float32, reserve=room * 2)
            if batch.decode_only and rt.act_dtype == torch.bfloat16 and n_splits <= 64 and ops.fuse_producers():
                # decode rows: the partial results stay as they are and the output product combines them while it
                # makes its token operand; no combine kernel and no tensor between the two
                ops.paged_attention_split(q, kv.k, kv.v, batch.positions, batch.item_of_token, table, kv.page_size,
                                          kv.n_pages, self.window, self.scale, None, part_acc, part_ml, chunk,
                                          n_splits, nh, self.nkv, hd, rt.status, fresh=1)
                if not ops.linear_of_attention_partials(part_acc, part_ml, T, nh, hd, n_splits, self.w_o, residual, rt.status):
                    ops.attention_split_combine(part_acc, part_ml, out, T * nh, hd, n_splits)
                    ops.linear(out, self.w_o, residual, accumulate=True, status=rt.status)
                if self.b_o is not None:
                    ops.add_bias(residual, self.b_o)
                return
            done = ops.paged_attention_split(q, kv.k, kv.v, batch.positions, batch.item_of_token, table, kv.page_size,
                                             kv.n_pages, self.window, self.scale, out, part_acc, part_ml, chunk,
                                             n_splits, nh, self.nkv, hd, rt.status, fresh=batch.max_tokens_per_item)
        if not done:
            ops.paged_attention(q, kv.k, kv.v, batch.positions, batch.item_of_token, table, kv.page_size, kv.n_pages,
                                self.window, self.scale, out, nh, self.nkv, hd, rt.status)
        ops.linear(out, self.w_o, residual, accumulate=True, status=rt.status)
        if self.b_o is not None:
            ops.add_bias(residual, self.b_o)

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
from .spec import PagedKV, PartSpec, WeightSpec


class AttentionMixer(Part):
    """params: hidden, n_heads, n_kv_heads, head_dim, eps, window (None or int), position
    (PartSpec), qk_norm (bool, default True: per-head RMS norm of q and k with a weight each; False: none, and
    no norm tensors are declared), bias (bool, default False: True declares optional q/k/v/out biases, used
    when the file carries them), names (optional dict of tensor names)."""
    adds_with_linear = True


    NAMES = {"q": "self_attn.q_proj.weight", "k": "self_attn.k_proj.weight", "v": "self_attn.v_proj.weight",
             "o": "self_attn.out_proj.weight", "q_norm": "self_attn.q_layernorm.weight",
             "k_norm": "self_attn.k_layernorm.weight", "q_bias": "self_attn.q_proj.bias", "k_bias": "self_attn.k_proj.bias",
             "v_bias": "self_attn.v_proj.bias", "o_bias": "self_attn.out_proj.bias"}

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden"])
        self.nh = int(p["n_heads"])
        self.nkv = int(p["n_kv_heads"])
        self.hd = int(p["head_dim"])
        self.eps = float(p["eps"])
        self.window = int(p["window"]) if p.get("window") else None
        self.qk_norm = bool(p.get("qk_norm", True))
        self.bias = bool(p.get("bias", False))
        if self.nh % self.nkv:
            raise ValueError(f"attention: kv heads {self.nkv} must divide heads {self.nh}")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ValueError(f"attention: head size {self.hd} is not supported by the kernels "
                             "(multiples of 16 from 16 to 256)")
        self.scale = 1.0 / math.sqrt(self.hd)
        self.names = {k: prefix + v for k, v in {**self.NAMES, **p.get("names", {})}.items()}
        self.position = make_part("position", p.get("position", PartSpec("none")), prefix, rt)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None

    def weight_specs(self):
        n, H, hd = self.names, self.hidden, self.hd
        specs = [WeightSpec(n["q"], ((self.nh * hd, H),)), WeightSpec(n["k"], ((self.nkv * hd, H),)),
                 WeightSpec(n["v"], ((self.nkv * hd, H),)), WeightSpec(n["o"], ((H, self.nh * hd),))]
        if self.qk_norm:
            specs += [WeightSpec(n["q_norm"], ((hd,),), role="vector", init=("norm",)),
                      WeightSpec(n["k_norm"], ((hd,),), role="vector", init=("norm",))]
        if self.bias:
            specs += [WeightSpec(n["q_bias"], ((self.nh * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["k_bias"], ((self.nkv * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["v_bias"], ((self.nkv * hd,),), role="vector", init=("bias",), optional=True),
                      WeightSpec(n["o_bias"], ((H,),), role="vector", init=("bias",), optional=True)]
        return specs + self.position.weight_specs()

    def bind(self, tensors):
        n = self.names
        # one fused projection [q | k | v]: a layout choice, the arithmetic is unchanged
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.q_norm = tensors[n["q_norm"]] if self.qk_norm else None
        self.k_norm = tensors[n["k_norm"]] if self.qk_norm else None
        if self.bias:
            parts = [(tensors.get(n["q_bias"]), self.nh * self.hd), (tensors.get(n["k_bias"]), self.nkv * self.hd),
                     (tensors.get(n["v_bias"]), self.nkv * self.hd)]
            if any(t is not None for t, _ in parts):      # one vector [q | k | v], zeros where the file has none
                ref = self.w_o
                self.b_qkv = torch.cat([t.float() if t is not None else torch.zeros(w, dtype=torch.float32, device=ref.device)
                                        for t, w in parts]).contiguous()
            self.b_o = tensors.get(n["o_bias"])
        self.position.bind(tensors)

    def cache_specs(self):
        return (PagedKV(self.nkv, self.hd, self.window),)

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

    def forward(self, x, batch, caches, residual):
        kv = caches[0]
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

"""Causal grouped-query attention over the paged cache: the mixer of the Llama decoder.

Formulas of the reference's ``Attention`` (edgerag/core/layers.py:278-322): bias-free q/k/v/o
projections, position encoding on q and k before the cache write, kv head ``h // (nq / nkv)``
serving query head ``h`` (edgerag/core/layers.py:117-134), scores scaled by ``head_dim ** -0.5``
(edgerag/core/layers.py:276), softmax in float32.  The three input projections are stored as one
matrix ``[Wq; Wk; Wv]`` (row concatenation leaves every output column's arithmetic unchanged), so
one product yields a row ``q heads | k heads | v heads`` per token.

Single new tokens go through the split-KV decode kernel, portions of prompts through the row
kernel; both read keys and values straight from the pages (no gather copy, unlike
edgerag/cache/paged.py:208-238).
"""

from __future__ import annotations

import torch

from ..cache.manager import KVGroupSpec
from ..ops import kernels
from .base import LayerCall, Mixer, PartSpec, WeightSpec, build_part, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden: int, n_q_heads: int, n_kv_heads: int, head_dim: int, position: PartSpec,
                 dtype: torch.dtype, device: torch.device, window: int = 0, own_kv: bool = True,
                 scale: float | None = None) -> None:
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads are not divisible by {n_kv_heads} kv heads")
        self.hidden, self.n_q, self.n_kv, self.head_dim = hidden, n_q_heads, n_kv_heads, head_dim
        self.window = int(window or 0)
        self.own_kv = own_kv
        self.scale = float(head_dim ** -0.5 if scale is None else scale)
        self.dtype, self.device = dtype, device
        self.position = build_part("position", position, dtype, device)
        self.q_width = n_q_heads * head_dim
        self.kv_width = n_kv_heads * head_dim
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None

    def cache_spec(self) -> KVGroupSpec:
        return KVGroupSpec(1, self.n_kv, self.head_dim, self.window)

    def weight_specs(self) -> list[WeightSpec]:
        specs = [WeightSpec("q_proj.weight", (self.q_width, self.hidden))]
        if self.own_kv:
            specs += [WeightSpec("k_proj.weight", (self.kv_width, self.hidden)),
                      WeightSpec("v_proj.weight", (self.kv_width, self.hidden))]
        return specs + [WeightSpec("o_proj.weight", (self.hidden, self.q_width))]

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        if self.own_kv:
            parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        else:  # rows for k and v stay zero: the layer reads another layer's cache
            pad = torch.zeros((2 * self.kv_width, self.hidden), dtype=self.dtype, device=self.device)
            parts = [tensors["q_proj.weight"], pad]
        self.w_qkv = torch.cat([p.to(device=self.device, dtype=self.dtype) for p in parts], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].to(device=self.device, dtype=self.dtype).contiguous()

    def forward(self, x: torch.Tensor, ctx, call: LayerCall) -> torch.Tensor:
        n = x.shape[0]
        d = self.head_dim
        qkv = ctx.buf("attn.qkv", (n, self.q_width + 2 * self.kv_width), self.dtype)
        k_pages, v_pages = ctx.pages_of(call.cache_layer)
        group = ctx.group_of(call.cache_layer)
        write = call.writes_cache and self.own_kv
        pages, slots = ((k_pages, v_pages), ctx.slots[group]) if write else (None, None)
        if not self.position.project_apply_store(x, self.w_qkv, qkv, ctx, self.n_q, self.n_kv, d, pages, slots):
            kernels.linear(x, self.w_qkv, qkv)
            self.position.apply_and_store(qkv, ctx, self.n_q, self.n_kv, d, pages, slots)
        out = ctx.buf("attn.out", (n, self.q_width), self.dtype)
        tables = ctx.block_tables[group]
        nd = ctx.n_decode
        if nd:
            grouped = self.n_q != self.n_kv and kernels.decode_gqa_supported(self.dtype, d, self.window, self.n_q, self.n_kv,
                                                                              ctx.page_size, kernels.DECODE_SPLIT_KEYS)
            if ctx.batch_invariant:     # one plan for every batch: a sequence's sums are then added in one order
                split, heads_per_block = kernels.DECODE_SPLIT_KEYS, 0
            else:
                split, heads_per_block = kernels.choose_decode_plan(nd, self.n_kv, ctx.max_keys_bound(), ctx.page_size, d,
                                                                    grouped or self.window > 0 or self.dtype != torch.bfloat16,
                                                                    ctx.keys_granule())
            max_splits = ctx.decode_splits(self.window, split)
            need_acc, need_ml = kernels.decode_scratch_floats(nd, self.n_q, d, max_splits)
            part_acc = ctx.buf("attn.part_acc", (need_acc,), torch.float32)
            part_ml = ctx.buf("attn.part_ml", (need_ml,), torch.float32)
            if kernels.decode_gqa_supported(self.dtype, d, self.window, self.n_q, self.n_kv, ctx.page_size, split, max_splits):
                kernels.attention_decode_gqa(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                             out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits, ctx.status,
                                             split_keys=split)
            elif kernels.decode_bulk_supported(self.dtype, d, self.window, self.n_q, self.n_kv, max_splits):
                kernels.attention_decode_bulk(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                              out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits, ctx.status,
                                              split_keys=split, head_group=heads_per_block)
            else:
                kernels.attention_decode(qkv[:nd], k_pages, v_pages, tables, ctx.token_of_seq[:nd], ctx.positions,
                                         out[:nd], self.n_q, self.scale, part_acc, part_ml, max_splits,
                                         window=self.window, split_keys=split)
        if n > nd and kernels.prefill_tc_supported(self.dtype, d, self.window, ctx.page_size):
            blocks = kernels.prefill_tc_blocks(ctx.host_q_len[nd:])
            # a portion that is short against its past: its few blocks' keys are cut into ranges
            ranges = kernels.prefill_tc_key_splits(blocks, self.n_q, ctx.max_keys_bound(), qkv.device)
            part_o = part_ml = None
            if ranges > 1:
                need_o, need_ml = kernels.prefill_tc_scratch_floats(n, self.n_q, ranges)
                part_o = ctx.buf("attn.range_o", (need_o,), torch.float32)
                part_ml = ctx.buf("attn.range_ml", (need_ml,), torch.float32)
            kernels.attention_prefill_tc(qkv, k_pages, v_pages, tables[nd:], ctx.seq_starts[nd:], ctx.positions, out, blocks,
                                         self.n_q, self.scale, ctx.status, key_splits=ranges, first_row=nd, part_o=part_o,
                                         part_ml=part_ml)
        elif n > nd:
            kernels.attention_rows(qkv[nd:], k_pages, v_pages, tables, ctx.seq_of_token[nd:], ctx.positions[nd:],
                                   out[nd:], self.n_q, self.scale, window=self.window)
        n_parts = kernels.linear_parts_count(out, self.w_o)
        if n_parts:      # the rows of a larger decode step: k split over the SMs, the norm after adds the parts
            y = ctx.buf("mixer.out_parts", (n_parts, n, self.hidden), torch.float32)
            kernels.linear_parts(out, self.w_o, y)
            return y
        y = ctx.buf("mixer.out", (n, self.hidden), self.dtype)
        kernels.linear(out, self.w_o, y)
        return y

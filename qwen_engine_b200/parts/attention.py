"""Grouped-query attention over the paged cache.

q, k, v projections (one product over the stacked weights), per-head RMS norm
of q and k, position encoding, write of k and v into the request's pages,
attention of the new queries over all keys of the request that the mask
allows, output projection (reference src/models/qwen3/model.py:200-213).
Query head h reads key/value head h // (heads / kv_heads)
(src/layers/fused_ops/attn.py:181-182); key j is allowed for the query at
position i iff j <= i (attn.py:195, 239) and, with a window w, j > i - w.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import PagedKVSpec
from ..weights.spec import MATRIX, NORM, WeightSpec
from .base import Mixer, PartSpec, StepContext, register, step_hint


@register("mixer", "gqa_attention")
class GQAAttention(Mixer):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, qk_norm_eps: Optional[float] = None,
                 position_encoding: Optional[PartSpec] = None, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.pos = position_encoding.build("position_encoding") if position_encoding else None
        self.q_width = num_heads * head_dim
        self.kv_width = num_kv_heads * head_dim
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def attention_geometry(self):
        return (self.num_heads, self.num_kv_heads, self.head_dim, self.window or 0)

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        specs = [
            WeightSpec(prefix + "q_proj.weight", (self.q_width, self.hidden_size), MATRIX),
            WeightSpec(prefix + "k_proj.weight", (self.kv_width, self.hidden_size), MATRIX),
            WeightSpec(prefix + "v_proj.weight", (self.kv_width, self.hidden_size), MATRIX),
            WeightSpec(prefix + "o_proj.weight", (self.hidden_size, self.q_width), MATRIX),
        ]
        if self.qk_norm_eps is not None:
            specs += [WeightSpec(prefix + "q_norm.weight", (self.head_dim,), NORM),
                      WeightSpec(prefix + "k_norm.weight", (self.head_dim,), NORM)]
        if self.pos is not None:
            specs += self.pos.weight_specs(prefix)
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        # q, k and v rows stacked: one product gives [T, q_width + 2 kv_width]
        stacked = torch.cat([source.get(prefix + n + "_proj.weight") for n in ("q", "k", "v")], dim=0)
        self.w_qkv = ops.prepare_matrix(stacked.to(dtype).to(device))
        self.w_o = ops.prepare_matrix(source.get(prefix + "o_proj.weight").to(dtype).to(device))
        if self.qk_norm_eps is not None:
            self.q_norm_w = source.get(prefix + "q_norm.weight").to(torch.float32).to(device).contiguous()
            self.k_norm_w = source.get(prefix + "k_norm.weight").to(torch.float32).to(device).contiguous()
        if self.pos is not None:
            self.pos.load(prefix, source, dtype, device)

    def first_weights(self):
        return self.w_qkv

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        T = ctx.num_tokens
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        view = ctx.groups[group]
        qkv = ctx.arena.alloc((T, self.q_width + 2 * self.kv_width), ctx.dtype)
        rot = self.pos.half_split_rotation() if self.pos is not None else None
        fused_rope = rot is not None
        attn = ctx.arena.alloc((T, self.q_width), ctx.dtype)
        if fused_rope and ops.qkv_rope_fused_applies(T, qkv.shape[1], self.hidden_size, ctx.dtype, D, rot.rotary_dim):
            table = rot.step_table(ctx)
            if table is not None:
                # many rows: norm, rotation and cache write happen in the epilogue of the QKV product
                if isinstance(x, ops.NormedInput):
                    x = x.materialize()
                ops.linear_qkv_rope(x, self.w_qkv, qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0, table,
                                    cache, view.slot_mapping, H, Hkv, write_kv=write_cache)
                ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                                    self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
                ops.linear(attn, self.w_o, out)
                return
        if fused_rope and ops.qkv_rope_small_applies(T, qkv.shape[1], self.hidden_size, ctx.dtype, D, rot.rotary_dim):
            # a few rows: the same in the epilogue of the product that streams the weights (a cluster of CTAs per head)
            ops.prefetch_next(self.w_o)
            ops.linear_qkv_rope_small(x, self.w_qkv, qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                                      ctx.positions, rot.inv_freq, rot.step_table(ctx), cache, view.slot_mapping, H, Hkv,
                                      write_kv=write_cache)
            ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                                self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
            ops.prefetch_next(step_hint(ctx, "weights_after_mixer"))
            ops.linear(attn, self.w_o, out)
            ops.prefetch_next(None)
            return
        ops.prefetch_next(self.w_o)
        ops.linear(x, self.w_qkv, qkv)
        if self.pos is not None and not fused_rope:
            # another position encoding: norm first (the order of model.py:204-208),
            # then the part's own rotation, then the plain cache write
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, self.q_norm_w, self.k_norm_w,
                                      self.qk_norm_eps or 0.0, None, 0, cache, view.slot_mapping,
                                      H, Hkv, D, write_kv=False)
            q3 = qkv[:, :self.q_width].unflatten(1, (H, D))
            k3 = qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (Hkv, D))
            self.pos.rotate(ctx, q3, k3)
            ops.qk_norm_rope_kv_write(qkv, ctx.positions, None, None, 0.0, None, 0, cache,
                                      view.slot_mapping, H, Hkv, D, write_kv=write_cache)
        else:
            ops.qk_norm_rope_kv_write(
                qkv, ctx.positions, self.q_norm_w, self.k_norm_w, self.qk_norm_eps or 0.0,
                rot.inv_freq if fused_rope else None,
                rot.rotary_dim if fused_rope else 0,
                cache, view.slot_mapping, H, Hkv, D, write_kv=write_cache,
                cos_sin=rot.step_table(ctx) if fused_rope else None)
        ops.paged_attention(qkv, cache, view.block_tables, ctx, attn, self.scale,
                            self.window or 0, H, Hkv, D, next_pages=step_hint(ctx, "next_cache"))
        ops.prefetch_next(step_hint(ctx, "weights_after_mixer"))
        ops.linear(attn, self.w_o, out)
        ops.prefetch_next(None)

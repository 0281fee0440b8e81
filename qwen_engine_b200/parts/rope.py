"""Rotary position encoding with half-split ("neox") pairs.

inv_freq[j] = theta^(-2j/rotary_dim); angle = position * inv_freq[j] in
float32; out = [cos*x1 - sin*x2 | sin*x1 + cos*x2] with x1, x2 the two halves of
the rotated dimensions (reference src/models/qwen3/model.py:75-84,
src/layers/ops/rope.py:37-121).  The reference keeps a float32 cos/sin table
of max_position rows in every layer; here one inv_freq vector is kept and the
angle, its cosine and its sine are computed in float32 inside the kernel that
also norms q and k and writes the cache.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, StepContext, register


@register("position_encoding", "rope_neox")
class NeoxRope(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {head_dim}")
        # the same float32 arithmetic as model.py:77-79
        self._inv_freq_cpu = 1.0 / (self.theta ** (
            torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        self.inv_freq: torch.Tensor | None = None

    def load(self, prefix, source, dtype, device) -> None:
        self.inv_freq = self._inv_freq_cpu.to(device).contiguous()

    def step_table(self, ctx: StepContext):
        """The cosines and sines of this step's angles [T, rotary_dim / 2, 2], computed once per step
        and shared by every layer with the same frequencies; None for small steps (the kernel then
        computes them itself) and where the fused kernel takes no table."""
        if not ops.rope_table_applies(ctx.num_tokens, ctx.dtype, self.head_dim, self.rotary_dim):
            return None
        key = ("rope_table", self.theta, self.rotary_dim)
        table = ctx.extras.get(key)
        if table is None:
            # (for the whole step: a layer's own scratch is handed to the next layer when the layer is done)
            table = ctx.arena.alloc_step((ctx.num_tokens, self.rotary_dim // 2, 2), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, table)
            ctx.extras[key] = table
        return table

    def rotate(self, ctx: StepContext, q, k) -> None:
        ops.rope_neox(q, k, ctx.positions, self.inv_freq, self.rotary_dim)

    def half_split_rotation(self):
        return self

"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(reference src/models/qwen3/model.py:227-237; silu(g) = g / (1 + exp(-g)) in
float32, src/layers/fused_ops/silumul.py:50-53).  gate and up are one product
over the stacked weights."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.spec import MATRIX, WeightSpec
from .base import FeedForward, StepContext, register, step_hint


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        I, H = self.intermediate_size, self.hidden_size
        return [WeightSpec(prefix + "gate_proj.weight", (I, H), MATRIX),
                WeightSpec(prefix + "up_proj.weight", (I, H), MATRIX),
                WeightSpec(prefix + "down_proj.weight", (H, I), MATRIX)]

    def load(self, prefix, source, dtype, device) -> None:
        stacked = torch.cat([source.get(prefix + "gate_proj.weight"),
                             source.get(prefix + "up_proj.weight")], dim=0)
        self.w_gate_up = ops.prepare_matrix(stacked.to(dtype).to(device))
        self.w_down = ops.prepare_matrix(source.get(prefix + "down_proj.weight").to(dtype).to(device))

    def first_weights(self):
        return self.w_gate_up

    def forward(self, ctx: StepContext, x, out) -> None:
        T, I = ctx.num_tokens, self.intermediate_size
        if ops.swiglu_fused_applies(T, I, self.hidden_size, ctx.dtype):
            # many rows: the activation comes out of the gate/up product's epilogue
            if isinstance(x, ops.NormedInput):
                x = x.materialize()
            act = ctx.arena.alloc((T, I), ctx.dtype)
            ops.linear_swiglu(x, self.w_gate_up, act)
            ops.linear(act, self.w_down, out)
            return
        if ops.swiglu_small_applies(T, I, self.hidden_size, ctx.dtype):
            # a few rows: the product that streams the gate and up weights forms the activation itself
            act = ctx.arena.alloc((T, I), ctx.dtype)
            ops.prefetch_next(self.w_down)
            ops.linear_swiglu_small(x, self.w_gate_up, act)
            ops.prefetch_next(step_hint(ctx, "weights_after_ffn"))
            ops.linear(act, self.w_down, out)
            ops.prefetch_next(None)
            return
        gate_up = ctx.arena.alloc((T, 2 * I), ctx.dtype)
        ops.prefetch_next(self.w_down)
        ops.linear(x, self.w_gate_up, gate_up)
        ops.prefetch_next(step_hint(ctx, "weights_after_ffn"))
        ops.linear_silu_mul(gate_up, self.w_down, out, ctx.arena.alloc)
        ops.prefetch_next(None)

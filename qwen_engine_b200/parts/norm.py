"""RMS norm over the width of the residual stream, with the add of the
previous branch fused in.

y = x * rsqrt(mean(x^2) + eps) * w, all in float32
(reference src/layers/ops/layernorm.py:50-88).  The reference adds residuals
with a separate ``+`` in the model's dtype (src/models/qwen3/model.py:291, 296);
here the stream is float32 and the add happens inside the norm kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights.spec import NORM, WeightSpec
from .base import Norm, StepContext, register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str = "weight"):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        return [WeightSpec(prefix + self.weight_name, (self.width,), NORM)]

    def load(self, prefix, source, dtype, device) -> None:
        # scale vectors are float32 on the device whatever the compute dtype
        self.weight = source.get(prefix + self.weight_name).to(torch.float32).to(device).contiguous()

    def normed(self, ctx: StepContext, stream, lazy: bool = False):
        x = ops.NormedInput(stream, self.weight, self.eps, ctx.arena.alloc, ctx.dtype)
        return x if lazy else x.materialize()

    def add_norm(self, ctx: StepContext, resid, delta, out):
        ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
        return out

    def add_norm_rows(self, ctx: StepContext, resid, delta, rows, out):
        ops.add_rmsnorm_rows(resid, delta, rows, self.weight, self.eps, out)
        return out

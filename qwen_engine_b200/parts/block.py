"""The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(reference src/models/qwen3/model.py:278-298).  Each add is carried to the
next norm as a pending delta so that one kernel adds and norms."""
from __future__ import annotations

from .base import Block, PartSpec, StepContext, register


@register("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, hidden_size: int, mixer: PartSpec, feed_forward: PartSpec, norm: PartSpec,
                 mixer_prefix: str = "self_attn.", ffn_prefix: str = "mlp.",
                 norm1_prefix: str = "input_layernorm.", norm2_prefix: str = "post_attention_layernorm."):
        self.hidden_size = hidden_size
        self.norm1 = norm.build("norm")
        self.norm2 = norm.build("norm")
        self.mixer = mixer.build("mixer")
        self.ffn = feed_forward.build("feed_forward")
        self.prefixes = (norm1_prefix, mixer_prefix, norm2_prefix, ffn_prefix)

    def _parts(self):
        return zip((self.norm1, self.mixer, self.norm2, self.ffn), self.prefixes)

    def weight_specs(self, prefix: str):
        return [s for part, p in self._parts() for s in part.weight_specs(prefix + p)]

    def load(self, prefix, source, dtype, device) -> None:
        for part, p in self._parts():
            part.load(prefix + p, source, dtype, device)

    def forward(self, ctx: StepContext, resid, delta, has_delta, cache, group, write_cache) -> bool:
        mark = ctx.arena.mark()
        h = ctx.arena.alloc((ctx.num_tokens, self.hidden_size), ctx.dtype)
        self.norm1.add_norm(ctx, resid, delta if has_delta else None, h)
        self.mixer.forward(ctx, h, cache, group, delta, write_cache)
        self.norm2.add_norm(ctx, resid, delta, h)
        self.ffn.forward(ctx, h, delta)
        ctx.arena.release(mark)
        return True

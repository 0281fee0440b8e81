"""The pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(reference src/models/qwen3/model.py:278-298).  Each add is carried to the
next norm as a pending delta so that one kernel adds and norms."""
from __future__ import annotations

from .. import ops
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

    @property
    def capturable(self) -> bool:
        return all(getattr(part, "capturable", True) for part, _ in self._parts())

    def weight_specs(self, prefix: str):
        return [s for part, p in self._parts() for s in part.weight_specs(prefix + p)]

    def load(self, prefix, source, dtype, device) -> None:
        for part, p in self._parts():
            part.load(prefix + p, source, dtype, device)

    def first_weights(self):
        return self.mixer.first_weights()

    def forward(self, ctx: StepContext, stream, cache, group, write_cache) -> None:
        mark = ctx.arena.mark()
        h = self.norm1.normed(ctx, stream, lazy=self.mixer.takes_lazy_input)
        out = self._branch_out(stream, self.mixer)
        if getattr(ctx, "extras", None) is not None:
            ctx.extras["weights_after_mixer"] = self.ffn.first_weights()
        self.mixer.forward(ctx, h, cache, group, out, write_cache)
        self._branch_done(stream, out)
        h = self.norm2.normed(ctx, stream, lazy=self.ffn.takes_lazy_input)
        out = self._branch_out(stream, self.ffn)
        self.ffn.forward(ctx, h, out)
        self._branch_done(stream, out)
        ctx.arena.release(mark)

    @staticmethod
    def _branch_out(stream, part):
        """Where a branch writes: a sink that adds into the stream for parts whose last operation is
        an ``ops`` product (they declare it), else the stream's delta buffer."""
        return ops.ResidualSink(stream) if part.writes_through_linear else stream.delta

    @staticmethod
    def _branch_done(stream, out) -> None:
        if not isinstance(out, ops.ResidualSink):      # the output waits in delta for the next norm
            stream.has_delta, stream.n_ssq = True, 0

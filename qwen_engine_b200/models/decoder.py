"""The generic decoder: embedding, a plan of layers, final norm, output head.

Which layers exist, what each is made of, and in which order they run is data
(``ModelLayout``), written by an architecture's layout function from its
configuration.  The plan is a list of entries; an entry names the layer to run,
the cache slot it uses, and whether it writes that slot (a layer may run twice
under two slots, or read the slot another layer wrote).

The reference's model runs embedding, its layers in order, the final norm and
the head over every row (src/models/qwen3/model.py:347-360, 420-422); here the
final norm and the head run on the rows whose logits are wanted only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..cache.spec import CacheSpec
from ..parts.base import Block, PartSpec, StepContext
from ..weights.loader import check_against_manifest
from ..weights.spec import MATRIX, TensorSource, WeightSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: which block arrangement with which parameters, and the prefix
    of its tensors in the checkpoint."""

    block: PartSpec
    weight_prefix: str


@dataclass(frozen=True)
class PlanEntry:
    layer: int                  # index into ModelLayout.layers
    cache_slot: Optional[int]   # which cache slot this run uses (None: the mixer keeps nothing)
    write_cache: bool = True    # False: read what another entry wrote into the slot


@dataclass(frozen=True)
class ModelLayout:
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    plan: tuple[PlanEntry, ...]
    final_norm: PartSpec
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    tie_head: bool = True
    max_positions: Optional[int] = None


class DecoderModel:
    def __init__(self, layout: ModelLayout):
        self.layout = layout
        self.blocks: list[Block] = [ls.block.build("block") for ls in layout.layers]
        self.final_norm = layout.final_norm.build("norm")
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        n_slots = 1 + max((e.cache_slot for e in layout.plan if e.cache_slot is not None), default=-1)
        specs: list[Optional[CacheSpec]] = [None] * n_slots
        writers = [0] * n_slots
        for e in layout.plan:
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"plan names layer {e.layer}, the model has {len(self.blocks)}")
            if e.cache_slot is None:
                continue
            spec = self.blocks[e.layer].mixer.cache_spec()
            if spec is None:
                raise ValueError(f"plan gives layer {e.layer} a cache slot but its mixer keeps nothing")
            if specs[e.cache_slot] is not None and specs[e.cache_slot] != spec:
                raise ValueError(f"cache slot {e.cache_slot} is used by layers with different needs")
            specs[e.cache_slot] = spec
            writers[e.cache_slot] += int(e.write_cache)
        for slot, n in enumerate(writers):
            if specs[slot] is not None and n != 1:
                raise ValueError(f"cache slot {slot} must be written by exactly one plan entry, not {n}")
        self._cache_specs = specs
        geos = []
        for b in self.blocks:
            geo = b.mixer.attention_geometry()
            if geo is not None and geo not in geos:
                geos.append(geo)
        self.attention_geometries = tuple(geos)
        self.capturable = all(getattr(b, "capturable", True) and getattr(b.mixer, "capturable", True) for b in self.blocks)

    # ---- what the cache manager and the loader ask --------------------------------------
    def cache_specs(self) -> list[Optional[CacheSpec]]:
        return list(self._cache_specs)

    def weight_manifest(self) -> list[WeightSpec]:
        lo = self.layout
        specs = [WeightSpec(lo.embed_name, (lo.vocab_size, lo.hidden_size), MATRIX)]
        for ls, block in zip(lo.layers, self.blocks):
            specs += block.weight_specs(ls.weight_prefix)
        specs += self.final_norm.weight_specs(lo.final_norm_prefix)
        specs.append(WeightSpec(lo.head_name, (lo.vocab_size, lo.hidden_size), MATRIX,
                                optional=lo.tie_head))
        return specs

    def load_weights(self, source: TensorSource, dtype: torch.dtype, device, where: str = "checkpoint") -> None:
        check_against_manifest(source, self.weight_manifest(), where)
        lo = self.layout
        self.dtype, self.device = dtype, torch.device(device)
        self.embed = ops.prepare_matrix(source.get(lo.embed_name).to(dtype).to(device))
        for ls, block in zip(lo.layers, self.blocks):
            block.load(ls.weight_prefix, source, dtype, device)
        self.final_norm.load(lo.final_norm_prefix, source, dtype, device)
        if lo.tie_head:
            self.head = self.embed            # the same storage (model.py:417-418)
            if lo.head_name in set(source.names()):
                # the reference lets such a tensor overwrite the shared storage (whichever of the two is read
                # last wins); here the embedding is the one that counts, and the user is told
                import warnings
                warnings.warn(f"{where}: the model ties its output head to the embedding; the stored "
                              f"{lo.head_name!r} is not used", stacklevel=2)
        else:
            self.head = ops.prepare_matrix(source.get(lo.head_name).to(dtype).to(device))

    def weight_bytes(self) -> int:
        """Bytes of every weight a decode step reads once (a tied head counts once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_floating_point():
                    key = v.untyped_storage().data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += v.numel() * v.element_size()
                elif hasattr(v, "weight_specs"):
                    visit(v)
        total += self.embed.numel() * self.embed.element_size()
        seen.add(self.embed.untyped_storage().data_ptr())
        if self.head is not None and self.head.untyped_storage().data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        for b in self.blocks:
            visit(b)
        visit(self.final_norm)
        return total

    # ---- one step ---------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: CacheManager) -> Optional[torch.Tensor]:
        """Run the tokens of ``ctx`` through the plan; float32 logits
        [num_logit_rows, vocab] (None when no logits are wanted)."""
        lo = self.layout
        T, H = ctx.num_tokens, lo.hidden_size
        stream = ops.ResidualStream.for_step(ctx.arena.alloc, T, H, ctx.dtype)
        ops.embedding(ctx.token_ids, self.embed, stream)
        views = [(cache.layer_view(e.cache_slot), cache.group_of_slot[e.cache_slot][0]) if e.cache_slot is not None
                 else (None, None) for e in lo.plan]
        for i, entry in enumerate(lo.plan):
            view, group = views[i]
            # a hint for mixers that can ask for it ahead of time: the cache that the next entry of the plan
            # with a cache of the same group will read (the same pages at the same places)
            ctx.extras["next_cache"] = next((v for v, g in views[i + 1:] if v is not None and g == group and v is not view), None)
            # and the weights that the step reads first after this block
            nxt = lo.plan[i + 1].layer if i + 1 < len(lo.plan) else None
            ctx.extras["weights_after_ffn"] = self.blocks[nxt].first_weights() if nxt is not None else None
            self.blocks[entry.layer].forward(ctx, stream, view, group, entry.write_cache)
        ctx.extras["next_cache"] = ctx.extras["weights_after_ffn"] = None
        if ctx.num_logit_rows == 0:
            return None
        N = ctx.num_logit_rows
        normed = ctx.arena.alloc((N, H), ctx.dtype)
        self.final_norm.add_norm_rows(ctx, stream.resid, stream.delta if stream.has_delta else None,
                                      ctx.logit_rows, normed)
        logits = ctx.arena.alloc((N, lo.vocab_size), torch.float32)
        ops.linear(normed, self.head, logits)
        return logits

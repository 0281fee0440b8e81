"""Interfaces of the parts a layer is put together from, and their registries.

A part takes its sizes and constants as constructor parameters, says which
checkpoint tensors it needs, loads them, and runs on the flat token batch of
one step.  No part knows which model it is in: a model is a list of layer
descriptions (which block, which mixer, which feed-forward, which norm, with
which parameters) plus the order in which the layers run.

Kinds of parts and what each must offer:

* ``Norm``: ``add_norm(ctx, resid, delta, out)`` adds ``delta`` (may be None) into
  the float32 residual stream in place and writes the normed rows;
  ``add_norm_rows`` does the same for chosen rows without touching the stream.
* ``PositionEncoding``: ``rotate(ctx, q, k)`` changes query and key rows in place
  given ``ctx.positions``.
* ``Mixer``: ``cache_spec()`` describes the cache it needs (pages of keys and
  values, state of fixed size, or None); ``forward(ctx, x, cache, group, out,
  write_cache)`` mixes information between the tokens of each request.
* ``FeedForward``: ``forward(ctx, x, out)`` works on each token alone.
* ``Block``: arranges norm, mixer and feed-forward around the residual stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from ..cache.spec import CacheSpec
from ..weights.spec import TensorSource, WeightSpec


# --------------------------------------------------------------------------------------
# what a part sees of the running step
# --------------------------------------------------------------------------------------

class Arena:
    """Scratch memory of a step: a bump allocator over one device buffer.

    ``mark()`` / ``release(mark)`` give stack discipline, so that a layer's
    intermediates are reused by the next layer.  Equal sequences of
    allocations give equal addresses, which CUDA graphs rely on.  When the
    buffer is too small the allocation falls back to a fresh tensor and the
    buffer grows at the next ``reset()``.  Steps repeat the same allocations, so
    the views into the buffer are kept by (offset, shape, dtype) and handed out
    again: making a view costs more host time than a launch.
    """

    ALIGN = 256

    def __init__(self, device, capacity: int = 1 << 20):
        self.device = torch.device(device)
        capacity = -(-int(capacity) // self.ALIGN) * self.ALIGN
        self.capacity = capacity
        self.buffer = torch.empty(capacity, dtype=torch.uint8, device=self.device)
        self.offset = 0
        self.high_water = 0
        self.top = capacity                   # step-lived allocations grow down from here (alloc_step)
        self._overflow: list[torch.Tensor] = []
        self._overflow_bytes = 0
        self._views: dict = {}

    def reset(self) -> None:
        if self._overflow:
            self._views = {}
            self.capacity = int((self.high_water + (self.capacity - self.top) + self._overflow_bytes) * 1.25) + self.ALIGN
            self.capacity = -(-self.capacity // self.ALIGN) * self.ALIGN
            self._overflow = []
            self._overflow_bytes = 0
            self.buffer = torch.empty(self.capacity, dtype=torch.uint8, device=self.device)
        self.offset = 0
        self.high_water = 0
        self.top = self.capacity

    def alloc_step(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """Memory that lives until the step ends, whatever marks are released meanwhile (a table that the
        first layer makes and every layer reads): taken from the buffer's far end, never given back
        before ``reset()``."""
        shape = tuple(int(s) for s in shape)
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * dtype.itemsize
        padded = -(-max(nbytes, 1) // self.ALIGN) * self.ALIGN
        if self.top - padded < max(self.offset, self.high_water):
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._overflow.append(t)
            self._overflow_bytes += padded
            return t
        self.top -= padded
        key = ("step", self.top, shape, dtype)
        view = self._views.get(key)
        if view is None:
            view = self.buffer[self.top:self.top + nbytes].view(dtype).view(shape)
            self._views[key] = view
        return view

    def mark(self) -> int:
        return self.offset

    def release(self, mark: int) -> None:
        self.offset = mark

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        hit = self._views.get((self.offset, shape, dtype))
        if hit is not None and hit[1] <= self.top:
            view, end = hit
            self.offset = end
            if end > self.high_water:
                self.high_water = end
            return view
        shape = tuple(int(s) for s in shape)
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * dtype.itemsize
        padded = -(-max(nbytes, 1) // self.ALIGN) * self.ALIGN
        if self.offset + padded > self.top:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._overflow.append(t)
            self._overflow_bytes += padded
            return t
        view = self.buffer[self.offset:self.offset + nbytes].view(dtype).view(shape)
        if len(self._views) < 4096:
            self._views[(self.offset, shape, dtype)] = (view, self.offset + padded)
        self.offset += padded
        self.high_water = max(self.high_water, self.offset)
        return view


@dataclass
class GroupStepView:
    """One cache group as a step sees it."""

    block_tables: torch.Tensor       # int32 [R, max_blocks], -1 where no page is held
    slot_mapping: torch.Tensor       # int32 [T]: page * page_size + offset of each new token
    max_blocks: int


@dataclass
class StepContext:
    """The flat batch of one step: T tokens of R requests.

    Request r brings tokens ``cu_q[r] .. cu_q[r+1]-1`` of the flat batch; they
    sit at positions ``ctx_lens[r] ...`` of the request, after ``ctx_lens[r]``
    tokens that are already in the cache."""

    num_tokens: int
    num_reqs: int
    dtype: torch.dtype                # activations and matrices: bfloat16 or float32
    device: torch.device
    page_size: int
    token_ids: torch.Tensor           # int32 [T]
    positions: torch.Tensor           # int32 [T]
    cu_q: torch.Tensor                # int32 [R+1]
    ctx_lens: torch.Tensor            # int32 [R]
    slot_ids: torch.Tensor            # int32 [R]: state slot of each request
    logit_rows: torch.Tensor          # int32 [N]: flat rows whose logits are wanted
    num_logit_rows: int
    groups: dict[int, GroupStepView]
    q_lens_host: list[int]
    ctx_lens_host: list[int]
    arena: Arena
    attn_plan: Any = None             # what ops.plan_attention made of this batch
    extras: dict[str, Any] = field(default_factory=dict)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens_host) if self.q_lens_host else 0

    @property
    def max_kv_len(self) -> int:
        return max((c + q for c, q in zip(self.ctx_lens_host, self.q_lens_host)), default=0)


def step_hint(ctx, key: str):
    """What the model or the block left in ``ctx.extras`` for the parts to use if they can (the cache the
    next layer reads, the weights read after this part); None where nobody left anything (a part run alone)."""
    extras = getattr(ctx, "extras", None)
    return extras.get(key) if extras else None


# --------------------------------------------------------------------------------------
# the parts
# --------------------------------------------------------------------------------------

class Part:
    """Common to all parts: the tensors it needs and how it takes them in."""

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        return []

    def load(self, prefix: str, source: TensorSource, dtype: torch.dtype, device) -> None:
        pass

    def first_weights(self) -> Optional[torch.Tensor]:
        """The matrix that the part's forward reads first, if it has one and cares to say: the product
        that runs just before the part may ask L2 for it ahead of time (``ops.prefetch_next``)."""
        return None


class Norm(Part):
    width: int

    def normed(self, ctx: "StepContext", stream, lazy: bool = False):
        """The normed rows of ``stream`` (an ``ops.ResidualStream``) after its pending branch output
        is added.  With ``lazy`` the result may be an ``ops.NormedInput`` that ``ops.linear`` fuses
        into the product; a consumer that needs a tensor calls its ``materialize()``."""
        raise NotImplementedError

    def add_norm(self, ctx: StepContext, resid: torch.Tensor, delta: Optional[torch.Tensor],
                 out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm_rows(self, ctx: StepContext, resid: torch.Tensor, delta: Optional[torch.Tensor],
                      rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotate(self, ctx: StepContext, q: torch.Tensor, k: torch.Tensor) -> None:
        """Encode ``ctx.positions`` into q [T, Hq, D] and k [T, Hkv, D] in place."""
        raise NotImplementedError

    def half_split_rotation(self):
        """None, or, for an encoding that rotates the pairs (x[j], x[j + rotary_dim / 2]) by
        position * inv_freq[j], an object with ``inv_freq`` (float32 on the device), ``rotary_dim`` and
        ``step_table(ctx)``: a mixer may then hand the rotation to the kernel that also norms q and k and
        writes the cache, instead of calling ``rotate``."""
        return None


class Mixer(Part):
    # False for a mixer whose forward reads device data on the host or allocates: steps of a model
    # that holds such a mixer are never captured in a CUDA graph.
    capturable = True
    # True if forward passes its input x only to ops.linear (which also takes an ops.NormedInput);
    # a mixer that looks at x itself keeps False and always gets a tensor.
    takes_lazy_input = False
    # True if forward writes ``out`` only as the ``out`` of ops.linear / ops.linear_silu_mul (which
    # also take an ops.ResidualSink and then add into the residual stream at once).
    writes_through_linear = False

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def attention_geometry(self) -> Optional[tuple[int, int, int, int]]:
        """(heads, kv heads, head size, window or 0) if the mixer calls ``ops.paged_attention``:
        the step function plans the attention kernels' work once per step for every geometry."""
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: Optional[torch.Tensor],
                group: Optional[int], out: torch.Tensor, write_cache: bool = True) -> None:
        raise NotImplementedError


class FeedForward(Part):
    capturable = True             # as for Mixer: False if forward reads step data on the host (routing by sizes)
    takes_lazy_input = False
    writes_through_linear = False

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    capturable = True             # False if any of its parts says so: steps of the model are then never graph-captured

    def forward(self, ctx: StepContext, stream, cache: Optional[torch.Tensor], group: Optional[int],
                write_cache: bool) -> None:
        """Run the layer on the residual stream (an ``ops.ResidualStream``: the float32 stream, and
        the last branch's output that is not yet added to it, so that the add is fused into the next
        norm).  Branches write their output to ``stream.delta`` and set ``stream.has_delta``."""
        raise NotImplementedError


# --------------------------------------------------------------------------------------
# registries: kind name -> factory(**params)
# --------------------------------------------------------------------------------------

NORMS: dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., PositionEncoding]] = {}
MIXERS: dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: dict[str, Callable[..., FeedForward]] = {}
BLOCKS: dict[str, Callable[..., Block]] = {}

_REGISTRIES = {"norm": NORMS, "position_encoding": POSITION_ENCODINGS, "mixer": MIXERS,
               "feed_forward": FEED_FORWARDS, "block": BLOCKS}


def register(kind: str, name: str):
    """Decorator: ``@register("mixer", "my_mixer")`` makes a part buildable by name."""
    table = _REGISTRIES[kind]

    def deco(factory):
        if name in table and table[name] is not factory:
            raise ValueError(f"{kind} {name!r} is already registered")
        table[name] = factory
        return factory
    return deco


@dataclass(frozen=True)
class PartSpec:
    """A part as data: its registered name and its parameters."""

    name: str
    params: dict[str, Any] = field(default_factory=dict)

    def build(self, kind: str):
        table = _REGISTRIES[kind]
        if self.name not in table:
            raise ValueError(f"unknown {kind} {self.name!r}; registered: {sorted(table)}")
        return table[self.name](**self.params)

"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mixture of prompt portions and single decoded tokens, cut
anywhere.  It runs only the tokens it is given, as one flat batch, against
what earlier steps left in the cache, and returns float32 logits at the places
asked for.  The reference runs either whole prompts or single tokens, never
both, builds its index tensors with per-token device writes and computes
logits for every row (src/engine/executor.py:56-103, 105-208;
src/models/qwen3/model.py:420-422); here all of a step's index data is packed
on the host and copied once.
"""
from __future__ import annotations

import gc
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .. import ops
from ..cache.manager import UNKNOWN_TOKEN, CacheManager, RequestCache
from ..cache.page_pool import OutOfPages
from ..models.decoder import DecoderModel
from ..parts.base import Arena, GroupStepView, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them
    (0-based within ``tokens``) whose logits are wanted."""

    cache: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    token_source: Optional[int] = None      # tokens == [UNKNOWN_TOKEN]: index into the step's ``device_tokens``


class _Pack:
    """Named int32 arrays laid out in one buffer, each starting on a 16-byte boundary."""

    def __init__(self):
        self.parts: list[tuple[str, int, int]] = []
        self.data: list[int] = []

    def add(self, name: str, values: Sequence[int]) -> None:
        pad = (-len(self.data)) % 4
        self.data.extend([0] * pad)
        self.parts.append((name, len(self.data), len(values)))
        self.data.extend(values)


class ModelRunner:
    GRAPH_BLOCK_BUCKET = 64       # block tables of replayed steps are padded to multiples of this

    def __init__(self, model: DecoderModel, cache: CacheManager, device, dtype: torch.dtype,
                 max_positions: Optional[int] = None, use_cuda_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.device = torch.device(device)
        self.dtype = dtype
        self.arena = Arena(self.device)
        self.max_positions = max_positions if max_positions is not None else model.layout.max_positions
        self._on_gpu = self.device.type == "cuda"
        self._host: list[Optional[torch.Tensor]] = [None, None]
        self._host_free: list[Optional[torch.cuda.Event]] = [None, None]
        self._dev_meta: Optional[torch.Tensor] = None
        self._flip = 0
        self.use_cuda_graphs = bool(use_cuda_graphs) and self._on_gpu and getattr(model, "capturable", True)
        # decode steps by shape: None after the first (eager) run, then (graph, logits, launches)
        self._graphs: dict[tuple, Optional[tuple]] = {}
        self._capture_stream = None
        self.capture_all_steps = True         # steps that are not all decoded tokens are captured too when they recur
        self.num_graph_replays = 0
        self.num_graph_captures = 0
        self.graph_capture_seconds = 0.0      # host time spent capturing and instantiating graphs
        self.num_steps = 0
        self.last_h2d_bytes = 0
        self.num_tokens_run = 0

    # ---- metadata transfer ----------------------------------------------------------------
    def _upload(self, pack: _Pack) -> dict[str, torch.Tensor]:
        n = len(pack.data)
        self.last_h2d_bytes = 4 * n
        src = torch.tensor(pack.data, dtype=torch.int32)
        if not self._on_gpu:
            dev = src.to(self.device)
        else:
            i = self._flip
            self._flip ^= 1
            if self._host[i] is None or self._host[i].numel() < n:
                self._host[i] = torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True)
                self._host_free[i] = None
            if self._host_free[i] is not None:
                self._host_free[i].synchronize()      # the copy that last read this buffer is done
            self._host[i][:n].copy_(src)
            if self._dev_meta is None or self._dev_meta.numel() < n:
                self._dev_meta = torch.empty(max(1 << 18, 2 * n), dtype=torch.int32, device=self.device)
                self._graphs.clear()                  # captured steps point into the old buffer
            dev = self._dev_meta[:n]
            dev.copy_(self._host[i][:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._host_free[i] = ev
        return {name: dev[off:off + cnt] for name, off, cnt in pack.parts}

    def _forward(self, ctx: StepContext, graph_key) -> Optional[torch.Tensor]:
        if graph_key is None:
            return self.model.forward(ctx, self.cache)
        if graph_key not in self._graphs:
            # first time: run eagerly (also sizes the arena)
            logits = self.model.forward(ctx, self.cache)
            if not self.arena._overflow:                  # else the buffers move at the next reset: try again
                self._graphs[graph_key] = None
            return logits
        entry = self._graphs[graph_key]
        if entry is None:
            if len(self._graphs) > 512:                   # many shapes: drop the oldest captures
                for k in list(self._graphs)[:256]:
                    del self._graphs[k]
            graph = torch.cuda.CUDAGraph()
            t_capture = time.perf_counter()
            before = ops.launch_count
            # captured on a stream of its own between capture_begin and capture_end: the context manager that torch
            # offers for this also collects garbage and empties the allocator's cache on entry, some tens of
            # milliseconds that a serving loop which meets new shapes all the time cannot afford.  What the
            # collection is there for is kept: no cyclic garbage is collected while the capture runs (an old
            # graph or device buffer destroyed then would invalidate the capture).
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(device=self.device)
            main = torch.cuda.current_stream(self.device)
            self._capture_stream.wait_stream(main)
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.stream(self._capture_stream):
                    graph.capture_begin()
                    try:
                        logits = self.model.forward(ctx, self.cache)
                    finally:
                        graph.capture_end()
            finally:
                if collecting:
                    gc.enable()
            main.wait_stream(self._capture_stream)
            self.num_graph_captures += 1
            self.graph_capture_seconds += time.perf_counter() - t_capture
            entry = (graph, logits, ops.launch_count - before, self.arena.buffer)
            self._graphs[graph_key] = entry
        graph, logits, launches, arena_buffer = entry
        if arena_buffer is not self.arena.buffer:         # the arena grew since: record and capture again
            del self._graphs[graph_key]
            return self._forward(ctx, graph_key)
        graph.replay()
        ops.launch_count += launches
        self.num_graph_replays += 1
        return logits

    @staticmethod
    def _device_plan(plan: dict, dev: dict, geometries) -> dict:
        """The plan's lists as device tensors, plus what the host keeps: which geometry has which
        index, and the small ``*_info`` lists as Python ints."""
        out = {k: dev["plan_" + k] for k in plan}
        out["geometry_index"] = {g: i for i, g in enumerate(geometries)}
        for k, v in plan.items():
            if k.endswith("_info"):
                out[k + "_host"] = list(v)
        return out

    # ---- the step -------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [wanted places, vocab] in the order
        of the entries and of each entry's ``want`` (None if nothing is wanted).
        The tensor lives in the step's scratch memory: it is valid until the next step.

        An entry whose one token is ``UNKNOWN_TOKEN`` takes it from ``device_tokens[entry.token_source]``
        (int32 on the device: what the step before sampled, not yet read by the host)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        cache = self.cache
        vocab = self.model.layout.vocab_size
        appended: list[RequestCache] = []
        try:
            for e in entries:
                if e.token_source is not None:
                    if device_tokens is None or list(e.tokens) != [UNKNOWN_TOKEN] or not (0 <= e.token_source < device_tokens.numel()):
                        raise ValueError(f"request {e.cache.req_id!r}: a token taken from the device must be the entry's only one")
                elif not (0 <= min(e.tokens) and max(e.tokens) < vocab):
                    bad = next(t for t in e.tokens if not (0 <= int(t) < vocab))
                    raise ValueError(f"token id {bad} of request {e.cache.req_id!r} is outside the vocabulary (0..{vocab - 1})")
                end = e.cache.num_tokens + len(e.tokens)
                if self.max_positions is not None and end > self.max_positions:
                    raise ValueError(f"request {e.cache.req_id!r} would reach {end} tokens, beyond "
                                     f"max_position_embeddings = {self.max_positions}")
                for w in e.want:
                    if not (0 <= int(w) < len(e.tokens)):
                        raise ValueError(f"wanted place {w} is outside the {len(e.tokens)} tokens of request {e.cache.req_id!r}")
                cache.append(e.cache, e.tokens)
                appended.append(e.cache)
        except (OutOfPages, ValueError):
            for rc in appended:
                cache.abort_pending(rc)
            raise

        token_ids: list[int] = []
        fix_rows: list[int] = []                   # rows of token_ids to be filled on the device, and from where
        fix_src: list[int] = []
        positions: list[int] = []
        cu_q = [0]
        ctx_lens: list[int] = []
        slot_ids: list[int] = []
        logit_rows: list[int] = []
        q_lens: list[int] = []
        for e in entries:
            rc = e.cache
            n, c = len(e.tokens), rc.num_tokens
            base = cu_q[-1]
            if e.token_source is not None:
                fix_rows.append(base)
                fix_src.append(e.token_source)
                token_ids.append(0)
            else:
                token_ids.extend(map(int, e.tokens))
            positions.extend(range(c, c + n))
            cu_q.append(base + n)
            ctx_lens.append(c)
            slot_ids.append(rc.state_slot)
            q_lens.append(n)
            logit_rows.extend(base + int(w) for w in e.want)
        T, R, N = cu_q[-1], len(entries), len(logit_rows)

        # A step of single decoded tokens has a shape that recurs: it is captured in a CUDA graph
        # the second time the shape is seen and replayed from then on.  Everything the kernels
        # read that changes from step to step lives in the metadata buffer.  Other steps recur too (a
        # long prompt in portions of the token budget, prompts of one length): they are captured by
        # what decides their launches, see below.
        graph_key = None
        uniform_splits = None
        buckets = None
        B = self.GRAPH_BLOCK_BUCKET
        if self.use_cuda_graphs and all(n == 1 for n in q_lens):
            buckets = tuple(-(-max(len(e.cache.tables[g.index]) for e in entries) // B) * B
                            for g in cache.paged_groups)
            graph_key = (R, N, buckets)
            uniform_splits = ops.decode_splits(R, max(buckets, default=B) * cache.page_size,
                                               self.model.attention_geometries, self.dtype)
        elif self.use_cuda_graphs and self.capture_all_steps:
            # block tables padded to 64 x a power of two entries, so that few widths occur
            buckets = tuple(B << max(0, (-(-max(len(e.cache.tables[g.index]) for e in entries) // B) - 1).bit_length())
                            for g in cache.paged_groups)

        pack = _Pack()
        pack.add("token_ids", token_ids)
        pack.add("positions", positions)
        pack.add("cu_q", cu_q)
        pack.add("ctx_lens", ctx_lens)
        pack.add("slot_ids", slot_ids)
        pack.add("logit_rows", logit_rows)
        max_blocks: dict[int, int] = {}
        for gi, g in enumerate(cache.paged_groups):
            mb = max(len(e.cache.tables[g.index]) for e in entries)
            if buckets is not None:
                mb = buckets[gi]
            max_blocks[g.index] = mb
            flat: list[int] = []
            slots: list[int] = []
            for e in entries:
                table = e.cache.tables[g.index]
                flat.extend(table)
                flat.extend([-1] * (mb - len(table)))
                slots.extend(cache.slot_mapping(e.cache, g.index))
            pack.add(f"bt{g.index}", flat)
            pack.add(f"sm{g.index}", slots)
        geometries = self.model.attention_geometries
        plan = ops.plan_attention(q_lens, ctx_lens, cache.page_size, geometries, self.dtype,
                                  uniform_splits=uniform_splits)
        for name, values in plan.items():
            pack.add("plan_" + name, values)
        if graph_key is None and buckets is not None:
            # what decides the launches of a step that is not all decoded tokens: the rows of every request,
            # the widths of the block tables, the lengths of the work lists and what the plan says about
            # them
            graph_key = ("step", N, tuple(q_lens), buckets,
                         tuple((k, tuple(v) if k.endswith("_info") else len(v)) for k, v in plan.items()))
        if fix_rows:        # last, so that the places of everything a captured step reads stay where they are
            pack.add("fix_rows", fix_rows)
            pack.add("fix_src", fix_src)
        page_copies = cache.page_copies_by_group()
        for gi, pairs in page_copies.items():
            pack.add(f"pc{gi}", pairs)
        dev = self._upload(pack)
        if fix_rows:
            ops.place_tokens(dev["token_ids"], dev["fix_rows"], device_tokens, dev["fix_src"])

        # private copies of shared pages that this step (or a later one) writes into: before any write
        for gi in page_copies:
            ops.copy_pages(cache.groups[gi].tensor, dev[f"pc{gi}"])
        cache.zero_fresh_state([e.cache for e in entries])

        groups = {g.index: GroupStepView(dev[f"bt{g.index}"].view(R, max_blocks[g.index]),
                                         dev[f"sm{g.index}"], max_blocks[g.index])
                  for g in cache.paged_groups}
        self.arena.reset()
        ctx = StepContext(
            num_tokens=T, num_reqs=R, dtype=self.dtype, device=self.device, page_size=cache.page_size,
            token_ids=dev["token_ids"], positions=dev["positions"], cu_q=dev["cu_q"],
            ctx_lens=dev["ctx_lens"], slot_ids=dev["slot_ids"], logit_rows=dev["logit_rows"],
            num_logit_rows=N, groups=groups, q_lens_host=q_lens, ctx_lens_host=ctx_lens,
            arena=self.arena, attn_plan=self._device_plan(plan, dev, geometries))
        logits = self._forward(ctx, graph_key)
        for e in entries:
            cache.commit(e.cache)
        self.num_steps += 1
        self.num_tokens_run += T
        return logits

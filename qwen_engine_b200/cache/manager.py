"""The cache manager: pages of keys and values with a block table per request,
grouped by what the layers need, and slots for state of fixed size.

A model hands over one cache description per cache slot of its layer plan
(``PagedKVSpec``, ``FixedStateSpec`` or None).  Slots with the same description
form a group; a group has pages (or state rows) of its own, a page pool of its
own and, for each request, a block table of its own.  Pages go back to the
pool when a request ends or is preempted and, in a group that keeps only a
window of keys, as soon as every later query has passed them; pages that come
back are handed out again.

The reference has one group, one 5-D tensor per K and V indexed by layer, and
frees pages only when its serving loop ends (src/engine/kvcache.py:47-65,
llm_engine.py:147-152).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .page_pool import OutOfPages, PagePool, hash_block
from .spec import CacheSpec, FixedStateSpec, PagedKVSpec
from .state_slots import StateSlotPool


class CacheGroup:
    """Cache slots with one description, their device tensor and their pool."""

    def __init__(self, index: int, spec: CacheSpec, cache_slots: list[int]):
        self.index = index
        self.spec = spec
        self.cache_slots = cache_slots          # ids of the model's cache slots, in order
        self.pool: Optional[PagePool] = None
        self.tensor: Optional[torch.Tensor] = None

    @property
    def is_paged(self) -> bool:
        return isinstance(self.spec, PagedKVSpec)

    def row_of(self, cache_slot: int) -> int:
        return self.cache_slots.index(cache_slot)


UNKNOWN_TOKEN = -1      # stands for a token that a step takes from the device: its id is not known on the host yet


@dataclass
class RequestCache:
    """What one live request holds."""

    req_id: object
    state_slot: int
    tokens: list[int] = field(default_factory=list)      # tokens whose entries are committed
    num_tokens: int = 0                                   # committed length
    tables: dict[int, list[int]] = field(default_factory=dict)   # group -> page per block, -1 = given back
    hashes: dict[int, list[int]] = field(default_factory=dict)   # group -> hash chain of registered blocks
    pending_tokens: list[int] = field(default_factory=list)      # appended, not yet committed
    shared_tokens: int = 0                                # length found in the prefix table at open()
    fresh_state: bool = True                              # its state rows must be zeroed before its first step
    closed: bool = False
    first_unknown: Optional[int] = None                   # position of a committed token whose id is not known yet


class CacheManager:
    def __init__(self, specs: Sequence[Optional[CacheSpec]], page_size: int, num_pages: int,
                 num_state_slots: int, dtype: torch.dtype, device, enable_prefix_cache: bool = True,
                 num_pages_of_group: Optional[dict[int, int]] = None, poison=False):
        """``poison``: for tests, what fresh pages hold instead of zeros: True for NaN (any key or value read
        before it was written shows in the logits), or a finite number for kernels that mask what they
        read from a held page past a request's length (a large value shows a mask that is off by one,
        where 0 x NaN would spoil every row)."""
        self.page_size = page_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = StateSlotPool(num_state_slots)
        self.groups: list[CacheGroup] = []
        self.group_of_slot: dict[int, tuple[int, int]] = {}   # cache slot -> (group, row)
        by_spec: dict[CacheSpec, CacheGroup] = {}
        for slot_id, spec in enumerate(specs):
            if spec is None:
                continue
            g = by_spec.get(spec)
            if g is None:
                g = CacheGroup(len(self.groups), spec, [])
                by_spec[spec] = g
                self.groups.append(g)
            g.cache_slots.append(slot_id)
            self.group_of_slot[slot_id] = (g.index, len(g.cache_slots) - 1)
        paged = [g for g in self.groups if g.is_paged]
        # A prefix can be shared if every group can hand over what the next query needs of it: a group that keeps
        # all keys, every page of the prefix; a group that keeps a window of keys, the pages its window still
        # reaches (pages it gave back stay findable until they are handed out again).  State of fixed size cannot
        # be handed over (that would take snapshots of it at page boundaries): a model that has some shares nothing.
        self.prefix_cache = bool(enable_prefix_cache and paged and all(g.is_paged for g in self.groups))
        for g in self.groups:
            if g.is_paged:
                n = (num_pages_of_group or {}).get(g.index, num_pages)
                g.pool = PagePool(n, page_size, self.prefix_cache)
                shape = (len(g.cache_slots), n, 2, g.spec.num_kv_heads, page_size, g.spec.head_dim)
                g.tensor = torch.zeros(shape, dtype=dtype, device=self.device)
                if poison is not False and poison is not None:
                    g.tensor.fill_(float("nan") if poison is True else float(poison))
            else:
                assert isinstance(g.spec, FixedStateSpec)
                shape = (len(g.cache_slots), num_state_slots) + tuple(g.spec.shape)
                g.tensor = torch.zeros(shape, dtype=g.spec.dtype, device=self.device)
        self.live: dict[object, RequestCache] = {}
        self._page_copies: list[tuple[int, int, int]] = []     # (group, src page, dst page)
        # counters for the engine's statistics
        self.prefix_hit_tokens = 0
        self.peak_pages_used = 0

    # ---- views for the parts ---------------------------------------------------------
    def layer_view(self, cache_slot: int) -> Optional[torch.Tensor]:
        """The tensor of one cache slot: [pages, 2, kv heads, page size, head dim] for
        paged keys and values, [state slots, *shape] for state of fixed size."""
        if cache_slot not in self.group_of_slot:
            return None
        g, row = self.group_of_slot[cache_slot]
        return self.groups[g].tensor[row]

    @property
    def paged_groups(self) -> list[CacheGroup]:
        return [g for g in self.groups if g.is_paged]

    def free_pages(self) -> dict[int, int]:
        return {g.index: g.pool.num_free for g in self.paged_groups}

    def pages_in_use(self) -> int:
        return sum(g.pool.num_used for g in self.paged_groups)

    # ---- a request's life ---------------------------------------------------------------
    def open(self, req_id, known_tokens: Optional[Sequence[int]] = None,
             max_shared_tokens: Optional[int] = None) -> RequestCache:
        """Admit a request: a state slot, empty block tables and, when its first
        tokens are known and sharing is on, the pages of the longest prefix
        that is already in the cache.

        If the whole of ``known_tokens`` is found, the last token is still
        left to be computed (its logits are needed), and because its key and
        value would be written into a shared page, that page is first copied
        to a private one (the reference writes into the shared page,
        src/engine/executor.py:114-119, 139-140)."""
        if req_id in self.live:
            raise ValueError(f"request {req_id!r} is already live")
        rc = RequestCache(req_id=req_id, state_slot=self.slots.allocate())
        for g in self.groups:
            if g.is_paged:
                rc.tables[g.index] = []
                rc.hashes[g.index] = []
        queued = len(self._page_copies)
        try:
            if self.prefix_cache and known_tokens:
                self._share_prefix(rc, list(known_tokens), max_shared_tokens)
        except Exception:
            del self._page_copies[queued:]       # copies into pages that go back with the rest
            self._release_all(rc)
            raise
        self.live[req_id] = rc
        return rc

    def _share_prefix(self, rc: RequestCache, tokens: list[int], max_shared_tokens: Optional[int]) -> None:
        P = self.page_size
        limit = len(tokens) // P
        if max_shared_tokens is not None:
            # n pages count as n P tokens computed, or, when they are the whole of ``tokens``, as one less
            cap = max(0, max_shared_tokens)
            limit = limit if (limit * P == len(tokens) and len(tokens) - 1 <= cap) else min(limit, cap // P)
        if limit == 0:
            return
        # the chained hashes of the leading full blocks (the same for every group), and what each group can find
        hashes: list[int] = []
        for b in range(limit):
            hashes.append(hash_block(hashes[-1] if hashes else 0, tokens[b * P:(b + 1) * P]))
        found = {g.index: [g.pool.find_page(hashes[b], tokens[b * P:(b + 1) * P]) for b in range(limit)]
                 for g in self.paged_groups}

        def first_needed(g: CacheGroup, n: int) -> int:
            """The first block of a prefix of n pages that the group's next query still reads."""
            if g.spec.window is None:
                return 0
            pos = n * P - 1 if n * P == len(tokens) else n * P       # the next token to run (the last one again on a full hit)
            return max(0, pos - g.spec.window + 1) // P

        n_pages = 0
        for n in range(limit, 0, -1):                    # the longest prefix that every group can hand over
            if all(all(found[g.index][b] is not None for b in range(first_needed(g, n), n)) for g in self.paged_groups):
                n_pages = n
                break
        if n_pages == 0:
            return
        for g in self.paged_groups:
            first = first_needed(g, n_pages)
            pages = [-1] * first + [found[g.index][b] for b in range(first, n_pages)]
            for p in pages[first:]:
                g.pool.retain(p)
            rc.tables[g.index] = pages
            rc.hashes[g.index] = list(hashes[:n_pages])
        shared = n_pages * P
        if shared == len(tokens):
            # whole prompt found: recompute its last token in a private copy of the last page
            for g in self.paged_groups:
                old = rc.tables[g.index][-1]
                new = g.pool.allocate()        # may raise OutOfPages: caller releases
                rc.tables[g.index][-1] = new
                rc.hashes[g.index].pop()
                self._page_copies.append((g.index, old, new))
                g.pool.release(old)
            shared -= 1
        rc.tokens = tokens[:shared]
        rc.num_tokens = shared
        rc.shared_tokens = shared
        self.prefix_hit_tokens += shared

    def pages_needed(self, rc: RequestCache, n_new: int) -> dict[int, int]:
        """New pages each group must hand out before ``n_new`` more tokens fit."""
        total = rc.num_tokens + len(rc.pending_tokens) + n_new
        blocks = -(-total // self.page_size)
        return {g.index: max(0, blocks - len(rc.tables[g.index])) for g in self.paged_groups}

    def pages_needed_for_new(self, n_tokens: int) -> dict[int, int]:
        blocks = -(-n_tokens // self.page_size)
        return {g.index: blocks for g in self.paged_groups}

    def can_append(self, rc: RequestCache, n_new: int, reserved: Optional[dict[int, int]] = None) -> bool:
        need = self.pages_needed(rc, n_new)
        return all(need[g.index] + (reserved or {}).get(g.index, 0) <= g.pool.num_free
                   for g in self.paged_groups)

    def append(self, rc: RequestCache, new_tokens: Sequence[int]) -> None:
        """Give the request pages for its next tokens (positions num_tokens ...).
        All or nothing: on OutOfPages what was taken is handed back."""
        if rc.closed:
            raise RuntimeError(f"request {rc.req_id!r} is closed")
        if rc.pending_tokens:
            raise RuntimeError("append() before the last append was committed")
        need = self.pages_needed(rc, len(new_tokens))
        taken: list[tuple[CacheGroup, int]] = []
        try:
            for g in self.paged_groups:
                for _ in range(need[g.index]):
                    taken.append((g, g.pool.allocate()))
        except OutOfPages:
            for g, p in taken:
                g.pool.release(p)
            raise
        for g, p in taken:
            rc.tables[g.index].append(p)
        rc.pending_tokens = list(map(int, new_tokens))
        self.peak_pages_used = max(self.peak_pages_used, self.pages_in_use())

    def slot_mapping(self, rc: RequestCache, group: int) -> list[int]:
        """Flat slot (page * page_size + offset) of each pending token in a group."""
        P = self.page_size
        table = rc.tables[group]
        out: list[int] = []
        pos, end = rc.num_tokens, rc.num_tokens + len(rc.pending_tokens)
        while pos < end:                             # a page's run of slots at a time
            page, off = table[pos // P], pos % P
            assert page >= 0
            n = min(P - off, end - pos)
            out.extend(range(page * P + off, page * P + off + n))
            pos += n
        return out

    def commit(self, rc: RequestCache) -> None:
        """The step that wrote the pending tokens is launched: count them in,
        make pages that became full sharable, and give back pages that a
        window has passed."""
        P = self.page_size
        old_len = rc.num_tokens
        if rc.first_unknown is None and UNKNOWN_TOKEN in rc.pending_tokens:
            rc.first_unknown = old_len + rc.pending_tokens.index(UNKNOWN_TOKEN)
        rc.tokens.extend(rc.pending_tokens)
        rc.num_tokens += len(rc.pending_tokens)
        rc.pending_tokens = []
        rc.fresh_state = False
        self._register_full_pages(rc)
        for g in self.paged_groups:
            table = rc.tables[g.index]
            window = g.spec.window
            if window is not None:
                # the next query sits at position num_tokens and needs keys
                # j > num_tokens - window; block b ends at (b+1)P - 1
                first_needed = rc.num_tokens - window + 1
                b = 0
                while (b + 1) * P <= first_needed and b < len(table):
                    if table[b] >= 0:
                        g.pool.release(table[b])
                        table[b] = -1
                    b += 1
        del old_len

    def _register_full_pages(self, rc: RequestCache) -> None:
        """Make the request's full pages findable by their tokens, in order (so that the chain of
        parents is complete), up to the first token whose id is not known yet."""
        if not self.prefix_cache:
            return
        P = self.page_size
        known = rc.num_tokens if rc.first_unknown is None else min(rc.num_tokens, rc.first_unknown)
        for g in self.paged_groups:
            table, chain = rc.tables[g.index], rc.hashes[g.index]
            for b in range(len(chain), known // P):
                parent = chain[-1] if chain else 0
                if table[b] >= 0:
                    chain.append(g.pool.register_full_page(table[b], parent, rc.tokens[b * P:(b + 1) * P]))
                else:               # a window gave the page back before its tokens were known
                    chain.append(hash_block(parent, rc.tokens[b * P:(b + 1) * P]))

    def resolve_token(self, rc: RequestCache, position: int, token: int) -> None:
        """The id of a token that was run before it was known on the host (a step launched ahead
        took it from the device) is known now."""
        if rc.closed:
            return
        if not (0 <= position < rc.num_tokens) or rc.tokens[position] != UNKNOWN_TOKEN:
            raise RuntimeError(f"request {rc.req_id!r} has no unknown token at position {position}")
        rc.tokens[position] = int(token)
        if rc.first_unknown == position:
            rc.first_unknown = None
            for p in range(position + 1, rc.num_tokens):
                if rc.tokens[p] == UNKNOWN_TOKEN:
                    rc.first_unknown = p
                    break
        self._register_full_pages(rc)

    def abort_pending(self, rc: RequestCache) -> None:
        """Forget an append whose step did not run; the pages stay with the request."""
        rc.pending_tokens = []

    def close(self, rc: RequestCache) -> None:
        """The request ended or is preempted: every page and the slot go back."""
        if rc.closed:
            raise RuntimeError(f"request {rc.req_id!r} closed twice")
        self._release_all(rc)
        rc.closed = True
        self.live.pop(rc.req_id, None)

    def _release_all(self, rc: RequestCache) -> None:
        if self._page_copies:
            # copies into this request's private pages that no step has run yet go with the pages
            own = {(g.index, p) for g in self.paged_groups for p in rc.tables.get(g.index, []) if p >= 0}
            self._page_copies = [c for c in self._page_copies if (c[0], c[2]) not in own]
        for g in self.paged_groups:
            for p in rc.tables.get(g.index, []):
                if p >= 0:
                    g.pool.release(p)
            rc.tables[g.index] = []
            rc.hashes[g.index] = []
        self.slots.release(rc.state_slot)

    # ---- device work the manager asks for ------------------------------------------------
    def take_page_copies(self) -> list[tuple[int, int, int]]:
        copies, self._page_copies = self._page_copies, []
        return copies

    def page_copies_by_group(self) -> dict[int, list[int]]:
        """The pending copy-on-write copies, taken: group -> flat list [src, dst, src, dst, ...].  The step
        function copies the lists to the device with the rest of the step's index data and runs one
        ``ops.copy_pages`` per group before anything of the step writes to the cache."""
        out: dict[int, list[int]] = {}
        for gi, src, dst in self.take_page_copies():
            out.setdefault(gi, []).extend((src, dst))
        return out

    def zero_fresh_state(self, requests: Sequence[RequestCache]) -> None:
        fresh = [rc.state_slot for rc in requests if rc.fresh_state]
        if not fresh:
            return
        for g in self.groups:
            if not g.is_paged:
                g.tensor[:, fresh] = 0

    def check_invariants(self) -> None:
        """No page lost, held twice or freed twice: the pools' counts equal the
        holders the live requests add up to."""
        for g in self.paged_groups:
            held: dict[int, int] = {}
            for rc in self.live.values():
                for p in rc.tables[g.index]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            g.pool.check_invariants(held)
        self.slots.check_invariants()
        slots = [rc.state_slot for rc in self.live.values()]
        assert len(slots) == len(set(slots)), "a state slot is held twice"

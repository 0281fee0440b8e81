"""Host-side bookkeeping of one group's pages: free list, reference counts and
the table of sharable full pages.

It restates what the reference's ``KVCachePool`` does on the host
(src/engine/kvcache.py:81-166: chained 64-bit block hashes, longest-prefix
match, retain/release with checks, LIFO free list that hands out page 0
first) and repairs what that one leaves open: a page's hash entry is dropped
when the page is handed out again (the reference's ``block_id2hash`` is never
filled, kvcache.py:45, 163-165), a page becomes sharable only once its last
slot is written, and a freed page that carries a hash stays findable until it
is really reused.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from typing import Optional, Sequence


class OutOfPages(RuntimeError):
    """No free page is left in a group (the reference raises RuntimeError
    "No free KV cache blocks available", src/engine/kvcache.py:150-151)."""


def hash_block(parent_hash: int, block_tokens: Sequence[int]) -> int:
    """blake2b-64 over the parent hash and the tokens, 8 bytes little-endian
    each (src/engine/kvcache.py:81-86); the first block's parent is 0."""
    h = hashlib.blake2b(digest_size=8)
    h.update(int(parent_hash).to_bytes(8, "little", signed=False))
    for token in block_tokens:
        h.update(int(token).to_bytes(8, "little", signed=True))
    return int.from_bytes(h.digest(), "little", signed=False)


class PagePool:
    def __init__(self, num_pages: int, page_size: int, enable_prefix_cache: bool = True):
        if num_pages < 1 or page_size < 1:
            raise ValueError("num_pages and page_size must be positive")
        self.num_pages = num_pages
        self.page_size = page_size
        self.enable_prefix_cache = enable_prefix_cache
        self.reset()

    def reset(self) -> None:
        self.refcounts = [0] * self.num_pages
        # popped from the end: page 0 is handed out first (kvcache.py:67, 152)
        self._free: list[int] = list(range(self.num_pages - 1, -1, -1))
        # freed pages that still carry a hash, oldest first; reused only after _free is empty
        self._cached_free: "OrderedDict[int, None]" = OrderedDict()
        self._page_of_hash: dict[int, int] = {}
        self._hash_of_page: dict[int, int] = {}
        self._tokens_of_page: dict[int, tuple[int, ...]] = {}

    # ---- counting ---------------------------------------------------------------------
    @property
    def num_free(self) -> int:
        """Pages that an allocation may take (never used, freed, or freed-but-findable)."""
        return len(self._free) + len(self._cached_free)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    def _check_id(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise ValueError(f"invalid page id {page}")

    # ---- allocate / retain / release ----------------------------------------------------
    def allocate(self) -> int:
        if self._free:
            page = self._free.pop()
        elif self._cached_free:
            page, _ = self._cached_free.popitem(last=False)
            self._forget_hash(page)
        else:
            raise OutOfPages("no free KV cache pages available")
        assert self.refcounts[page] == 0
        self.refcounts[page] = 1
        return page

    def retain(self, page: int) -> None:
        """One more holder of a page.  A findable freed page comes back to life."""
        self._check_id(page)
        if self.refcounts[page] == 0:
            if page not in self._cached_free:
                raise RuntimeError(f"cannot retain page {page}: it is free")
            del self._cached_free[page]
        self.refcounts[page] += 1

    def release(self, page: int) -> None:
        self._check_id(page)
        if self.refcounts[page] <= 0:
            raise RuntimeError(f"cannot release page {page} with refcount {self.refcounts[page]}")
        self.refcounts[page] -= 1
        if self.refcounts[page] == 0:
            if page in self._hash_of_page:
                self._cached_free[page] = None
            else:
                self._free.append(page)

    def _forget_hash(self, page: int) -> None:
        h = self._hash_of_page.pop(page, None)
        if h is not None and self._page_of_hash.get(h) == page:
            del self._page_of_hash[h]
        self._tokens_of_page.pop(page, None)

    # ---- sharing ----------------------------------------------------------------------
    def register_full_page(self, page: int, parent_hash: int, tokens: Sequence[int]) -> int:
        """Make a page whose every slot is written findable; returns its hash.

        If another page already answers to the same hash, that one stays the
        sharable copy and this page stays private."""
        self._check_id(page)
        if len(tokens) != self.page_size:
            raise ValueError("only full pages are sharable")
        h = hash_block(parent_hash, tokens)
        if not self.enable_prefix_cache:
            return h
        if self.refcounts[page] <= 0:
            raise RuntimeError(f"cannot register free page {page}")
        if h not in self._page_of_hash and page not in self._hash_of_page:
            self._page_of_hash[h] = page
            self._hash_of_page[page] = h
            self._tokens_of_page[page] = tuple(int(t) for t in tokens)
        return h

    def match_prefix(self, tokens: Sequence[int], max_pages: Optional[int] = None) -> tuple[list[int], list[int]]:
        """The longest run of leading full pages of ``tokens`` that are findable:
        (page ids, their hashes).  Hash and tokens must both be equal
        (src/engine/kvcache.py:104-125).  Nothing is retained."""
        pages: list[int] = []
        hashes: list[int] = []
        if not self.enable_prefix_cache:
            return pages, hashes
        n_full = len(tokens) // self.page_size
        if max_pages is not None:
            n_full = min(n_full, max_pages)
        parent = 0
        for b in range(n_full):
            chunk = tuple(int(t) for t in tokens[b * self.page_size:(b + 1) * self.page_size])
            h = hash_block(parent, chunk)
            page = self._page_of_hash.get(h)
            if page is None or self._tokens_of_page.get(page) != chunk:
                break
            pages.append(page)
            hashes.append(h)
            parent = h
        return pages, hashes

    def find_page(self, block_hash: int, block_tokens: Sequence[int]) -> Optional[int]:
        """The findable page that answers to a block's chained hash and holds exactly its tokens, or None.
        Nothing is retained."""
        if not self.enable_prefix_cache:
            return None
        page = self._page_of_hash.get(block_hash)
        if page is None or self._tokens_of_page.get(page) != tuple(int(t) for t in block_tokens):
            return None
        return page

    # ---- checks for tests ---------------------------------------------------------------
    def check_invariants(self, held: Optional[dict[int, int]] = None) -> None:
        """Every page is in exactly one place; with ``held`` (page -> holders as
        the caller counts them) the reference counts must agree."""
        free = list(self._free) + list(self._cached_free)
        assert len(free) == len(set(free)), "a page is in the free lists twice"
        for p in range(self.num_pages):
            in_free = p in self._cached_free or p in self._free
            assert (self.refcounts[p] == 0) == in_free, f"page {p}: refcount/free mismatch"
            assert self.refcounts[p] >= 0
        for p in self._cached_free:
            assert p in self._hash_of_page
        for h, p in self._page_of_hash.items():
            assert self._hash_of_page.get(p) == h
        if held is not None:
            for p in range(self.num_pages):
                assert self.refcounts[p] == held.get(p, 0), \
                    f"page {p}: refcount {self.refcounts[p]} but {held.get(p, 0)} holders"

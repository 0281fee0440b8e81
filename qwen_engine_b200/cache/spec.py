"""What a mixer asks of the cache: the description a cache slot is built from."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every token, in pages.

    ``window`` = None keeps every key; a number keeps only the last ``window``
    keys of a request alive: pages that every later query has passed are given
    back while the request still runs.
    """

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    @property
    def kind(self) -> str:
        return "paged_kv"


@dataclass(frozen=True)
class FixedStateSpec:
    """State of fixed size per request (a recurrent mixer's, for instance).

    ``shape`` is the state of ONE request in ONE layer; it lives in the slot
    the request holds from admission to its end and starts as zeros.
    """

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    @property
    def kind(self) -> str:
        return "fixed_state"


CacheSpec = PagedKVSpec | FixedStateSpec

"""A request's record on the host (reference src/engine/sequence.py:12-80)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Optional

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    """The reference has WAITING, PREFILLED, DECODING, FINISHED (sequence.py:5-9); here a
    request that is in the cache is RUNNING whether it is still reading its prompt or decoding,
    because one step may do either."""

    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class Sequence:
    seq_id: int
    prompt_token_ids: list[int]
    sampling: SamplingParams
    prompt_text: Optional[str] = None
    output_token_ids: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    finish_reason: Optional[str] = None
    cache: Optional[RequestCache] = None
    admit_order: int = -1            # larger: admitted later (the first to be preempted)
    num_preemptions: int = 0
    shared_prefix_len: int = 0       # tokens found in the cache at the last admission
    hold: bool = False               # not to be scheduled: its last token is on its way and it ends with it

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def output_len(self) -> int:
        return len(self.output_token_ids)

    @property
    def total_len(self) -> int:
        return self.prompt_len + self.output_len

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_computed_tokens(self) -> int:
        """Tokens whose keys and values are in the cache (sequence.py:29-30 keeps two counters
        that are always equal)."""
        return self.cache.num_tokens if self.cache is not None else 0

    @property
    def num_remaining_tokens(self) -> int:
        """Known tokens not yet run: the rest of the prompt, or the one newest sampled token."""
        return self.total_len - self.num_computed_tokens

    @property
    def last_token_id(self) -> int:
        return self.output_token_ids[-1] if self.output_token_ids else self.prompt_token_ids[-1]

    def get_tokens(self, start: int, total: int) -> list[int]:
        """Tokens [start, start + total) of prompt followed by outputs (sequence.py:40-56)."""
        return self.all_token_ids[start:start + total]

"""The scheduler: which requests run in the next step, and with how many tokens.

The reference's loop prefills every waiting request whole, then decodes one
token for up to ``max_num_seqs`` requests, never both in one batch, admits
without looking at free pages, frees pages only when the loop ends and dies
when pages run out (src/engine/llm_engine.py:101-152,
src/engine/kvcache.py:150-151).  Here each step is one mixed batch under a
token budget:

1. every running request that is decoding gets its one token;
2. running requests that still read their prompt get a portion of it;
3. waiting requests are admitted in arrival order (never skipping ahead) while
   a request slot, budget and pages for the first portion are there.

When a running request cannot get the pages it needs, the request admitted
last is preempted: its pages and slot go back, it keeps its tokens, and it
waits at the head of the queue to be recomputed (shared pages make that
cheap).  A request that is alone and still cannot fit is an error.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..cache.manager import UNKNOWN_TOKEN, CacheManager
from ..cache.page_pool import OutOfPages
from ..cache.state_slots import OutOfSlots
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledSeq:
    seq: Sequence
    start: int            # position of the first token run in this step
    num_tokens: int
    wants_logits: bool    # the portion ends at the request's last known token


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSeq] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    admitted: list[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 prefill_chunk_size: Optional[int], max_model_len: int, eos_token_id=None):
        """``eos_token_id``: one id, several (any of them ends a request), or None."""
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.prefill_chunk_size = prefill_chunk_size or max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos_token_ids = frozenset(
            () if eos_token_id is None else ([int(eos_token_id)] if isinstance(eos_token_id, int) else map(int, eos_token_id)))
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.finished: list[Sequence] = []
        self._admit_counter = 0
        self.num_preemptions = 0
        self.prefix_hit_tokens = 0

    # ---- intake -------------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        if seq.prompt_len < 1:
            raise ValueError("a request needs at least one prompt token")
        if seq.prompt_len >= self.max_model_len:
            raise ValueError(f"prompt of {seq.prompt_len} tokens leaves no room under max_model_len = {self.max_model_len}")
        pages_for_one = self.cache.pages_needed_for_new(self.max_model_len)
        for g in self.cache.paged_groups:
            if pages_for_one[g.index] > g.pool.num_pages:
                raise ValueError(
                    f"the cache has {g.pool.num_pages} pages of {self.cache.page_size} tokens; one request of "
                    f"max_model_len = {self.max_model_len} tokens needs {pages_for_one[g.index]}")
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one decision ---------------------------------------------------------------------
    def schedule(self, may_preempt: bool = True) -> SchedulerOutput:
        """``may_preempt`` False (a step launched while the one before it is still in flight): a running
        request that finds no pages is left out of the step instead of making room by preemption."""
        out = SchedulerOutput()
        budget = self.max_num_batched_tokens
        reserved: dict[int, int] = {g.index: 0 for g in self.cache.paged_groups}

        def reserve(seq: Sequence, n: int) -> bool:
            need = self.cache.pages_needed(seq.cache, n)
            if not all(need[g] + reserved[g] <= self.cache.groups[g].pool.num_free for g in need):
                return False
            for g in need:
                reserved[g] += need[g]
            return True

        # decoding requests first, then unfinished prompts, both in admission order
        order = sorted(self.running, key=lambda s: (s.num_remaining_tokens != 1, s.admit_order))
        for seq in order:
            if seq.status is not SequenceStatus.RUNNING:
                continue                                  # preempted a moment ago
            if seq.hold or seq.num_remaining_tokens <= 0:
                continue                                  # nothing to run until its token is known
            if budget <= 0:
                break
            n = min(seq.num_remaining_tokens, self.prefill_chunk_size, budget)
            fits = reserve(seq, n)
            while not fits and may_preempt:
                victim = self._preempt_newest(out, reserved)
                if victim is seq:
                    break
                fits = reserve(seq, n)
            if not fits or seq.status is not SequenceStatus.RUNNING:
                continue
            out.scheduled.append(ScheduledSeq(seq, seq.num_computed_tokens, n,
                                              n == seq.num_remaining_tokens))
            budget -= n

        # admissions, strictly in arrival order; not in a step that had to preempt
        while self.waiting and not out.preempted and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            try:
                rc = self.cache.open(seq.seq_id, known_tokens=seq.all_token_ids)
            except (OutOfSlots, OutOfPages):              # OutOfPages: no page for the private copy
                break
            seq.cache = rc
            n = min(seq.num_remaining_tokens, self.prefill_chunk_size, budget)
            if not reserve(seq, n):
                self.cache.close(rc)
                seq.cache = None
                if not self.running:
                    raise RuntimeError(
                        f"request {seq.seq_id} cannot get pages for its first {n} tokens although nothing else runs")
                break
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            seq.admit_order = self._admit_counter
            self._admit_counter += 1
            seq.shared_prefix_len = rc.shared_tokens
            self.prefix_hit_tokens += rc.shared_tokens
            self.running.append(seq)
            out.admitted.append(seq)
            out.scheduled.append(ScheduledSeq(seq, seq.num_computed_tokens, n,
                                              n == seq.num_remaining_tokens))
            budget -= n
        return out

    def _preempt_newest(self, out: SchedulerOutput, reserved: dict[int, int]) -> Sequence:
        live = [s for s in self.running if s.status is SequenceStatus.RUNNING]
        if len(live) <= 1:
            raise RuntimeError("out of cache pages with a single running request: the cache is too "
                               "small for max_model_len")
        victim = max(live, key=lambda s: s.admit_order)
        # a victim that was already given tokens in this step loses them and its reservation
        for i, sch in enumerate(out.scheduled):
            if sch.seq is victim:
                need = self.cache.pages_needed(victim.cache, sch.num_tokens)
                for g in need:
                    reserved[g] -= need[g]
                del out.scheduled[i]
                break
        self.cache.close(victim.cache)
        victim.cache = None
        victim.status = SequenceStatus.WAITING
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        out.preempted.append(victim)
        return victim

    # ---- after the step -------------------------------------------------------------------
    def finish_reason_for(self, seq: Sequence) -> Optional[str]:
        """The reference stops on the count of new tokens alone and calls that "eos"
        (src/engine/llm_engine.py:36-42); here: "length" for the count or the model's length
        limit, "stop" for an end-of-sequence or stop token."""
        last = seq.output_token_ids[-1]
        sp = seq.sampling
        if not sp.ignore_eos and last in self.eos_token_ids:
            return "stop"
        if last in sp.stop_token_ids:
            return "stop"
        if seq.output_len >= sp.max_new_tokens:
            return "length"
        if seq.total_len >= self.max_model_len:
            return "length"
        return None

    def ends_by_length_after(self, seq: Sequence, more: int) -> bool:
        """Whether the request ends by a count once it has ``more`` more output tokens, whatever they are."""
        return (seq.output_len + more >= seq.sampling.max_new_tokens
                or seq.total_len + more >= self.max_model_len)

    def update(self, out: SchedulerOutput, new_tokens: dict[int, int],
               placed: Optional[dict[int, int]] = None) -> list[Sequence]:
        """Take in the step's sampled tokens (seq_id -> token); returns the requests that ended.
        Their pages and slots go back at once.

        ``placed`` (seq_id -> index in its output tokens): requests whose token of this step already
        has a place, holding ``UNKNOWN_TOKEN``, because a step was launched ahead with it; the token
        goes there (and into the cache's record of the request) instead of being appended.  A
        request that ended while a step launched ahead still carried it is passed over."""
        ended = []
        for sch in out.scheduled:
            seq = sch.seq
            if not sch.wants_logits or seq.status is SequenceStatus.FINISHED:
                continue
            token = int(new_tokens[seq.seq_id])
            if placed is not None and seq.seq_id in placed:
                idx = placed[seq.seq_id]
                if seq.output_token_ids[idx] != UNKNOWN_TOKEN or idx != seq.output_len - 1:
                    raise RuntimeError(f"request {seq.seq_id}: no place is waiting for its token")
                seq.output_token_ids[idx] = token
                if seq.cache is not None and seq.cache.num_tokens > seq.prompt_len + idx:
                    self.cache.resolve_token(seq.cache, seq.prompt_len + idx, token)
            else:
                seq.output_token_ids.append(token)
            seq.hold = False
            reason = self.finish_reason_for(seq)
            if reason is not None:
                seq.finish_reason = reason
                seq.status = SequenceStatus.FINISHED
                self.cache.close(seq.cache)
                seq.cache = None
                self.running.remove(seq)
                self.finished.append(seq)
                ended.append(seq)
        return ended

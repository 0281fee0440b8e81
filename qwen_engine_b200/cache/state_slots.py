"""Slots for per-request state of fixed size.

A live request holds one slot from admission until it ends or is preempted.
Mixers that keep state of fixed size (none in Qwen3) index their state tensors
by the slot id; the step batch carries the ids as ``slot_ids[R]``.
"""
from __future__ import annotations


class OutOfSlots(RuntimeError):
    pass


class StateSlotPool:
    def __init__(self, num_slots: int):
        if num_slots < 1:
            raise ValueError("num_slots must be positive")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfSlots("no free state slot")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise RuntimeError(f"state slot {slot} is not held")
        self._held.remove(slot)
        self._free.append(slot)

    def check_invariants(self) -> None:
        assert len(self._free) == len(set(self._free))
        assert not (set(self._free) & self._held)
        assert len(self._free) + len(self._held) == self.num_slots
